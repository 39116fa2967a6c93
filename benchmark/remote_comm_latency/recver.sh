#!/usr/bin/env bash
# usage: recver.sh <sender-host> <recver-host> [transport]   (start this side first)
python "$(dirname "$0")/recver.py" --sender-host "${1:-127.0.0.1}" --recver-host "${2:-127.0.0.1}" --transport "${3:-socket}"
