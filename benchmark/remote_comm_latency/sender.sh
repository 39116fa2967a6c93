#!/usr/bin/env bash
# usage: sender.sh <sender-host> <recver-host> [transport]
python "$(dirname "$0")/sender.py" --sender-host "${1:-127.0.0.1}" --recver-host "${2:-127.0.0.1}" --transport "${3:-socket}"
