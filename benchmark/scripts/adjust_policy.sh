#!/bin/bash
# Switches the layer-scheduling policy of a running benchmark server (reference: benchmark/scripts/adjust_policy.sh).
# usage: adjust_policy.sh [policy] [step]      policy: mbfs | flfs | mbflfs | mbtfs | bin
curl -s -X POST "http://localhost:${PORT:-6699}/set_schedule" -H "Content-Type: application/json" \
  -d "{\"policy\": \"${1:-flfs}\", \"step\": ${2:-32}}"
echo
