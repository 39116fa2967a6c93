#!/bin/bash
# Layer-scheduler sweep (reference: benchmark/scripts/benchmark_layer_scheduler.sh): policies mbfs / flfs / mbflfs with
# block steps 1..32 through the HTTP server (start `python -m benchmark.server ... --port 6699` first).
set -e
URL=${URL:-http://127.0.0.1:6699}
for policy in mbfs flfs; do
  curl -s -X POST $URL/set_schedule -H 'content-type: application/json' -d "{\"policy\": \"$policy\"}"
  curl -s -X POST $URL/run_once -H 'content-type: application/json' -d '{"rate": 20, "time": 60, "distribution": "poisson"}'; echo
done
for step in 1 2 4 8 16 32; do
  curl -s -X POST $URL/set_schedule -H 'content-type: application/json' -d "{\"policy\": \"mbflfs\", \"step\": $step}"
  curl -s -X POST $URL/run_once -H 'content-type: application/json' -d '{"rate": 30, "time": 60, "distribution": "poisson"}'; echo
done
