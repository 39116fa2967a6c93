#!/bin/bash
# Sends one workload description to a running benchmark server and prints the metrics it returns (reference:
# benchmark/scripts/benchmark_instructions.sh). usage: benchmark_instructions.sh [rate] [duration_s]
curl -s -X POST "http://localhost:${PORT:-6699}/run_once" -H "Content-Type: application/json" \
  -d "{\"rate\": ${1:-20}, \"time\": ${2:-60}, \"distribution\": \"poisson\"}"
echo
