#!/bin/bash
# Smoke run (reference: benchmark/scripts/benchmark_serving.sh): 10 requests, input 1, output 100, 4 experts, DP 2 / EP 2,
# top-1, tracing on, one node with 4 GPUs.
set -e
cd "$(dirname "$0")/../.."
python -m benchmark.benchmark_serving -n 10 -r 0 -i 2 --min-input-len 1 -o 101 --min-output-len 100 -N 1 -g 4 -K 1 -E 4 \
  -L 32 --dp-size 2 --ep-size 2 --step-attn 1 --step-expert 1 --placement pipeline --trace -f reports/smoke.csv
