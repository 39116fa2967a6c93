#!/bin/bash
# Long-running benchmark server (reference: benchmark/scripts/launch_server.sh): one node with 4 GPUs, 2 attention
# replicas + 2 expert GPUs, 32 layers, 4 experts top-1. POST /run_once runs a workload, POST /set_schedule switches the
# layer-scheduling policy while it is up (benchmark/scripts/adjust_policy.sh).
set -e
cd "$(dirname "$0")/../.."
mkdir -p reports
python -m benchmark.server --min-input-len 100 -i 300 --min-output-len 100 -o 500 -N 1 -g 4 -K 1 -u 0.65 \
  -L 32 -E 4 --max-batch-size-attn 160 --max-batch-size-expert 512 --graph-stride 8 --step-attn 1 --dp-size 2 \
  --step-expert 1 --ep-size 2 --placement pipeline -ca -f reports/benchmark.csv --port "${PORT:-6699}" "$@"
