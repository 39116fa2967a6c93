#!/bin/bash
# Poisson serving sweep on one 8-GPU node (workload of the reference's benchmark/scripts/benchmark_poisson.sh):
# Mixtral 32 layers / 8 experts; 2 attention stages x DP 2 + 1 expert stage x EP 4; attention batch <= 256, expert batch
# <= 512; CUDA-graph attention, graph stride 8; rates 10/20/30/40 req/s for 120 s each, output <= 1024.
set -e
cd "$(dirname "$0")/../.."
for rate in 10 20 30 40; do
  python -m benchmark.benchmark_serving -r $rate --duration 120 -o 1024 --min-output-len 100 -i 300 --min-input-len 100 \
    -N 1 -g 8 -K 2 -L 32 -E 8 --dp-size 2 --ep-size 4 --step-attn 2 --step-expert 1 --placement pipeline \
    --max-batch-size-attn 256 --max-batch-size-expert 512 -ca --graph-stride 8 --generator-type poisson \
    -f reports/poisson.csv --analyze-throughput
done
