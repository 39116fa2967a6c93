#!/bin/bash
# Placement sweep (reference: benchmark/scripts/benchmark_placement_search.sh), scaled to one 8-GPU node: 4 attention +
# 4 expert GPUs, every power-of-two split of (stages, DP) and (stages, EP); 6000 requests, output 128.
set -e
cd "$(dirname "$0")/../.."
for sa in 1 2 4; do for se in 1 2 4; do
  dp=$((4 / sa)); ep=$((4 / se))
  python -m benchmark.benchmark_serving -n 6000 -r 0 -o 129 --min-output-len 128 -N 1 -g 8 -K 2 -L 32 -E 8 \
    --dp-size $dp --ep-size $ep --step-attn $sa --step-expert $se --placement pipeline -f reports/placement_search.csv
done; done
