#!/usr/bin/env bash
# Every plot of every run directory under <benchmark_dir>.
benchmark_dir=$1
if [[ -z "$benchmark_dir" || ! -d "$benchmark_dir" ]]; then
    echo "Usage: $0 <benchmark_dir>"
    exit 1
fi
for working_dir in "$benchmark_dir"/*/; do
    bash "$(dirname "$0")/plot_trace.sh" "${working_dir%/}"
done
