#!/usr/bin/env bash
# Every plot of one run directory (the files benchmark_serving --analyze-throughput --trace leaves there).
working_dir=$1
if [[ -z "$working_dir" || ! -d "$working_dir" ]]; then
    echo "Usage: $0 <working_dir>"
    exit 1
fi
here=$(dirname "$0")
[[ -f "$working_dir/req_finish_time.csv" ]] && python "$here/output_req.py" "$working_dir"
[[ -f "$working_dir/sampler_step.csv" ]] && python "$here/sampler_step.py" --gap-t 5 "$working_dir"
[[ -f "$working_dir/ttft.csv" ]] && python "$here/ttft.py" "$working_dir"
ls "$working_dir"/*_queueing_delay.csv >/dev/null 2>&1 && python "$here/queueing_delay.py" "$working_dir"
[[ -f "$working_dir/queue_length.pkl" ]] && python "$here/queue_length.py" "$working_dir/queue_length.pkl" --out-dir "$working_dir/plots"
exit 0
