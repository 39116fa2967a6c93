"""Where the files of one benchmark run live and what they are called (reference: benchmark/plotter/namer.py).

A run is identified by its arrival rate, node count, DP / EP degrees and layer-scheduler settings; all of its CSVs,
traces and plots go under ``reports/<those settings>/`` (``DMOE_REPORTS_DIR`` replaces ``reports``)."""
import os
from argparse import ArgumentParser


def add_args(parser: ArgumentParser) -> ArgumentParser:
    parser.add_argument("path", type=str, help="directory of one benchmark run (as returned by get_dir_path)")
    return parser


def reports_root() -> str:
    return os.environ.get("DMOE_REPORTS_DIR", "reports")


def get_dir_path(args, root: str = None) -> str:
    d = os.path.join(root or reports_root(), f"rate={args.rate}-nodes={args.num_nodes}-dp={args.dp_size}-ep={args.ep_size}-"
                           f"layersch={args.layer_scheduler_type}-layerstep={args.layer_scheduler_step}")
    os.makedirs(d, exist_ok=True)
    return d


def _in_dir(name):
    return lambda args, root=None: os.path.join(get_dir_path(args, root), name)


get_sampler_step_name = _in_dir("sampler_step.csv")
get_ttft_name = _in_dir("ttft.csv")
get_req_finish_time_name = _in_dir("req_finish_time.csv")
get_trace_name = _in_dir("trace.json.gz")
get_queue_length_name = _in_dir("queue_length.pkl")
get_trace_metrics_name = _in_dir("trace_metrics.json")


def get_worker_queueing_delay_name(args, worker, root: str = None) -> str:
    return os.path.join(get_dir_path(args, root), f"{worker}_queueing_delay.csv")


def get_plot_dir(data_dir_path: str) -> str:
    d = os.path.join(data_dir_path, "plots")
    os.makedirs(d, exist_ok=True)
    return d
