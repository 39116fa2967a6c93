"""Requests finished per second over the run, from ``<run dir>/req_finish_time.csv`` (reference:
benchmark/plotter/output_req.py)."""
import os
import sys
from argparse import ArgumentParser

import numpy as np
import pandas as pd

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from benchmark.plotter.common import save_series
from benchmark.plotter.namer import add_args, get_plot_dir


def main(argv=None):
    ap = add_args(ArgumentParser())
    ap.add_argument("--window", type=float, default=2.0, help="seconds per bucket")
    a = ap.parse_args(argv)
    df = pd.read_csv(os.path.join(a.path, "req_finish_time.csv"))
    t = np.sort(df[df.columns[0]].to_numpy(dtype=float))
    n_win = int(t[-1] // a.window) + 1 if len(t) else 0
    rate = np.bincount((t // a.window).astype(int), minlength=n_win) / a.window if n_win else np.zeros(0)
    f = save_series(os.path.join(get_plot_dir(a.path), "output_reqs_over_time.png"),
                    {"requests/s": (np.arange(n_win) * a.window, rate)}, "finished requests per second", "s", "requests/s")
    print(f)
    return f


if __name__ == "__main__":
    main()
