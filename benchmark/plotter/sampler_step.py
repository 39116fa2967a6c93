"""Sampler output over the run: tokens per ``--gap-i`` sampler steps and tokens per second in ``--gap-t`` second
windows, from ``<run dir>/sampler_step.csv`` (reference: benchmark/plotter/sampler_step.py). Prints the peak."""
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
    ap.add_argument("--gap-i", type=int, default=1)
    ap.add_argument("--gap-t", type=float, default=5.0)
    a = ap.parse_args(argv)
    df = pd.read_csv(os.path.join(a.path, "sampler_step.csv"))
    out = get_plot_dir(a.path)
    tok = df["num_tokens"].to_numpy()
    per_i = np.add.reduceat(tok, np.arange(0, len(tok), a.gap_i)) if len(tok) else tok
    files = [save_series(os.path.join(out, "output_tokens_over_index.png"),
                         {"tokens": (np.arange(len(per_i)) * a.gap_i, per_i)}, "sampler output", "step",
                         f"tokens per {a.gap_i} step(s)")]
    t = df["time_stamp"].to_numpy(dtype=float)
    t = t - t[0] if len(t) else t
    n_win = int(t[-1] // a.gap_t) + 1 if len(t) else 0
    per_t = np.bincount((t // a.gap_t).astype(int), weights=tok, minlength=n_win) / a.gap_t if n_win else np.zeros(0)
    print(f"peak throughput: {per_t.max() if len(per_t) else 0.0:.1f} tokens/s")
    files.append(save_series(os.path.join(out, "output_tokens_over_time.png"),
                             {"tokens/s": (np.arange(n_win) * a.gap_t, per_t)}, "sampler output", "s", "tokens/s"))
    print("\n".join(files))
    return files


if __name__ == "__main__":
    main()
