"""CDFs from the CSVs of ``benchmark_serving --analyze-throughput``: time to first token (``ttft.csv``) and the sampler's
token throughput over time (``sampler_step.csv``); also request completion rate (reference: benchmark/plotter/*)."""
import argparse
import os
import sys

import numpy as np
import pandas as pd

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from benchmark.plotter.common import save_series


def cdf(values):
    v = np.sort(np.asarray(values, dtype=float))
    return v, np.arange(1, len(v) + 1) / max(1, len(v))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ttft", default=None)
    ap.add_argument("--sampler", default=None)
    ap.add_argument("--out-dir", default="reports")
    ap.add_argument("--window", type=float, default=1.0, help="seconds per throughput bucket")
    a = ap.parse_args(argv)
    outs = []
    if a.ttft:
        df = pd.read_csv(a.ttft)
        xs, ys = cdf(df["ttft_ms"])
        outs.append(save_series(os.path.join(a.out_dir, "ttft_cdf.png"), {"ttft": (xs, ys)}, "time to first token",
                                "ms", "fraction of requests", kind="cdf"))
    if a.sampler:
        df = pd.read_csv(a.sampler)
        t = df["time_stamp"] - df["time_stamp"].min()
        buckets = (t // a.window).astype(int)
        thr = df.groupby(buckets)["num_tokens"].sum() / a.window
        outs.append(save_series(os.path.join(a.out_dir, "sampler_throughput.png"),
                                {"tokens/s": (thr.index.to_numpy() * a.window, thr.to_numpy())}, "sampler throughput",
                                "s", "tokens/s"))
        done = np.cumsum(df["num_tokens"].to_numpy()) / max(1, df["num_tokens"].sum())
        outs.append(save_series(os.path.join(a.out_dir, "completion_rate.png"), {"completed": (t.to_numpy(), done)},
                                "token completion", "s", "fraction"))
    print("\n".join(outs))
    return outs


if __name__ == "__main__":
    main()
