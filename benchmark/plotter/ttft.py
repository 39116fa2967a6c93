"""CDF of the time to first token, from ``<run dir>/ttft.csv`` (reference: benchmark/plotter/ttft.py)."""
import os
import sys
from argparse import ArgumentParser

import pandas as pd

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from benchmark.plotter.common import save_series
from benchmark.plotter.latency_cdf import cdf
from benchmark.plotter.namer import add_args, get_plot_dir


def main(argv=None):
    a = add_args(ArgumentParser()).parse_args(argv)
    df = pd.read_csv(os.path.join(a.path, "ttft.csv"))
    col = "ttft_ms" if "ttft_ms" in df.columns else df.columns[-1]
    f = save_series(os.path.join(get_plot_dir(a.path), "ttft_cdf.png"), {"ttft": cdf(df[col])}, "time to first token",
                    "ms", "fraction of requests", kind="cdf")
    print(f)
    return f


if __name__ == "__main__":
    main()
