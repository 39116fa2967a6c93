"""CDF of the per-step queueing delay of every worker (how long the oldest row of an executed batch had waited in the
worker's pool), from the ``<run dir>/<worker>_queueing_delay.csv`` files (reference:
benchmark/plotter/queueing_delay.py)."""
import glob
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
    series = {}
    for f in sorted(glob.glob(os.path.join(a.path, "*_queueing_delay.csv"))):
        df = pd.read_csv(f)
        if len(df):
            series[os.path.basename(f)[:-len("_queueing_delay.csv")]] = cdf(df[df.columns[-1]])
    out = save_series(os.path.join(get_plot_dir(a.path), "queueing_delay_cdf.png"), series, "queueing delay per step",
                      "ms", "fraction of steps", kind="cdf")
    print(out)
    return out


if __name__ == "__main__":
    main()
