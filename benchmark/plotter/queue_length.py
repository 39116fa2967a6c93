"""Heat map of queued tokens per layer over time for every worker, from ``queue_length.pkl`` written by
``benchmark_serving --trace`` (reference: benchmark/plotter/ queue-length heat-maps)."""
import argparse
import os
import pickle
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from benchmark.plotter.common import save_matrix


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("pkl")
    ap.add_argument("--out-dir", default="reports")
    a = ap.parse_args(argv)
    with open(a.pkl, "rb") as f:
        queues = pickle.load(f)
    outs = []
    for pid, hist in queues.items():
        if not hist:
            continue
        n_layers = max(len(s) for _, s in hist)
        m = np.zeros((n_layers, len(hist)))
        for j, (_, snap) in enumerate(hist):
            for l, v in snap.items():
                m[int(l), j] = v
        outs.append(save_matrix(os.path.join(a.out_dir, f"queue_length_worker{pid}.png"), m,
                                f"queued tokens, worker {pid}", "engine step", "local layer"))
    print("\n".join(outs))
    return outs


if __name__ == "__main__":
    main()
