"""Shared plotting helper: matplotlib when it is installed, otherwise the plotted series are written as CSV next to
the requested image path (no graphics stack is needed either way: the Agg backend renders to a file)."""
from __future__ import annotations

import csv
import os
from typing import Dict, Sequence


def save_series(path: str, series: Dict[str, Sequence], title: str = "", xlabel: str = "", ylabel: str = "",
                kind: str = "line") -> str:
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        fig, ax = plt.subplots(figsize=(7, 4))
        for name, (xs, ys) in series.items():
            (ax.step if kind == "cdf" else ax.plot)(xs, ys, label=name)
        ax.set_title(title); ax.set_xlabel(xlabel); ax.set_ylabel(ylabel)
        if len(series) > 1:
            ax.legend()
        fig.tight_layout()
        fig.savefig(path)
        plt.close(fig)
        return path
    except ImportError:
        out = os.path.splitext(path)[0] + ".csv"
        with open(out, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["series", xlabel or "x", ylabel or "y"])
            for name, (xs, ys) in series.items():
                for x, y in zip(xs, ys):
                    w.writerow([name, x, y])
        return out


def save_matrix(path: str, matrix, title: str = "", xlabel: str = "", ylabel: str = "") -> str:
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        fig, ax = plt.subplots(figsize=(8, 4))
        im = ax.imshow(matrix, aspect="auto", origin="lower")
        fig.colorbar(im)
        ax.set_title(title); ax.set_xlabel(xlabel); ax.set_ylabel(ylabel)
        fig.tight_layout()
        fig.savefig(path)
        plt.close(fig)
        return path
    except ImportError:
        import numpy as np
        out = os.path.splitext(path)[0] + ".csv"
        np.savetxt(out, np.asarray(matrix), delimiter=",", fmt="%g")
        return out
