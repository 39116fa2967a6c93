"""Queue-length history of ONE worker as a self-contained HTML page: one cell per (step, layer), shaded by the number
of queued tokens, with the step's start time and the exact count as hover text (reference:
benchmark/plotter/queue_length_interact.py, which opens an interactive matplotlib window; there is no display on a
serving box, so this writes a file that any browser opens)."""
import os
import pickle
import sys
from argparse import ArgumentParser

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from benchmark.plotter.namer import get_plot_dir


def sample_from_mid(ls, steps):
    if len(ls) <= steps:
        return ls
    start = (len(ls) - steps) // 2
    return ls[start:start + steps]


def main(argv=None):
    ap = ArgumentParser()
    ap.add_argument("path", help="run directory or queue_length.pkl")
    ap.add_argument("--worker", type=int, required=True)
    ap.add_argument("--steps", type=int, default=2000)
    a = ap.parse_args(argv)
    pkl = a.path if a.path.endswith(".pkl") else os.path.join(a.path, "queue_length.pkl")
    with open(pkl, "rb") as f:
        data = pickle.load(f)
    hist = sample_from_mid(data[a.worker], a.steps)           # [(start ms, {layer: tokens})]
    layers = sorted({l for _, snap in hist for l in snap})
    peak = max([v for _, snap in hist for v in snap.values()] + [1])
    cw, ch = max(2, min(12, 1600 // max(1, len(hist)))), 14
    cells = []
    for x, (t_ms, snap) in enumerate(hist):
        for y, l in enumerate(layers):
            v = snap.get(l, 0)
            shade = 255 - int(220 * v / peak)
            cells.append(f'<rect x="{x * cw}" y="{y * ch}" width="{cw}" height="{ch}" fill="rgb({shade},{shade},255)">'
                         f'<title>step {x}, t={t_ms:.1f} ms, layer {l}: {v} tokens</title></rect>')
    svg = (f'<svg xmlns="http://www.w3.org/2000/svg" width="{len(hist) * cw}" height="{len(layers) * ch}">'
           + "".join(cells) + "</svg>")
    out = os.path.join(get_plot_dir(os.path.dirname(os.path.abspath(pkl))), f"queue_length_worker{a.worker}.html")
    with open(out, "w") as f:
        f.write(f"<html><body><h3>worker {a.worker}: queued tokens per layer (rows) over {len(hist)} steps; "
                f"peak {peak}</h3>{svg}</body></html>")
    print(out)
    return out


if __name__ == "__main__":
    main()
