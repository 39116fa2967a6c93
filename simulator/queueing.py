"""Discrete-event model of layer scheduling on one worker (reference: simulator/queueing.py:1-136).

Tokens arrive as a Poisson stream at layer 0; every scheduling step takes a fixed ``step_ms`` and serves the whole
queue of one layer, whose tokens then move to the next layer (tokens leaving the last layer re-enter layer 0 as the
next decode token until their request is done). Policies: ``largest`` (most queued tokens), ``fcfs`` (layer whose head
token waited longest), ``first`` (lowest non-empty layer). Prints inter-token latency statistics.
"""
from __future__ import annotations

import argparse
from collections import deque

import numpy as np


def simulate(rate: float, n_layers: int, step_ms: float, duration_s: float, policy: str, out_len: int, seed: int = 0):
    rng = np.random.default_rng(seed)
    arrivals = np.cumsum(rng.exponential(1.0 / rate, int(rate * duration_s)))
    queues = [deque() for _ in range(n_layers)]      # entries: (request id, time the token entered this queue)
    remaining, last_emit, itl = {}, {}, []
    t, nxt, served_steps = 0.0, 0, 0
    step = step_ms / 1e3
    while nxt < len(arrivals) or any(queues):
        while nxt < len(arrivals) and arrivals[nxt] <= t:
            queues[0].append((nxt, arrivals[nxt]))
            remaining[nxt] = out_len
            nxt += 1
        cand = [i for i in range(n_layers) if queues[i]]
        if not cand:
            t = arrivals[nxt] if nxt < len(arrivals) else t + step
            continue
        if policy == "largest":
            l = max(cand, key=lambda i: len(queues[i]))
        elif policy == "fcfs":
            l = min(cand, key=lambda i: queues[i][0][1])
        else:
            l = cand[0]
        batch = list(queues[l])
        queues[l].clear()
        t += step
        served_steps += 1
        for rid, _ in batch:
            if l + 1 < n_layers:
                queues[l + 1].append((rid, t))
                continue
            if rid in last_emit:
                itl.append(t - last_emit[rid])
            last_emit[rid] = t
            remaining[rid] -= 1
            if remaining[rid] > 0:
                queues[0].append((rid, t))
    itl = np.asarray(itl) * 1e3 if itl else np.zeros(1)
    return {"steps": served_steps, "itl_mean_ms": float(itl.mean()), "itl_p50_ms": float(np.median(itl)),
            "itl_p99_ms": float(np.percentile(itl, 99)), "makespan_s": t}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rate", type=float, default=20)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--step-ms", type=float, default=3.0)
    ap.add_argument("--duration", type=float, default=10)
    ap.add_argument("--output-len", type=int, default=32)
    ap.add_argument("--policy", default="largest", choices=["largest", "fcfs", "first"])
    a = ap.parse_args()
    print(simulate(a.rate, a.layers, a.step_ms, a.duration, a.policy, a.output_len))


if __name__ == "__main__":
    main()
