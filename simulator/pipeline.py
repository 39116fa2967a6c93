"""Event model of the fused disaggregated decode pipeline: attention GPUs and expert GPUs in lock step over
micro-batches and layers, coupled by the dispatch (attention -> experts) and combine (experts -> attention) flags.

    python simulator/pipeline.py --n-attn 4 --n-expert 4 --experts 8 --layers 32 --micro-batches 2 \
        --attn-us 279 --expert-us-per-expert 125 --hop-us 8

Per layer l and micro-batch m:
  attention GPU a   starts A(a, l, m) when its previous launch is done and, for l > 0, every expert GPU has combined
                    (l - 1, m) back; takes ``attn_us`` (with a per-GPU, per-launch jitter)
  expert GPU x      starts E(x, l, m) when its previous launch is done and every attention GPU has dispatched (l, m);
                    takes ``experts_on_x * expert_us_per_expert`` (weight streaming dominates decode-size expert GEMMs,
                    so the time scales with the experts a GPU holds, not with its tokens)
Flags cost ``hop_us`` each way. The model answers sizing questions (how many attention vs expert GPUs, how many
micro-batches) before a run is spent on them; its inputs are the stand-alone side times that
``benchmark/profile_disagg_sides.py`` measures.

Calibration against the measured Mixtral runs (256 sequences per micro-batch). First build: stand-alone side times
attention 279 us, experts 250 us per launch at 2 experts per GPU, 309 us at 4, 8 us hop: the model gives 18.4 ms at
4 + 4 GPUs and 20.3 ms at 2 + 2, where 22.1 ms and 26.8 ms were measured. Current build: attention 248 us
(data-parallel; 260 us for a TP4 rank), experts 239 us at 2 per GPU (120 us per expert), 281 us at 4 (70 us per expert):
the model gives 16.8 ms and 18.4 ms, measured 19.9 ms (4 + 4, data-parallel attention; 20.9 ms with TP4) and 23.1 ms
(2 + 2). Raising the hop to 50 us moves the model by ~2.5 ms at most, so flag latency alone does not explain the gap:
the coupled sides run slower than they do alone (remote atomics and stores over NVLink inside the sender kernels,
dispatch and combine traffic landing while the GEMMs stream weights, the gate waiting for the slowest sender), and
every step pays a pipeline fill and drain. The model is therefore a lower bound on the step time and a tool for
relative comparisons between layouts.
"""
from __future__ import annotations

import argparse
import random
from typing import Dict, List


def simulate(n_attn: int, n_expert: int, experts: int, layers: int, micro_batches: int, attn_us: float,
             expert_us_per_expert: float, hop_us: float = 8.0, jitter: float = 0.03, head_us: float = 120.0,
             seed: int = 0) -> Dict[str, float]:
    rnd = random.Random(seed)
    per = -(-experts // n_expert)                                   # ceil: contiguous blocks, the last GPU may hold fewer
    held = [max(0, min(per, experts - x * per)) for x in range(n_expert)]
    t_attn = [0.0] * n_attn                                         # time each GPU becomes free
    t_exp = [0.0] * n_expert
    combined: Dict[tuple, float] = {}                               # (l, m) -> time all experts have combined back
    busy_attn = busy_exp = 0.0
    for l in range(layers):
        for m in range(micro_batches):
            dispatched = []
            for a in range(n_attn):
                ready = t_attn[a]
                if l > 0:
                    ready = max(ready, combined[(l - 1, m)] + hop_us)
                dur = attn_us * (1.0 + rnd.uniform(-jitter, jitter))
                t_attn[a] = ready + dur
                busy_attn += dur
                dispatched.append(t_attn[a])
            arrive = max(dispatched) + hop_us
            done = []
            for x in range(n_expert):
                dur = held[x] * expert_us_per_expert * (1.0 + rnd.uniform(-jitter, jitter))
                start = max(t_exp[x], arrive)
                t_exp[x] = start + dur
                busy_exp += dur
                done.append(t_exp[x])
            combined[(l, m)] = max(done)
    end = 0.0
    for m in range(micro_batches):                                  # LM head after the last combine of every micro-batch
        for a in range(n_attn):
            t_attn[a] = max(t_attn[a], combined[(layers - 1, m)] + hop_us) + head_us
            end = max(end, t_attn[a])
    return {"step_ms": end / 1e3, "attention_busy": busy_attn / n_attn / end, "expert_busy": busy_exp / n_expert / end,
            "experts_per_gpu_max": max(held)}


def main(argv=None) -> List[Dict[str, float]]:
    ap = argparse.ArgumentParser()
    ap.add_argument("--n-attn", type=int, default=4)
    ap.add_argument("--n-expert", type=int, default=4)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--micro-batches", type=int, default=2)
    ap.add_argument("--attn-us", type=float, default=279.0, help="attention side of one layer and micro-batch")
    ap.add_argument("--expert-us-per-expert", type=float, default=125.0, help="GEMM-1 + GEMM-2 of one expert")
    ap.add_argument("--hop-us", type=float, default=8.0, help="flag latency per direction")
    ap.add_argument("--jitter", type=float, default=0.03)
    ap.add_argument("--sequences-per-micro-batch", type=int, default=256)
    ap.add_argument("--sweep-splits", type=int, default=0, help="total GPUs: print every attention / expert split")
    a = ap.parse_args(argv)
    rows = []
    splits = [(a.n_attn, a.n_expert)] if not a.sweep_splits else \
        [(k, a.sweep_splits - k) for k in range(1, a.sweep_splits) if a.sweep_splits - k <= a.experts]
    for na, nx in splits:
        r = simulate(na, nx, a.experts, a.layers, a.micro_batches, a.attn_us, a.expert_us_per_expert, a.hop_us, a.jitter)
        r.update(n_attn=na, n_expert=nx,
                 tokens_per_s=na * a.micro_batches * a.sequences_per_micro_batch / (r["step_ms"] / 1e3))
        rows.append(r)
        print(f"{na} attention + {nx} expert GPUs (<= {r['experts_per_gpu_max']} experts each): step {r['step_ms']:.2f} ms, "
              f"{r['tokens_per_s']:.0f} tokens/s, attention busy {r['attention_busy']:.2f}, expert busy {r['expert_busy']:.2f}")
    return rows


if __name__ == "__main__":
    main()
