"""Eager (no CUDA graph) decode steps of the colocated engine, for per-kernel profiling.

    python benchmark/profile_decode_step.py --layers 32 --steps 3          # launch list: 9 * layers + 4 launches per step
    python benchmark/profile_decode_step.py --layers 2 --steps 3           # small case for `ncu --set full -k regex:...`

Prints the mean device time per step (CUDA events). Sequences get a random-valued KV history of the requested
context length; token ids are random so that routing spreads over all experts.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from disagmoe_b200.config import CacheConfig, get_preset
from disagmoe_b200.frontend.colocated import ColocatedEngine


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral")
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx-min", type=int, default=192)
    ap.add_argument("--ctx-max", type=int, default=1536)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--graph", action="store_true", help="replay the captured CUDA graph instead of eager launches")
    args = ap.parse_args()
    cfg = get_preset(args.model).clone(num_layers=args.layers)
    g = torch.Generator().manual_seed(0)
    B = args.batch
    ctx = torch.randint(args.ctx_min, args.ctx_max + 1, (B,), generator=g).tolist()
    blocks = sum((c + args.steps + 18) // 16 for c in ctx) + 64
    eng = ColocatedEngine(cfg, CacheConfig(block_size=16), device="cuda", max_batch_size=B, max_prefill_tokens=B,
                          num_blocks=blocks, enable_cuda_graph=args.graph)
    eng.executor.kv_cache.normal_(0, 0.5)
    if args.graph:
        eng.executor.capture([B])
    first = torch.randint(0, cfg.vocab_size, (B,), generator=g).tolist()
    for i in range(B):
        eng.add_synthetic_request(i, ctx[i], first[i], args.steps + 1)
    eng.profile_events = True
    for _ in range(args.steps):
        eng.step()
    torch.cuda.synchronize()
    ms = [a.elapsed_time(b) for a, b in eng.event_pairs]
    ms = [round(x, 2) for x in ms]
    print(f"layers={args.layers} batch={B} steps={args.steps} graph={args.graph} ms/step={ms} launches/step={9 * args.layers + 4}")


if __name__ == "__main__":
    main()
