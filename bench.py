#!/usr/bin/env python
"""Headline benchmark: decode output tokens/s of Mixtral-8x7B-shaped serving (bf16, random-init weights, synthetic
requests) on N GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

A "step" is one decode iteration: every running sequence gets one new token through all 32 layers (attention on
the attention GPUs, routed experts on the expert GPUs), the LM head and greedy sampling. N = 1 runs the colocated
engine; N = 2/4/8 run N/2 attention GPUs, by default as ONE tensor-parallel group (N = 8: 4 attention GPUs with TP 4 +
4 expert GPUs with 2 experts each; ``--attn-tp 1`` makes them data-parallel replicas instead), + N/2 expert GPUs
(expert parallel) with the fused peer-memory dispatch / combine / all-gather / reduce-scatter kernels. Per-GPU work is
fixed as N grows (weak scaling): ``--batch`` sequences per attention GPU and micro-batch.

``--impl baseline`` runs the reference-style restatement (NCCL + library kernels, benchmark/reference_style.py) on the
same shapes; its recorded numbers (baseline/reference_style_measured.json) are what ``vs_baseline`` divides by.

Timing: CUDA events on the launching stream, max over ranks. ``value`` counts the device time of the steps (input
copy + kernels + result copy); ``e2e`` is the same K steps through the public engine API including the host-side
scheduling / block-table work between steps, the host->device copy of every step's inputs from pinned memory and the
device->host read of the sampled ids. Each step streams ~93 GB of weights, far more than the 126 MB L2, so no cache
flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

METRIC = "decode output tokens/s (device-timed, max over ranks)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    # The unmodified reference cannot be installed on this image: the offline `pip install --no-index
    # --no-build-isolation --target baseline/_ref <reference checkout>` stops at the C++ build (zmq.hpp and the
    # cereal headers are missing: its third_party submodules are empty) and its Python side needs ray and vllm 0.6.2.
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference does not build offline: third_party submodules (cereal, grouped_gemm) are empty, "
                      "zmq.hpp / ray / vllm==0.6.2 are not on the image"}))
    return 0


BASELINE_FILE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "reference_style_measured.json")


def baseline_number(n_gpus: int, model: str):
    """tokens/s of the reference-style baseline (``--impl baseline``) recorded for this GPU count, or None."""
    try:
        with open(BASELINE_FILE) as f:
            return float(json.load(f)[model][str(n_gpus)]["value"])
    except Exception:
        return None


def percentile(xs, q):
    xs = sorted(xs)
    if not xs:
        return None
    i = min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))
    return xs[i]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"],
                    help="ours: this package's engine; baseline: the reference-style restatement with NCCL and library "
                         "kernels (benchmark/reference_style.py); reference: the unmodified reference (unavailable here)")
    ap.add_argument("--batch", type=int, default=256, help="decode sequences per attention GPU")
    ap.add_argument("--ctx-min", type=int, default=192)
    ap.add_argument("--ctx-max", type=int, default=1536)
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (the result is then marked invalid)")
    ap.add_argument("--model", default="mixtral")
    ap.add_argument("--attn-tp", type=int, default=0,
                    help="tensor-parallel degree of the attention GPUs; 0 = all attention GPUs form one TP group (the "
                         "layout of the headline configuration: 4 attention GPUs TP4 + 4 expert GPUs at N = 8); 1 = "
                         "data-parallel attention replicas")
    ap.add_argument("--n-attn", type=int, default=0, help="attention GPUs out of N (default N/2); the rest hold experts")
    ap.add_argument("--micro-batches", type=int, default=2)
    ap.add_argument("--route-skew", type=float, default=0.0,
                    help="Zipf exponent of a synthetic expert-popularity skew added to the router logits (0 = none)")
    ap.add_argument("--no-selfcheck", action="store_true", help="skip the tiny-model correctness run at N >= 2")
    ap.add_argument("--timeline", type=int, default=0,
                    help="N >= 2: after the timed region, run this many eager coupled iterations with a timing event after "
                         "every launch and print one JSON line per rank role with the device time per kernel (waits on "
                         "peers' flags included)")
    ap.add_argument("--serve", action="store_true",
                    help="N >= 2: open-loop serving instead of the fixed decode batch: Poisson arrivals over a rate sweep "
                         "(--rates, --duration seconds each), prompts U[128,1024], outputs U[64,512], real prefill, "
                         "continuous batching; prints output tokens/s with p50 / p99 time per output token per rate")
    ap.add_argument("--rates", default="2,8,16,32")
    ap.add_argument("--duration", type=float, default=60.0)
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.serve:
        from benchmark import serve_fused
        A = args.n_attn or max(1, args.gpus // 2)
        tp = args.attn_tp or A
        argv = ["--model", args.model, "--n-attn", str(A), "--attn-tp", str(tp), "--rates", args.rates, "--duration",
                str(args.duration), "--min-input-len", "128", "-i", "1024", "--min-output-len", "64", "-o", "512",
                "--max-seqs-per-mb", "256", "--max-tokens-per-mb", "2048", "--max-prefill-tokens-per-mb", "1024",
                "--num-blocks", "32768", "--time-limit", str(args.duration * 4 + 120)]
        if args.layers:
            argv += ["-L", str(args.layers)]
        return serve_fused.main(argv)

    import torch
    import torch.distributed as dist
    from disagmoe_b200.config import CacheConfig, get_preset

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local_rank)
    W = max(args.warmup, 3)
    K = args.steps
    cfg = get_preset(args.model)
    if args.layers:
        cfg = cfg.clone(num_layers=args.layers)
    cfg.max_seq_len = max(4096, (args.ctx_max + K + W + args.timeline + 2 + 15) // 16 * 16)
    g = torch.Generator().manual_seed(1234 + rank)
    B = args.batch
    selfcheck = None
    ours = args.impl == "ours"

    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if not ours:
        from benchmark.reference_style import ReferenceStyleDecode
        runner = ReferenceStyleDecode(cfg, world, rank, local_rank, B, args.ctx_min, args.ctx_max, K + W, g)
        par = [runner.parallelism if rank == 0 else None]
        parallelism = par[0]
    elif world > 1:
        from disagmoe_b200.parallel.disagg import DisaggDecodeBench, selfcheck_against_colocated
        A = args.n_attn or world // 2
        tp = args.attn_tp or A
        while A % tp or cfg.num_heads % tp:
            tp -= 1
        if not args.no_selfcheck:
            selfcheck = selfcheck_against_colocated(world, rank, local_rank, A, tp, args.micro_batches)
            if tp > 1 and (selfcheck["kernel_status"] != 0 or selfcheck["rows_within_2pct"] < 0.9 * selfcheck["rows"]):
                # the tensor-parallel layout did not reproduce the colocated logits on this box: measure the
                # data-parallel layout instead and say so, rather than time a wrong computation
                bad = selfcheck
                tp = 1
                selfcheck = selfcheck_against_colocated(world, rank, local_rank, A, tp, args.micro_batches)
                selfcheck["fell_back_from_tp"] = bad
        runner = DisaggDecodeBench(cfg, world, rank, local_rank, B, args.ctx_min, args.ctx_max, K + W + args.timeline, g, tp=tp,
                                   n_attn=A, route_skew=args.route_skew, n_mb=args.micro_batches)
        parallelism = runner.parallelism
    else:
        from disagmoe_b200.frontend.colocated import ColocatedEngine
        from disagmoe_b200.ops import _lib
        ctx = torch.randint(args.ctx_min, args.ctx_max + 1, (B,), generator=g).tolist()
        blocks = sum((c + K + W + 2 + 15) // 16 for c in ctx) + 64
        eng = ColocatedEngine(cfg, CacheConfig(block_size=16), device="cuda", max_batch_size=B, max_prefill_tokens=B,
                              num_blocks=blocks, enable_cuda_graph=True)
        for layer in eng.executor.attn.values():
            layer.set_route_skew(args.route_skew)
        eng.executor.kv_cache.normal_(0, 0.5)      # synthetic KV history (the reference fills its cache with randn too)
        eng.executor.capture([B])
        first = torch.randint(0, cfg.vocab_size, (B,), generator=g).tolist()
        for i in range(B):
            eng.add_synthetic_request(i, ctx[i], first[i], K + W + 1)
        runner = eng
        parallelism = f"colocated1 (attention + {cfg.num_experts} experts on one GPU)" + \
            (f", Zipf({args.route_skew}) expert popularity" if args.route_skew > 0 else "")

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(W):
        runner.step()
    sync_all()
    launches0 = runner.launch_count() if hasattr(runner, "launch_count") else 0
    sampler = ClockSampler(local_rank)
    sampler.start()
    runner.profile_events = True
    runner.event_pairs = []
    sync_all()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    h2d = d2h = 0
    for _ in range(K):
        runner.step()
        h2d += runner.h2d_bytes_last
        d2h += runner.d2h_bytes_last
    t_end.record()
    sync_all()
    clocks = sampler.stop()
    e2e_ms = t_start.elapsed_time(t_end)
    step_ms = [a.elapsed_time(b) for a, b in runner.event_pairs]
    dev_ms = sum(step_ms)
    launches = (runner.launch_count() - launches0) if hasattr(runner, "launch_count") else 0

    tokens_local = runner.tokens_per_step() if hasattr(runner, "tokens_per_step") else B
    kstatus = 0
    if ours:
        from disagmoe_b200.ops import gemm as _gemm
        kstatus = _gemm.check_status(torch.device("cuda", local_rank))   # non-zero: a bounded device wait gave up
    t = torch.tensor([dev_ms, e2e_ms, float(tokens_local), float(launches), float(h2d), float(d2h), float(kstatus)],
                     device="cuda", dtype=torch.float64)
    steps_t = torch.tensor(step_ms, device="cuda", dtype=torch.float64)
    if world > 1:
        mx = t.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = t.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        dist.all_reduce(steps_t, op=dist.ReduceOp.MAX)      # per step: the slowest rank
        dev_ms, e2e_ms, kstatus = float(mx[0]), float(mx[1]), int(mx[6])
        tokens_step, launches, h2d, d2h = float(sm[2]), int(sm[3]), float(sm[4]), float(sm[5])
    else:
        tokens_step = float(tokens_local)
    value = tokens_step * K / (dev_ms / 1e3)
    e2e = tokens_step * K / (e2e_ms / 1e3)
    if rank == 0:
        # a decode step gives every running sequence one token, so the time per output token of a sequence is the step time
        per_step = steps_t.tolist()
        base = baseline_number(world, cfg.name) if ours and not args.layers else None
        mhz, mhz_max = clocks.get("sm_mhz"), clocks.get("sm_max_mhz")
        out = {
            "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": round(dev_ms / K, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(e2e / base, 3) if base else None,
            "dtype": "bf16", "data": "synthetic (random-init weights, random token ids, randn KV history)",
            "impl": args.impl,
            "config": {"model": cfg.name + ("" if not args.layers else f" TRUNCATED to {args.layers} layers (invalid)"),
                       "global_batch": int(tokens_step), "seq_len": f"context uniform[{args.ctx_min},{args.ctx_max}]",
                       "parallelism": parallelism, "kv_block_size": 16,
                       "l2": "no flush: every step streams all expert weights (>> 126 MB L2)"},
            "clocks": clocks,
            "tpot_ms": {"p50": round(percentile(per_step, 0.5), 3), "p99": round(percentile(per_step, 0.99), 3),
                        "max": round(max(per_step), 3), "how": "device time of each decode step, max over ranks"},
            "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / K, 3),
                    "h2d_bytes_per_step": int(h2d / K), "d2h_bytes_per_step": int(d2h / K)},
            "gpu_launches": int(launches),
            "kernel_status": int(kstatus),
        }
        if mhz and mhz_max:
            # the same work at the clock the GPU could not hold: value scaled by median / max SM clock, and the step in
            # millions of SM cycles (a clock-independent figure for compute-bound parts)
            out["clock_normalised"] = {"value_x_mhz_over_max": round(value * mhz / mhz_max, 1),
                                       "mcycles_per_step": round(dev_ms / K * mhz / 1e3, 2)}
        if base:
            out["baseline"] = {"what": "reference-style baseline (ours): bench.py --impl baseline, e2e tokens/s measured "
                                       "on this pool, recorded in baseline/reference_style_measured.json",
                               "value": base, "vs_baseline_is": "e2e.value / baseline value"}
        if selfcheck is not None:
            out["selfcheck"] = selfcheck
        if not ours:
            out["gpu_launches"] = 0
            out["note"] = "library kernels only (cuBLAS, torch._grouped_mm, library attention, NCCL): none of this package's kernels"
            out.pop("kernel_status")
        if kstatus != 0:
            out["invalid"] = "a device-side wait timed out (kernel status %d): results are not valid" % kstatus
        print(json.dumps(out))
    if ours and world > 1 and args.timeline > 0:
        tl = runner.timeline(args.timeline)
        rows = [None] * world if rank == 0 else None
        dist.gather_object({k: (n, round(ms, 3)) for k, (n, ms) in tl.items()}, rows, dst=0)
        if rank == 0:
            A = runner.shape.n_attn
            for name, r in (("attention rank 0", rows[0]), (f"expert rank 0 (global rank {A})", rows[A])):
                tot = sum(ms for _, ms in r.values())
                print(json.dumps({"timeline": name, "iterations": args.timeline, "total_ms": round(tot, 2),
                                  "ms_per_iteration": round(tot / args.timeline, 2),
                                  "kernels": {k: {"launches": n, "ms": ms, "share": round(ms / tot, 3)}
                                              for k, (n, ms) in sorted(r.items(), key=lambda kv: -kv[1][1])}}))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
