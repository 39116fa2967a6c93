"""Open-loop serving benchmark on the fused disaggregated data plane (one process per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29600 \
        benchmark/serve_fused.py --model mixtral --n-attn 4 --attn-tp 4 -r 16 -n 256 \
        --min-input-len 128 -i 1024 --min-output-len 64 -o 512

Every rank builds the same synthetic workload from the seed (Poisson arrivals, uniform prompt / output lengths,
uniform random token ids) and the same request -> attention group assignment (least outstanding KV demand at arrival,
``assign_requests``), so no request ever travels between processes. Rank 0 gathers the per-request timestamps and prints the same metrics as
``benchmark.benchmark_serving`` (request / token throughput, request latency, inter-token latency and time to first
token: mean / median / p99), the share of iterations that replayed a CUDA graph, and the device status word.
``--check`` replays the same requests through the single-GPU colocated engine on rank 0 afterwards and reports the
fraction of generated tokens that agree (greedy decoding; bf16 reduction orders differ, so near-ties may flip).
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np
import torch
import torch.distributed as dist

from benchmark.benchmark_serving import analyze_results
from benchmark.workload import get_generator
from disagmoe_b200.config import CacheConfig, get_preset
from disagmoe_b200.parallel.serving import FusedServingRank, HostOnlyAttention, host_only_runner


def assign_requests(reqs, groups: int):
    """Request -> attention group, computed identically on every rank from the workload alone: in arrival order, each
    request goes to the group with the least KV demand (prompt + output tokens) still outstanding at its arrival time,
    assuming a request holds its tokens from arrival until ``output length`` inter-token steps later. The same idea as
    the DP admission policy of the host-scheduled path (most free KV blocks first), without any communication."""
    load = [[] for _ in range(groups)]            # per group: (release time estimate, tokens)
    owner = {}
    step = 0.02                                   # nominal seconds per token, only used to age out old requests
    for rid, prompt, n_out, at in sorted(reqs, key=lambda r: (r[3], r[0])):
        cur = [sum(t for rel, t in g if rel > at) for g in load]
        g = min(range(groups), key=lambda i: (cur[i], i))
        owner[rid] = g
        load[g].append((at + n_out * step, len(prompt) + n_out))
    return owner


def write_trace(results, path: str) -> str:
    """Chrome trace: one process per attention rank, one event per iteration carrying the rows of its micro-batches
    and whether it replayed a CUDA graph."""
    import gzip
    events = []
    for r in results:
        for t0, t1, Ts, g in r.get("step_log", []):
            events.append({"name": ("graph %d" % g) if g else "eager", "cat": "iteration", "ph": "X", "ts": t0 * 1e6,
                           "dur": (t1 - t0) * 1e6, "pid": r["rank"], "tid": 0,
                           "args": {"rows_per_micro_batch": list(Ts)}})
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    with gzip.open(path, "wt") as f:
        json.dump(events, f)
    return path


def sweep(args, srv, cfg, groups, tp, rank, world, A):
    """Poisson arrivals at each rate of ``--rates`` for ``--duration`` seconds on one engine (request ids are unique across
    rates); per rate one JSON line: output tokens/s, time per output token p50 / p99 (inter-token latency), TTFT."""
    from dataclasses import asdict
    next_id = 0
    for ri, rate in enumerate(float(r) for r in args.rates.split(",")):
        n = max(4, int(round(rate * args.duration)))
        gen = get_generator("poisson")(rate, 1.0, args.min_input_len, args.max_input_len, args.seed + ri,
                                       args.min_output_len, args.max_output_len)
        wl = gen.generate_num(n)
        rng = np.random.default_rng(args.seed + 100 + ri)
        reqs = []
        for i in range(len(wl)):
            at, n_in = wl[i]
            reqs.append((next_id + i, rng.integers(0, cfg.vocab_size, int(n_in)).tolist(), int(wl.output_lens[i]), float(at)))
        next_id += len(reqs)
        ids = {r[0] for r in reqs}
        owner = assign_requests(reqs, groups)
        mine = [r for r in reqs if srv.is_leader and owner[r[0]] == rank // tp]
        it0, g0 = srv.iterations, srv.graph_iterations
        res = srv.serve(mine, time_limit=args.time_limit)
        gathered = [None] * world if rank == 0 else None
        dist.gather_object(res, gathered, dst=0, group=srv.ctl)
        if rank == 0:
            slo = [s for g in gathered for s in g["slo"] if s.req_id in ids]
            arrivals = {k: v for g in gathered for k, v in g["arrivals"].items() if k in ids}
            m = analyze_results(slo, arrivals, max(g["duration"] for g in gathered))
            line = {"rate_req_s": rate, "requests": len(slo), "output_tokens_per_s": round(m.token_throughput, 1),
                    "tpot_ms": {"p50": round(m.itl_latency_median_ms, 2), "p99": round(m.itl_latency_p99_ms, 2),
                                "mean": round(m.itl_latency_mean_ms, 2)},
                    "ttft_ms": {"mean": round(m.ttft_mean_ms, 1), "p99": round(m.ttft_p99_ms, 1)},
                    "duration_s": round(m.e2e_duration, 2), "iterations": srv.iterations - it0,
                    "graph_iterations": srv.graph_iterations - g0,
                    "kernel_status": max(g["kernel_status"] for g in gathered),
                    "layout": f"{groups} attention group(s) x tp{tp} + {world - A} expert GPUs",
                    "workload": f"poisson, prompts U[{args.min_input_len},{args.max_input_len}], outputs "
                                f"U[{args.min_output_len},{args.max_output_len}], {args.duration:.0f} s of arrivals"}
            print(json.dumps(line), flush=True)
            if args.file:
                with open(args.file, "a") as f:
                    f.write(json.dumps({**line, **asdict(m)}) + "\n")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral")
    ap.add_argument("-L", "--num-layers", type=int, default=0)
    ap.add_argument("--n-attn", type=int, default=0)
    ap.add_argument("--attn-tp", type=int, default=1)
    ap.add_argument("-r", "--rate", type=float, default=8.0, help="requests per second over the whole job; 0 = all at once")
    ap.add_argument("-n", "--num-requests", type=int, default=64)
    ap.add_argument("--min-input-len", type=int, default=128)
    ap.add_argument("-i", "--max-input-len", type=int, default=1024)
    ap.add_argument("--min-output-len", type=int, default=64)
    ap.add_argument("-o", "--max-output-len", type=int, default=512)
    ap.add_argument("--generator-type", default="poisson")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--max-seqs-per-mb", type=int, default=128)
    ap.add_argument("--max-tokens-per-mb", type=int, default=2048)
    ap.add_argument("--max-prefill-tokens-per-mb", type=int, default=0)
    ap.add_argument("--num-blocks", type=int, default=16384)
    ap.add_argument("--route-skew", type=float, default=0.0)
    ap.add_argument("--time-limit", type=float, default=600.0)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--host-only", action="store_true",
                    help="dry run of the host side (scheduling, lock-step protocol, result collection) as CPU processes "
                         "over gloo with a stand-in for the GPU side; --check then verifies the stand-in's tokens")
    ap.add_argument("-f", "--file", default="", help="append the metrics as one JSON line")
    ap.add_argument("--trace", default="", help="write a Chrome trace (json.gz) of every attention rank's iterations")
    ap.add_argument("--rates", default="", help="comma-separated request rates (req/s): runs the workload once per rate on "
                    "the same engine, --duration seconds of arrivals each, and prints one JSON line per rate")
    ap.add_argument("--duration", type=float, default=60.0, help="seconds of arrivals per rate of a --rates sweep")
    args = ap.parse_args(argv)

    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    if os.environ.get("DMOE_SERVE_DEBUG"):
        # where is every rank if the job stops making progress: Python stacks of all threads to stderr, repeatedly
        import faulthandler
        faulthandler.dump_traceback_later(float(os.environ["DMOE_SERVE_DEBUG"]), repeat=True)
    if args.host_only:
        dist.init_process_group("gloo")
    else:
        torch.cuda.set_device(lr)
        dist.init_process_group("nccl", device_id=torch.device("cuda", lr))
    cfg = get_preset(args.model)
    if args.num_layers:
        cfg = cfg.clone(num_layers=args.num_layers)
    cfg = cfg.clone(dtype=torch.bfloat16)
    A = args.n_attn or world // 2
    tp = args.attn_tp
    groups = A // tp

    Gen = get_generator(args.generator_type if args.rate > 0 else "offline")
    gen = Gen(max(args.rate, 1e-9), 1.0, args.min_input_len, args.max_input_len, args.seed, args.min_output_len,
              args.max_output_len)
    wl = gen.generate_num(args.num_requests)
    rng = np.random.default_rng(args.seed + 1)
    reqs = []
    for i in range(len(wl)):
        at, n_in = wl[i]
        n_out = int(wl.output_lens[i]) if len(wl.output_lens) else args.max_output_len
        reqs.append((i, rng.integers(0, cfg.vocab_size, int(n_in)).tolist(), n_out, float(at)))

    srv = FusedServingRank(cfg, world, rank, lr, A, tp, max_seqs_per_mb=args.max_seqs_per_mb,
                           max_tokens_per_mb=args.max_tokens_per_mb, num_blocks=args.num_blocks,
                           route_skew=args.route_skew,
                           max_prefill_tokens_per_mb=args.max_prefill_tokens_per_mb or None,
                           host_only_runner=host_only_runner(cfg.vocab_size) if args.host_only else None)
    if args.rates:
        sweep(args, srv, cfg, groups, tp, rank, world, A)
        dist.destroy_process_group()
        return 0
    owner = assign_requests(reqs, groups)
    mine = [r for r in reqs if srv.is_leader and owner[r[0]] == rank // tp]
    res = srv.serve(mine, time_limit=args.time_limit)
    gathered = [None] * world if rank == 0 else None
    dist.gather_object(res, gathered, dst=0, group=srv.ctl)
    if rank == 0:
        slo = [s for g in gathered for s in g["slo"]]
        arrivals = {k: v for g in gathered for k, v in g["arrivals"].items()}
        duration = max(g["duration"] for g in gathered)
        m = analyze_results(slo, arrivals, duration)
        print(m)
        its = gathered[0]["iterations"]
        extra = {"iterations": its, "graph_iterations": gathered[0]["graph_iterations"],
                 "kernel_status": max(g["kernel_status"] for g in gathered), "requests_finished": len(slo),
                 "layout": f"{groups} attention group(s) x tp{tp} + {world - A} expert GPUs"}
        print(json.dumps(extra))
        if args.trace:
            write_trace(gathered, args.trace)
        if args.check and args.host_only:
            outs = {k: v for g in gathered for k, v in g.get("outputs", {}).items()}
            ok = 0
            for rid, prompt, n_out, _ in reqs:
                tok, pos, want = prompt[-1], len(prompt) - 1, []
                for _ in range(n_out):
                    tok = HostOnlyAttention.next_token(tok, pos, cfg.vocab_size)
                    want.append(tok)
                    pos += 1
                ok += int(outs.get(rid) == want)
            print(json.dumps({"check_requests_exact": ok, "requests": len(reqs)}))
        elif args.check:
            from disagmoe_b200.frontend.colocated import ColocatedEngine
            outs = {k: v for g in gathered for k, v in g.get("outputs", {}).items()}
            del srv
            torch.cuda.empty_cache()
            eng = ColocatedEngine(cfg, CacheConfig(block_size=16), device="cuda", max_batch_size=64,
                                  max_prefill_tokens=2048, num_blocks=4096, enable_cuda_graph=False)
            for r in reqs:
                eng.add_request(r[0], r[1], r[2])
            ref = eng.run_until_done()
            same = sum(int(a == b) for k in ref for a, b in zip(ref[k], outs.get(k, [])))
            first = sum(int(ref[k][0] == outs[k][0]) for k in ref if outs.get(k))
            total = sum(len(v) for v in ref.values())
            print(json.dumps({"check_tokens_agree": round(same / max(total, 1), 4),
                              "check_first_tokens_agree": round(first / max(len(ref), 1), 4)}))
        if args.file:
            from dataclasses import asdict
            with open(args.file, "a") as f:
                f.write(json.dumps({"args": vars(args), **asdict(m), **extra}) + "\n")
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main() or 0)
