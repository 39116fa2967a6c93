"""Open-loop serving benchmark (reference: benchmark/benchmark_serving.py).

    python -m benchmark.benchmark_serving -r 8 -n 200 -i 1024 --min-input-len 128 -o 512 --min-output-len 64 -K 2 \
        --backend colocated --model mixtral
    python -m benchmark.benchmark_serving --device cpu --model tiny -g 2 --ep-size 1 --step-attn 1 -n 16 -r 50 ...

Requests arrive by the chosen generator; every request is a prompt of random token ids and a fixed output length.
Reported: duration, request and output-token throughput, request latency and inter-token latency (TPOT) mean /
median / p99, time to first token; optional CSV row, sampler-throughput and TTFT CSVs, and a Chrome trace of the
engine steps with the per-layer queue snapshot.
"""
from __future__ import annotations

import gzip
import json
import os
import pickle
import sys
import time
from dataclasses import dataclass, asdict
from typing import Dict, List, Optional

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmark.utils import get_parser_base
from benchmark.workload import Workload, get_generator
from disagmoe_b200.config import CacheConfig, SamplingConfig, get_preset
from disagmoe_b200.frontend.datatypes import SloStat
from disagmoe_b200.utils.placement import ClusterConfig, get_model_placement


@dataclass
class BenchmarkMetrics:
    e2e_duration: float = -1
    req_throughput: float = -1
    token_throughput: float = -1
    req_latency_mean_ms: float = -1
    req_latency_median_ms: float = -1
    req_latency_p99_ms: float = -1
    itl_latency_mean_ms: float = -1
    itl_latency_median_ms: float = -1
    itl_latency_p99_ms: float = -1
    ttft_mean_ms: float = -1
    ttft_p99_ms: float = -1

    def __repr__(self):
        return "Metrics:\n" + "\n".join(f"  {k}: {v:.2f}" for k, v in asdict(self).items())

    def write_to_file(self, args) -> None:
        import pandas as pd
        row = {"num_requests": args.num_requests, "rate": args.rate, "DP_size": args.dp_size, "EP_size": args.ep_size,
               "num_experts": args.num_experts, **{k: round(v, 3) for k, v in asdict(self).items()}}
        os.makedirs(os.path.dirname(os.path.abspath(args.file)) or ".", exist_ok=True)
        df = pd.read_csv(args.file) if os.path.exists(args.file) else pd.DataFrame(columns=list(row))
        df.loc[len(df)] = row
        df.to_csv(args.file, index=False)


def analyze_results(results: List[SloStat], arrivals: Dict[int, float], duration: float) -> BenchmarkMetrics:
    """``results`` carry absolute timestamps (seconds); ``arrivals`` maps request id -> submission time."""
    lat, itl, ttft, total = [], [], [], 0
    for r in results:
        total += len(r.t_tokens)
        t0 = arrivals.get(r.req_id, r.t_prefill)
        lat.append(r.t_decode - t0)
        ttft.append(r.t_prefill - t0)
        itl.extend(np.diff(r.t_tokens).tolist())
    if not itl:
        itl = [0.0]
    ms = 1000.0
    return BenchmarkMetrics(
        e2e_duration=duration, req_throughput=len(results) / duration, token_throughput=total / duration,
        req_latency_mean_ms=float(np.mean(lat)) * ms, req_latency_median_ms=float(np.median(lat)) * ms,
        req_latency_p99_ms=float(np.percentile(lat, 99)) * ms,
        itl_latency_mean_ms=float(np.mean(itl)) * ms, itl_latency_median_ms=float(np.median(itl)) * ms,
        itl_latency_p99_ms=float(np.percentile(itl, 99)) * ms,
        ttft_mean_ms=float(np.mean(ttft)) * ms, ttft_p99_ms=float(np.percentile(ttft, 99)) * ms)


def model_config_from_args(args):
    cfg = get_preset(args.model)
    if args.model in ("mixtral", "duo"):
        cfg = cfg.clone(num_layers=args.num_layers, num_experts=args.num_experts, top_k=args.topk)
    return cfg.clone(ep_size=args.ep_size, tp_size=args.tp_size, dp_size=args.dp_size,
                     enable_cuda_graph_attn=args.cuda_graph_attn, enable_grouped_gemm=not args.serial_gemm,
                     graph_stride=args.graph_stride, max_batch_size_attn=args.max_batch_size_attn,
                     max_batch_size_expert=args.max_batch_size_expert, enable_trace=args.trace)


def make_workload(args) -> Workload:
    Gen = get_generator(args.generator_type if args.rate > 0 else "offline")
    gen = Gen(max(args.rate, 1e-9), 1.0, args.min_input_len, args.max_input_len, args.seed, args.min_output_len,
              args.max_output_len)
    return gen.generate_duration(args.duration) if args.duration > 0 else gen.generate_num(args.num_requests)


def parse_worker_addresses(spec: str):
    """'3=10.0.0.2:7700,4=10.0.0.2:7700' -> {3: ('10.0.0.2', 7700), 4: ('10.0.0.2', 7700)}"""
    out = {}
    for item in filter(None, (x.strip() for x in spec.split(","))):
        dev, addr = item.split("=")
        host, port = addr.rsplit(":", 1)
        out[int(dev)] = (host, int(port))
    return out


def launch(args):
    """Builds the placement and the controller, starts every worker (reference: benchmark_serving.py:88-131)."""
    from disagmoe_b200.frontend.controller import init_controller
    cfg = model_config_from_args(args)
    cluster = ClusterConfig(n_node=args.num_nodes, n_gpu=args.num_gpus)
    if args.placement == "pipeline":
        place = get_model_placement(cfg, cluster, "pipeline", args.step_attn, args.step_expert, args.zigzag_attn)
    else:
        place = get_model_placement(cfg, cluster, args.placement)
    master = init_controller(args.num_nodes, args.num_gpus, device=args.device,
                             worker_addresses=parse_worker_addresses(getattr(args, "worker_addresses", "")))
    master.init_engine(place, cfg, CacheConfig(block_size=args.block_size, gpu_memory_utilization=args.gpu_usage,
                                               num_gpu_blocks=args.num_blocks or 4096),
                       SamplingConfig(args.min_output_len, args.max_output_len))
    master.start_engine()
    if args.layer_scheduler_type != "mbfs":
        master.set_schedule_policy(args.layer_scheduler_type)
    if args.layer_scheduler_step > 1:
        master.set_schedule_block(args.layer_scheduler_step)
    return master, cfg


def run_benchmark_controller(master, cfg, wl: Workload, args):
    rng = np.random.default_rng(args.seed)
    t0 = time.time()
    results, arrivals = [], {}
    for i, (arrival, in_len) in enumerate(wl):
        now = time.time() - t0
        if arrival > now:
            time.sleep(arrival - now)
        prompt = rng.integers(3, cfg.vocab_size, in_len).tolist()
        out_len = wl.output_lens[i] if wl.output_lens else args.max_output_len
        res = master.put_single_request(prompt, output_len=out_len)
        arrivals[res.req_id] = time.time()
        results.append(res)
    stats = [r.get(timeout=3600) for r in results]
    return stats, arrivals, time.time() - t0


def run_benchmark_colocated(cfg, wl: Workload, args):
    """One GPU, fused executor: the driver loop admits arrived requests and steps the engine."""
    import torch
    from disagmoe_b200.frontend.colocated import ColocatedEngine
    from disagmoe_b200.frontend.colocated_mixed import MixedBatchEngine
    budget = getattr(args, "prefill_budget", 0)
    kw = dict(prefill_budget=budget) if budget > 0 else {}
    # --prefill-budget N: mixed batches (decode tokens + at most N prompt rows per step, chunked prefill) instead of
    # alternating whole-prompt prefill steps and decode steps
    Engine = MixedBatchEngine if budget > 0 else ColocatedEngine
    eng = Engine(cfg, CacheConfig(block_size=args.block_size, gpu_memory_utilization=args.gpu_usage,
                                  num_gpu_blocks=args.num_blocks), device=args.device,
                 max_batch_size=args.max_batch_size_attn,
                 max_prefill_tokens=max(args.max_input_len, args.max_batch_size_attn, 2048) + (budget if budget > 0 else 0),
                 enable_cuda_graph=args.cuda_graph_attn,
                 dtype=torch.float32 if args.device == "cpu" else None, **kw)
    if args.cuda_graph_attn:
        eng.executor.capture()
    rng = np.random.default_rng(args.seed)
    t0 = time.time()
    nxt, arrivals = 0, {}
    while nxt < len(wl) or eng.has_unfinished():
        now = time.time() - t0
        while nxt < len(wl) and wl.arrivals[nxt] <= now:
            out_len = wl.output_lens[nxt] if wl.output_lens else args.max_output_len
            eng.add_request(nxt, rng.integers(3, cfg.vocab_size, wl.input_lens[nxt]).tolist(), out_len)
            arrivals[nxt] = time.time()
            nxt += 1
        if eng.has_unfinished():
            eng.step()
        elif nxt < len(wl):
            time.sleep(max(0.0, min(0.001, wl.arrivals[nxt] - now)))
    stats = [SloStat(r, s.t_tokens[0], s.t_arrival, s.t_tokens[-1], s.t_tokens) for r, s in eng.finished.items()]
    return stats, arrivals, time.time() - t0


def generate_step_trace(step_stats, path_prefix: str) -> None:
    """Chrome trace (one pid per worker; each engine step is an event carrying the per-layer queue snapshot), the
    running metrics, and the queue-length history (reference: benchmark_serving.py:187-259)."""
    events, metrics, queues = [], {}, {}
    for pid, (infos, traces, metric) in step_stats.items():
        metrics[pid] = metric.as_dict() if hasattr(metric, "as_dict") else metric
        queues[pid] = [(s.start_timestamp_ms, s.pool_snapshot) for s in infos]
        for s in infos:
            events.append({"name": f"layer {s.layer_id}, batch {s.batch_size}", "cat": "step", "ph": "X",
                           "ts": s.start_timestamp_ms * 1e3, "dur": (s.end_timestamp_ms - s.start_timestamp_ms) * 1e3,
                           "pid": pid, "tid": 0, "args": {"pool": s.pool_snapshot}})
        for tname, ranges in traces.items():
            for msg, t_start, t_dur, track in ranges:
                events.append({"name": msg, "cat": "native", "ph": "X", "ts": t_start * 1e3, "dur": t_dur * 1e3,
                               "pid": pid, "tid": f"{tname}/{track}"})
    os.makedirs(os.path.dirname(os.path.abspath(path_prefix)) or ".", exist_ok=True)
    with gzip.open(path_prefix + "trace.json.gz", "wt") as f:
        json.dump(events, f)
    with open(path_prefix + "trace_metrics.json", "w") as f:
        json.dump(metrics, f, indent=1)
    with open(path_prefix + "queue_length.pkl", "wb") as f:
        pickle.dump(queues, f)


def write_ttft_and_throughput(stats: List[SloStat], arrivals, sampler_steps, prefix: str, queueing_delays=None) -> None:
    """ttft.csv, sampler_step.csv, req_finish_time.csv (seconds since the first arrival) and one
    ``<worker>_queueing_delay.csv`` per worker: the inputs of benchmark/plotter/*."""
    import pandas as pd
    os.makedirs(os.path.dirname(os.path.abspath(prefix)) or ".", exist_ok=True)
    t0 = min(arrivals.values()) if arrivals else 0.0
    pd.DataFrame({"finish_time_s": sorted(s.t_decode - t0 for s in stats)}).to_csv(prefix + "req_finish_time.csv",
                                                                                   index=False)
    for kind, lists in (queueing_delays or {}).items():
        for i, delays in enumerate(lists):
            pd.DataFrame({"queueing_delay_ms": delays}).to_csv(prefix + f"{kind}{i}_queueing_delay.csv", index=False)
    pd.DataFrame({"req_id": [s.req_id for s in stats],
                  "ttft_ms": [(s.t_prefill - arrivals.get(s.req_id, s.t_prefill)) * 1e3 for s in stats]}
                 ).to_csv(prefix + "ttft.csv", index=False)
    if sampler_steps:
        pd.DataFrame({"time_stamp": [s.time_stamp for s in sampler_steps],
                      "num_tokens": [s.num_tokens for s in sampler_steps]}).to_csv(prefix + "sampler_step.csv", index=False)


def fused_command(args) -> List[str]:
    """The torchrun command line that serves the same workload on the fused peer-memory path
    (``benchmark/serve_fused.py``, one process per GPU): attention GPUs = tp x dp, the other GPUs hold the experts."""
    n_gpu = args.num_nodes * args.num_gpus
    n_attn = args.tp_size * args.dp_size
    assert 1 <= n_attn < n_gpu, "--tp-size x --dp-size attention GPUs must leave at least one expert GPU"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n_gpu),
           "--master-addr", "127.0.0.1", "--master-port", str(29700 + args.seed % 200),
           os.path.join(os.path.dirname(os.path.abspath(__file__)), "serve_fused.py"), "--model", args.model,
           "--n-attn", str(n_attn), "--attn-tp", str(args.tp_size), "-r", str(args.rate), "-n", str(args.num_requests),
           "--min-input-len", str(args.min_input_len), "-i", str(args.max_input_len),
           "--min-output-len", str(args.min_output_len), "-o", str(args.max_output_len),
           "--generator-type", args.generator_type, "--seed", str(args.seed),
           "--max-seqs-per-mb", str(max(1, args.max_batch_size_attn // 2))]
    if args.num_blocks:
        cmd += ["--num-blocks", str(args.num_blocks)]
    if args.model in ("mixtral", "duo") and args.num_layers != 32:
        cmd += ["-L", str(args.num_layers)]
    return cmd


def run_benchmark_fused(args) -> BenchmarkMetrics:
    """Runs ``fused_command`` and reads the metrics line it appends to a JSON-lines file."""
    import subprocess
    import tempfile
    out = os.path.join(tempfile.mkdtemp(), "fused.jsonl")
    proc = subprocess.run(fused_command(args) + ["-f", out], capture_output=True, text=True)
    if proc.returncode != 0 or not os.path.exists(out):
        raise RuntimeError("fused serving run failed:\n" + (proc.stdout + proc.stderr)[-2000:])
    row = json.loads(open(out).read().strip().splitlines()[-1])
    return BenchmarkMetrics(**{k: row[k] for k in BenchmarkMetrics.__dataclass_fields__ if k in row})


def main(argv=None):
    args = get_parser_base().parse_args(argv)
    np.random.seed(args.seed)
    if args.backend == "fused":
        try:
            metrics = run_benchmark_fused(args)
        except Exception as e:
            print("benchmark failed:", repr(e))
            metrics = BenchmarkMetrics()
        print(metrics)
        metrics.write_to_file(args)
        return metrics
    wl = make_workload(args)
    prefix = os.path.join(os.path.dirname(os.path.abspath(args.file)), "")
    try:
        if args.backend == "colocated":
            cfg = model_config_from_args(args)
            stats, arrivals, dur = run_benchmark_colocated(cfg, wl, args)
            sampler_steps, queueing = [], {}
        else:
            master, cfg = launch(args)
            try:
                if args.profile_dir or args.trace:
                    master.start_profile(args.profile_dir)
                stats, arrivals, dur = run_benchmark_controller(master, cfg, wl, args)
                from disagmoe_b200.frontend.datatypes import SamplerStepInfo
                sampler_steps = [SamplerStepInfo.from_c(s) for s in master.fetch_sampler_step_infos()]
                attn_q, exp_q = master.fetch_queueing_delays()
                queueing = {"attn": attn_q, "expert": exp_q}
                if args.trace:
                    generate_step_trace(master.fetch_step_stats(), prefix)
                if args.profile_dir:
                    master.stop_profile()
            finally:
                master.stop_workers()
        metrics = analyze_results(stats, arrivals, dur)
        if args.analyze_throughput:
            write_ttft_and_throughput(stats, arrivals, sampler_steps, prefix, queueing)
            # the same files under the run's own directory (reports/<settings>/), where the plotters look for them
            from benchmark.plotter.namer import get_dir_path
            write_ttft_and_throughput(stats, arrivals, sampler_steps, os.path.join(get_dir_path(args), ""), queueing)
    except Exception as e:   # a failed run still leaves a row, as the reference does
        print("benchmark failed:", repr(e))
        metrics = BenchmarkMetrics()
    print(metrics)
    metrics.write_to_file(args)
    return metrics


if __name__ == "__main__":
    main()
