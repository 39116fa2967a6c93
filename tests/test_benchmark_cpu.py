"""Benchmark harness on CPU: workload generators, metric analysis, an end-to-end tiny serving run with trace output."""
import os

import numpy as np

from benchmark.benchmark_serving import analyze_results, main
from benchmark.workload import get_generator
from disagmoe_b200.frontend.datatypes import SloStat


def test_generators():
    for name in ("uniform", "poisson", "offline", "incremental_poisson"):
        g = get_generator(name)(10.0, 1.0, 5, 9, seed=1, min_output_len=2, max_output_len=4)
        wl = g.generate_num(50)
        assert len(wl) == 50 and all(5 <= l < 9 for l in wl.input_lens) and all(2 <= o < 4 for o in wl.output_lens)
        assert all(b >= a for a, b in zip(wl.arrivals, wl.arrivals[1:]))
    p = get_generator("poisson")(20.0, 1.0, 1, 2, seed=0).generate_num(4000)
    assert abs(np.mean(np.diff(p.arrivals)) - 0.05) < 0.005
    assert get_generator("uniform")(4.0, 1.0, 1, 2).generate_duration(10).arrivals[-1] == 39 / 4.0


def test_analyze_results():
    stats = [SloStat(0, 1.0, 0.5, 2.0, [1.0, 1.5, 2.0]), SloStat(1, 1.2, 0.6, 1.6, [1.2, 1.4, 1.6])]
    m = analyze_results(stats, {0: 0.5, 1: 0.6}, duration=2.0)
    assert m.req_throughput == 1.0 and m.token_throughput == 3.0
    assert abs(m.req_latency_mean_ms - 1250) < 1e-6 and abs(m.itl_latency_median_ms - 350) < 1e-6
    assert abs(m.ttft_mean_ms - 550) < 1e-6


def test_end_to_end_tiny_cpu(tmp_path, monkeypatch):
    monkeypatch.setenv("DMOE_REPORTS_DIR", str(tmp_path / "reports"))
    out = tmp_path / "bench.csv"
    m = main(["--device", "cpu", "--model", "tiny", "-g", "2", "--ep-size", "1", "--step-attn", "1", "--step-expert", "1",
              "-n", "6", "-r", "200", "--min-input-len", "4", "-i", "9", "--min-output-len", "3", "-o", "5", "-K", "2",
              "--trace", "--analyze-throughput", "-f", str(out), "--num-blocks", "128"])
    assert m.token_throughput > 0 and m.itl_latency_p99_ms >= 0
    assert out.exists() and (tmp_path / "trace.json.gz").exists() and (tmp_path / "ttft.csv").exists()
    # the run's own directory holds what the plotters read; every plotter runs on it (CSV fallback without matplotlib)
    runs = list((tmp_path / "reports").iterdir())
    assert len(runs) == 1 and runs[0].name.startswith("rate=200")
    run = runs[0]
    for name in ("ttft.csv", "sampler_step.csv", "req_finish_time.csv", "attn0_queueing_delay.csv",
                 "expert0_queueing_delay.csv"):
        assert (run / name).exists(), name
    from benchmark.plotter import output_req, queue_length_interact, queueing_delay, sampler_step, ttft
    for mod in (output_req, sampler_step, ttft, queueing_delay):
        assert mod.main([str(run)])
    html = queue_length_interact.main([str(tmp_path / "queue_length.pkl"), "--worker", "0"])
    assert os.path.getsize(html) > 200
    from benchmark.plotter import latency_cdf, queue_length
    heat = queue_length.main([str(tmp_path / "queue_length.pkl"), "--out-dir", str(tmp_path / "plots")])
    assert len(heat) == 2 and all(os.path.exists(f) for f in heat)           # one heat map per worker
    cdfs = latency_cdf.main(["--ttft", str(run / "ttft.csv"), "--sampler", str(run / "sampler_step.csv"),
                             "--out-dir", str(tmp_path / "plots")])
    assert len(cdfs) == 3 and all(os.path.exists(f) for f in cdfs)


def test_colocated_backend_cpu(tmp_path):
    m = main(["--device", "cpu", "--model", "tiny", "--backend", "colocated", "-n", "5", "-r", "0", "--min-input-len", "4",
              "-i", "8", "--min-output-len", "2", "-o", "4", "-f", str(tmp_path / "b.csv"), "--num-blocks", "64",
              "--max-batch-size-attn", "4"])
    assert m.req_throughput > 0
    # the same workload with mixed batches (8 prompt rows per step)
    m2 = main(["--device", "cpu", "--model", "tiny", "--backend", "colocated", "-n", "5", "-r", "0", "--min-input-len", "4",
               "-i", "8", "--min-output-len", "2", "-o", "4", "-f", str(tmp_path / "b.csv"), "--num-blocks", "64",
               "--max-batch-size-attn", "4", "--prefill-budget", "8"])
    assert m2.req_throughput > 0 and m2.token_throughput > 0


def test_remote_comm_latency_socket_pair():
    """sender.py / recver.py as two processes on this host over the runtime's TCP channel."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = ["--transport", "socket", "--iters", "4", "--warmup", "1", "--rows", "64", "--hidden", "256", "--port-base", "3200"]
    rx = subprocess.Popen([sys.executable, os.path.join(root, "benchmark/remote_comm_latency/recver.py")] + args,
                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    tx = subprocess.run([sys.executable, os.path.join(root, "benchmark/remote_comm_latency/sender.py")] + args,
                        capture_output=True, text=True, timeout=120)
    out_rx, _ = rx.communicate(timeout=60)
    assert tx.returncode == 0, tx.stdout + tx.stderr
    assert rx.returncode == 0, out_rx
    assert "one way in" in tx.stdout and "receiver done: 10 transfers" in out_rx


def test_http_server_run_once_and_policy_switch():
    """The benchmark server in-process: start-up launches the workers, /run_once runs a small workload, /set_schedule
    switches the layer-scheduling policy of every worker, bad input is rejected with 400."""
    from fastapi.testclient import TestClient
    from benchmark.server import create_app
    from benchmark.utils import get_parser_base
    args = get_parser_base().parse_args(
        ["--device", "cpu", "--model", "tiny", "-g", "2", "--ep-size", "1", "--step-attn", "1", "--step-expert", "1",
         "--min-input-len", "4", "-i", "8", "--min-output-len", "2", "-o", "4", "-K", "2", "--num-blocks", "128"])
    with TestClient(create_app(args)) as client:
        assert client.get("/health").json() == {"suspect_workers": [], "workers": 2}
        assert client.post("/set_schedule", json={"policy": "flfs", "step": 2}).json() == {"ok": True}
        assert client.post("/set_schedule", json={"policy": "nonsense"}).status_code == 400
        assert client.post("/set_schedule", json={}).status_code == 400
        m = client.post("/run_once", json={"rate": 40, "time": 0.2, "distribution": "poisson"}).json()
        assert m["token_throughput"] > 0 and m["req_throughput"] > 0
        g = client.post("/generate", json={"prompt_ids": [5, 6, 7, 8], "max_new_tokens": 3}).json()
        assert len(g["tokens"]) == 3 and len(g["t_tokens"]) == 3
        again = client.post("/generate", json={"prompt_ids": [5, 6, 7, 8], "max_new_tokens": 3}).json()
        assert again["tokens"] == g["tokens"]                         # greedy decoding is deterministic
        assert client.post("/generate", json={"prompt_ids": []}).status_code == 400
        assert client.post("/generate", json={"prompt_ids": [10 ** 9]}).status_code == 400


def test_queueing_simulator_policies():
    from simulator.queueing import simulate
    for policy in ("largest", "fcfs", "first"):
        out = simulate(rate=30, n_layers=4, step_ms=3.0, duration_s=2.0, policy=policy, out_len=4, seed=1)
        # a token passes 4 layers of 3 ms each between two outputs of its request, whatever the policy
        assert out["steps"] > 0 and out["itl_mean_ms"] >= 3.0 * 4 - 1e-6 and out["itl_p99_ms"] >= out["itl_p50_ms"], (policy, out)


def test_preprocess_microbenchmark_runs():
    from benchmark import benchmark_preprocess
    out = benchmark_preprocess.main(["--iters", "3"])
    assert out is None or out


def test_fused_backend_command_line():
    """--backend fused maps the benchmark flags onto the torchrun job of benchmark/serve_fused.py."""
    from benchmark.benchmark_serving import fused_command
    from benchmark.utils import get_parser_base
    a = get_parser_base().parse_args(["--backend", "fused", "-g", "8", "--tp-size", "4", "--dp-size", "1", "-r", "16", "-n",
                                      "96", "--min-input-len", "128", "-i", "1024", "--min-output-len", "64", "-o", "512",
                                      "--num-blocks", "16384", "--max-batch-size-attn", "256"])
    cmd = fused_command(a)
    joined = " ".join(cmd)
    assert "--nproc-per-node 8" in joined and "serve_fused.py" in joined
    assert "--n-attn 4 --attn-tp 4" in joined and "-r 16.0 -n 96" in joined and "--max-seqs-per-mb 128" in joined
    assert "--num-blocks 16384" in joined


def test_worker_address_flag():
    from benchmark.benchmark_serving import parse_worker_addresses
    assert parse_worker_addresses("") == {}
    assert parse_worker_addresses("3=10.0.0.2:7700, 4=node-b:7701") == {3: ("10.0.0.2", 7700), 4: ("node-b", 7701)}


def test_pipeline_model_regimes():
    """The event model of the fused pipeline: the slower side sets the step, hops only matter when there is no slack,
    and a single micro-batch serialises the two sides."""
    from simulator.pipeline import simulate
    kw = dict(experts=8, layers=32, jitter=0.0, head_us=0.0)
    attn_bound = simulate(4, 4, micro_batches=2, attn_us=300, expert_us_per_expert=100, hop_us=5, **kw)     # experts 200 us
    assert abs(attn_bound["step_ms"] - 64 * 0.300) < 0.5 and attn_bound["attention_busy"] > 0.97
    exp_bound = simulate(2, 2, micro_batches=2, attn_us=200, expert_us_per_expert=100, hop_us=5, **kw)      # experts 400 us
    assert abs(exp_bound["step_ms"] - 64 * 0.400) < 0.7 and exp_bound["expert_busy"] > 0.95
    serial = simulate(4, 4, micro_batches=1, attn_us=300, expert_us_per_expert=100, hop_us=5, **kw)
    assert abs(serial["step_ms"] - 32 * (0.300 + 0.200 + 0.010)) < 0.3
    slow_hops = simulate(4, 4, micro_batches=2, attn_us=300, expert_us_per_expert=100, hop_us=80, **kw)
    assert slow_hops["step_ms"] > attn_bound["step_ms"] + 1.0          # 200 + 2 x 80 > 300: the attention side now waits
    uneven = simulate(5, 3, micro_batches=2, attn_us=300, expert_us_per_expert=100, hop_us=5, **kw)
    assert uneven["experts_per_gpu_max"] == 3
