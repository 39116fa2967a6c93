"""Host-scheduled disaggregated serving on CPU (fp32): attention worker + expert worker over the native runtime
(pools, layer schedulers, dispatchers, tokenizer / sampler), logits against the single-process fp32 oracle."""
import os
import tempfile

import pytest
import torch

from disagmoe_b200.config import CacheConfig, SamplingConfig, tiny_config
from disagmoe_b200.frontend.controller import init_controller
from disagmoe_b200.models.oracle import OracleModel
from disagmoe_b200.models.weights import init_state_dict, save_state_dict
from disagmoe_b200.utils.placement import ClusterConfig, get_model_placement


def _run(cfg, placement_args, n_dev, in_process, n_req, prompt_len, n_new, strategy="pipeline", worker_addresses=None):
    sd = init_state_dict(cfg)
    tmp = tempfile.mkdtemp()
    path = os.path.join(tmp, "tiny.pt")
    save_state_dict(sd, path)
    place = get_model_placement(cfg, ClusterConfig(1, n_dev), strategy, *placement_args)
    ctl = init_controller(1, n_dev, device="cpu", in_process=in_process, worker_addresses=worker_addresses)
    try:
        ctl.init_engine(place, cfg, CacheConfig(block_size=16, num_gpu_blocks=256), SamplingConfig(n_new, n_new + 1),
                        state_dict_path=path, keep_logits=True, dtype=torch.float32)
        ctl.start_engine()
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(n_req)]
        res = [ctl.put_single_request(p, output_len=n_new) for p in prompts]
        ctl.wait_for_requests(n_req, timeout=240)
        logits = ctl.fetch_logits()
        oracle = OracleModel(cfg, sd)
        worst = 0.0
        for r, p in zip(res, prompts):
            toks, rows = oracle.generate(r.req_id, p, n_new)
            assert r.tokens == toks, f"request {r.req_id}: {r.tokens} vs {toks}"
            for i in range(n_new):
                got = logits[(r.req_id, prompt_len - 1 + i)]
                worst = max(worst, (got - rows[i]).abs().max().item())
            assert len(r.slo.t_tokens) == n_new and r.slo.t_decode >= r.slo.t_prefill
        assert worst < 1e-4, f"max logit error {worst}"
        errs = [e for e in ctl.worker_errors().values() if e]
        assert not errs, errs
        # bookkeeping the reference controller exposes under the same names
        attn_q, exp_q = ctl.fetch_queueing_delays()
        assert attn_q and all(len(q) > 0 and min(q) >= 0.0 for q in attn_q)
        if strategy != "colocate":
            assert exp_q and all(len(q) > 0 for q in exp_q) and max(max(q) for q in attn_q + exp_q) > 0.0
        assert set(ctl.fetch_submitted_time()) == {r.req_id for r in res}
        assert ctl.determine_worker_type(0) in ("attention", "hybrid") and len(ctl.all_device_ids) == n_dev + 2
    finally:
        ctl.stop_workers()


def test_disaggregated_in_process_1attn_1expert():
    cfg = tiny_config.clone(ep_size=1)
    _run(cfg, (1, 1), 2, True, n_req=4, prompt_len=12, n_new=4)


def test_colocated_in_process():
    cfg = tiny_config.clone(ep_size=1)
    _run(cfg, (), 1, True, n_req=3, prompt_len=9, n_new=3, strategy="colocate")


def test_two_processes_16_requests_prompt32_decode16():
    """1 attention worker + 1 expert worker as separate processes over TCP: 16 requests, prompt 32, 16 greedy
    tokens, paged KV with block size 16; logits within 1e-4 of the colocated single-process oracle."""
    cfg = tiny_config.clone(ep_size=1)
    _run(cfg, (1, 1), 2, False, n_req=16, prompt_len=32, n_new=16)


def test_four_processes_ep2_striped_attention():
    """2 attention stages (layers striped) + EP=2 expert workers: residual stream crosses attention workers."""
    cfg = tiny_config.clone(ep_size=2)
    _run(cfg, (2, 1), 4, False, n_req=6, prompt_len=10, n_new=5)


def test_three_processes_attention_tp2():
    """Attention tensor parallelism on the host-scheduled path: a TP group of two attention processes (the driver takes
    part in the token flow and broadcasts every batch it schedules; both run their head / KV shard and all-reduce the
    o_proj partial sums over gloo) + one expert process; logits against the single-process oracle."""
    cfg = tiny_config.clone(ep_size=1, tp_size=2)
    _run(cfg, (1, 1), 3, False, n_req=5, prompt_len=11, n_new=6)


def test_serial_expert_gemm_mode_matches_oracle():
    """enable_grouped_gemm = False: expert workers run one dense GEMM per expert; same logits."""
    cfg = tiny_config.clone(ep_size=1, enable_grouped_gemm=False)
    _run(cfg, (1, 1), 2, True, n_req=3, prompt_len=7, n_new=3)


def test_expert_worker_hosted_by_a_node_agent():
    """Multi-node deployment path: the expert worker is hosted by a node agent reached over TCP (here on this host), the
    attention worker is a local process; same logits as the oracle. A dead remote worker is noticed too."""
    from disagmoe_b200.frontend.node_agent import NodeAgent
    agent = NodeAgent("127.0.0.1", 7791)
    agent.start_in_thread()
    try:
        cfg = tiny_config.clone(ep_size=1)
        _run(cfg, (1, 1), 2, False, n_req=4, prompt_len=9, n_new=4, worker_addresses={1: ("127.0.0.1", 7791)})
    finally:
        agent.stop()
