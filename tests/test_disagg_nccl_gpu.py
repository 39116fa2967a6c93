"""Reference-style data path on real GPUs: host-scheduled workers in separate processes, NCCL p2p per edge
(native NcclChannel), bf16 kernels. Needs 2 GPUs; skipped otherwise."""
import os
import tempfile

import pytest
import torch

from disagmoe_b200.config import CacheConfig, SamplingConfig, tiny_config
from disagmoe_b200.models.oracle import OracleModel
from disagmoe_b200.models.weights import init_state_dict, save_state_dict
from disagmoe_b200.utils.placement import ClusterConfig, get_model_placement

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_workers_over_nccl_channels():
    from disagmoe_b200.frontend.controller import init_controller
    cfg = tiny_config.clone(ep_size=1, dtype=torch.bfloat16)
    sd = {k: v.to(torch.bfloat16) for k, v in init_state_dict(cfg, dtype=torch.float32).items()}
    path = os.path.join(tempfile.mkdtemp(), "tiny_bf16.pt")
    save_state_dict(sd, path)
    place = get_model_placement(cfg, ClusterConfig(1, 2), "pipeline", 1, 1)
    ctl = init_controller(1, 2, device="cuda")
    try:
        ctl.init_engine(place, cfg, CacheConfig(block_size=16, num_gpu_blocks=256), SamplingConfig(4, 5),
                        state_dict_path=path, keep_logits=True)
        ctl.start_engine()
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (12,), generator=g).tolist() for _ in range(4)]
        res = [ctl.put_single_request(p, output_len=4) for p in prompts]
        ctl.wait_for_requests(4, timeout=120)
        logits = ctl.fetch_logits()
        oracle = OracleModel(cfg, {k: v.float() for k, v in sd.items()})
        for r, p in zip(res, prompts):
            ref = oracle.forward(r.req_id, p)[-1]
            got = logits[(r.req_id, 11)]
            assert (got - ref).abs().max() / ref.abs().max() < 0.06
            assert len(r.tokens) == 4
        assert not [e for e in ctl.worker_errors().values() if e]
    finally:
        ctl.stop_workers()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_fused_serving_matches_colocated():
    """Continuous batching on the fused peer-memory path (1 attention + 1 expert GPU, one process each): Poisson
    arrivals with real prefill; the generated tokens are compared with the single-GPU colocated engine."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29655", os.path.join(root, "benchmark", "serve_fused.py"), "--model", "tiny",
           "-r", "200", "-n", "24", "--min-input-len", "8", "-i", "40", "--min-output-len", "4", "-o", "12",
           "--max-seqs-per-mb", "8", "--max-tokens-per-mb", "96", "--max-prefill-tokens-per-mb", "24", "--num-blocks", "512",
           "--time-limit", "120", "--check"]       # prompts of up to 40 tokens against a 24-token budget: chunked prefill
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    lines = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    info = next(l for l in lines if "iterations" in l)
    check = next(l for l in lines if "check_tokens_agree" in l)
    assert info["kernel_status"] == 0 and info["requests_finished"] == 24
    assert check["check_first_tokens_agree"] >= 0.9, check
    assert check["check_tokens_agree"] >= 0.7, check
