"""Model-level attention tensor parallelism over the native NCCL group channel, on 2 GPUs (one process per GPU):
group-channel collectives (barrier, tensor broadcast, metadata broadcast, all-reduce), then a TP = 2
``ParallelAttnExecutor`` (heads and KV heads sharded, o_proj partial sums all-reduced through the channel) against the
single-GPU ``AttnExecutor``. Also the in-module two-device NCCL point-to-point test."""
import os
import tempfile

import pytest
import torch

from disagmoe_b200.config import CacheConfig, tiny_config
from disagmoe_b200.models.weights import init_state_dict, save_state_dict

pytestmark = pytest.mark.gpu
needs_two = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")


def _cfg(**kw):
    return tiny_config.clone(dtype=torch.bfloat16, max_seq_len=256, **kw)


def _inputs(cfg):
    g = torch.Generator().manual_seed(11)
    n = 6
    x = torch.randn(n, cfg.hidden_size, generator=g).to(torch.bfloat16)
    ctx = torch.tensor([3, 17, 30, 9, 22, 1], dtype=torch.int32)
    bt = torch.arange(n * 2, dtype=torch.int32).view(n, 2)
    slots = bt.gather(1, (ctx // 16).long()[:, None]).squeeze(1).long() * 16 + (ctx % 16).long()
    kv = (torch.randn(cfg.num_layers, 2, 32, 16, cfg.num_kv_heads, cfg.head_dim, generator=g) * 0.5).to(torch.bfloat16)
    return x, ctx, bt, slots, kv


def _run_layers(ex, cfg, x, ctx, bt, slots, dev):
    from disagmoe_b200.models.attention import AttnMeta
    outs = []
    meta = AttnMeta(ctx.to(dev), slots.to(dev), bt.to(dev), None, (ctx + 1).to(dev), num_decode_tokens=len(ctx), max_ctx=64)
    for layer in range(cfg.num_layers):
        h = x.to(dev).clone()
        y, w, ids = ex.execute(layer, ctx.to(dev), h, meta)
        # numpy, not tensors: a tensor put on a multiprocessing queue is shared by file descriptor and the sending
        # process would have to outlive the receive
        outs.append((y.float().cpu().numpy(), w.float().cpu().numpy(), ids.cpu().numpy(), h.float().cpu().numpy()))
    torch.cuda.synchronize()
    return outs


def _tp_worker(rank, uid, sd_path, q):
    from disagmoe_b200 import disagmoe_c as C
    from disagmoe_b200.executor.executor import ParallelAttnExecutor
    from disagmoe_b200.models import distributed as D
    from disagmoe_b200.models.weights import load_state_dict
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    res = {}
    ch = C.create_nccl_group_channel(rank, 2, uid)
    ch.instantiate()
    ch.barrier()
    # tensor broadcast from rank 0
    m = C.Metadata()
    m.shape, m.dtype = [3, 4], "fp32"
    src = torch.arange(12, dtype=torch.float32, device=dev).view(3, 4)
    if rank == 0:
        ch.send(src, m)
        res["bcast"] = True
    else:
        res["bcast"] = bool(torch.equal(ch.recv(m).cpu(), src.cpu()))
    # metadata broadcast
    md = C.Metadata()
    md.shape, md.dtype, md.layer_id = [2, 8], "bf16", 5
    md.req_ids, md.exp_ids, md.attn_dp_ranks, md.init_prefill_lens = [7, 9], [1, 3], [0, 1], [-1, 4]
    md.topk_weights = [0.25, 0.75]
    if rank == 0:
        ch.send_metadata(md)
        res["meta"] = True
    else:
        got = ch.recv_metadata()
        res["meta"] = (got.layer_id == 5 and list(got.req_ids) == [7, 9] and list(got.exp_ids) == [1, 3]
                       and list(got.init_prefill_lens) == [-1, 4] and list(got.shape) == [2, 8])
    # all-reduce
    t = torch.full((4, 8), float(rank + 1), dtype=torch.bfloat16, device=dev)
    ch.all_reduce(t)
    ch.sync()
    res["allreduce"] = bool((t.float() == 3.0).all())
    # TP = 2 attention executor over the channel
    cfg = _cfg(tp_size=2, rank=rank)
    D.set_tensor_model_parallel_config(cfg)
    D.set_tensor_model_parallel_channel(ch)
    sd = load_state_dict(sd_path)
    ex = ParallelAttnExecutor(cfg, CacheConfig(block_size=16), device=dev, state_dict=sd)
    ex.initialize_cache(32)
    x, ctx, bt, slots, kv = _inputs(cfg)
    kvh = cfg.num_kv_heads // 2
    ex.cache.copy_(kv[..., rank * kvh:(rank + 1) * kvh, :].to(dev))
    res["layers"] = _run_layers(ex, cfg, x, ctx, bt, slots, dev)
    ch.barrier()
    q.put((rank, res))


@needs_two
def test_group_channel_and_tp_executor_two_gpus():
    import torch.multiprocessing as mp
    from disagmoe_b200 import disagmoe_c as C
    from disagmoe_b200.executor.executor import AttnExecutor
    cfg = _cfg()
    sd = {k: v.to(torch.bfloat16) for k, v in init_state_dict(cfg, dtype=torch.float32).items()}
    path = os.path.join(tempfile.mkdtemp(), "tiny_bf16.pt")
    save_state_dict(sd, path)
    uid = C.get_nccl_unique_id()
    ctx_mp = mp.get_context("spawn")
    q = ctx_mp.Queue()
    env = dict(NCCL_NVLS_ENABLE="0")
    os.environ.update(env)
    ps = [ctx_mp.Process(target=_tp_worker, args=(r, uid, path, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = dict(q.get(timeout=240) for _ in ps)
    for p in ps:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in (0, 1):
        assert got[r]["bcast"] and got[r]["meta"] and got[r]["allreduce"], got[r]
    ref = AttnExecutor(cfg, CacheConfig(block_size=16), device="cuda:0", state_dict=sd)
    ref.initialize_cache(32)
    x, ctx, bt, slots, kv = _inputs(cfg)
    ref.cache.copy_(kv.cuda())
    want = _run_layers(ref, cfg, x, ctx, bt, slots, torch.device("cuda", 0))
    for r in (0, 1):
        for layer, ((y, w, ids, h), (y0, w0, ids0, h0)) in enumerate(zip(got[r]["layers"], want)):
            assert abs(h - h0).max() / abs(h0).max() < 3e-2, f"rank {r} layer {layer}: residual stream"
            assert abs(y - y0).max() / abs(y0).max() < 3e-2, f"rank {r} layer {layer}: expert input"
            assert (ids == ids0).mean() >= 0.8, f"rank {r} layer {layer}: router ids"


@needs_two
def test_in_module_nccl_p2p_two_devices():
    from disagmoe_b200 import disagmoe_c as C
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    assert C.test_nccl_p2p(0, 1, 64, 256)


@needs_two
def test_in_module_nccl_group_and_overlap():
    """The native module's own tests of the N-rank group channel (barrier, tensor and object broadcast, all-reduce; one
    thread per device in this process) and of collective / compute overlap (broadcasts on the channel's stream while the
    debug kernel runs on a compute stream): counterparts of the reference's test_nccl_group and test_op_overlap."""
    from disagmoe_b200 import disagmoe_c as C
    n = min(4, torch.cuda.device_count())
    assert C.test_nccl_group(list(range(n)))
    tb, tk, tboth = C.test_op_overlap(0, 1, 64, 400)
    assert tb > 0 and tk > 0 and tboth > 0
    # overlap: running both takes clearly less than running one after the other (generous margin: shared machine)
    assert tboth < 0.95 * (tb + tk) or tboth < 1.5 * max(tb, tk), (tb, tk, tboth)
