"""Fused dispatch / combine pipeline: 2 attention + 2 expert "ranks" emulated on one GPU (arenas that point at each
other, kernels launched in an order in which no flag wait has to block) against the colocated executor."""
import pytest
import torch

from disagmoe_b200.config import CacheConfig, tiny_config
from disagmoe_b200.executor.fused import FusedModelExecutor
from disagmoe_b200.models.weights import init_state_dict
from disagmoe_b200.ops import gemm
from disagmoe_b200.parallel.disagg import AttentionRank, DisaggShape, ExpertRank, build_layout
from disagmoe_b200.parallel.peer import PeerArena

pytestmark = pytest.mark.gpu


def assert_close(got, ref, what):
    """Logits of two bf16 pipelines that differ in summation order: every element within 2^-5 |ref| + 2^-5 rms(ref)
    (each is ~2^-8 relative per rounding; a handful of roundings per layer accumulate over the layers)."""
    got, ref = got.float(), ref.float()
    bound = ref.abs() * 2 ** -5 + ref.pow(2).mean().sqrt() * 2 ** -5
    bad = int(((got - ref).abs() > bound).sum())
    assert bad == 0, f"{what}: {bad} of {ref.numel()} elements off, max err {(got - ref).abs().max().item():.4g}, " \
                     f"rms {ref.pow(2).mean().sqrt().item():.4g}"


def _model(variant, num_layers):
    """'mixtral': routed experts only. 'shared_dense': first layer with a dense FFN, a sigmoid-gated shared expert next to
    the routed ones and a Zipf(1.2) popularity skew on the router (the Qwen-MoE / DeepSeek-V2-Lite layer types)."""
    cfg = tiny_config.clone(dtype=torch.bfloat16, num_layers=num_layers)
    skew = 0.0
    if variant == "shared_dense":
        cfg = cfg.clone(first_k_dense=1, dense_intermediate_size=768, num_shared_experts=1, shared_intermediate_size=512,
                        shared_expert_gate=True, norm_topk_prob=False)
        skew = 1.2
    sd = {k: v.to(torch.bfloat16) for k, v in init_state_dict(cfg, dtype=torch.float32).items()}
    return cfg, sd, skew


@pytest.mark.parametrize("A,X,n_mb,variant", [(1, 1, 1, "mixtral"), (2, 2, 2, "mixtral"), (1, 4, 2, "mixtral"),
                                              (2, 3, 2, "shared_dense"), (1, 3, 1, "mixtral")])
def test_emulated_disagg_matches_colocated(A, X, n_mb, variant):
    cfg, sd, skew = _model(variant, 3)
    B = 3 if n_mb * 3 * 4 <= 60 else 2
    shape = DisaggShape(A, X, n_mb, B, cfg.top_k, cfg.hidden_size, cfg.num_experts)
    layout = build_layout(shape)
    arenas = PeerArena.emulated(A + X, layout.size)
    attn = [AttentionRank(cfg, shape, arenas[a], layout, a, num_blocks=64, state_dict=sd) for a in range(A)]
    exps = [ExpertRank(cfg, shape, arenas[A + x], layout, x, state_dict=sd) for x in range(X)]
    ref = FusedModelExecutor(cfg, CacheConfig(block_size=16), device="cuda", max_batch_size=B, max_prefill_tokens=B,
                             state_dict=sd, num_blocks=64, enable_cuda_graph=False)
    for layer in [x for a in attn for x in a.layers] + list(ref.attn.values()):
        layer.set_route_skew(skew)
    g = torch.Generator().manual_seed(0)
    kv = torch.randn(ref.kv_cache.shape, generator=g).to(torch.bfloat16).cuda() * 0.5
    for step in range(2):   # two iterations: epochs and cleared histograms must carry over
        inputs = {}
        for a in range(A):
            if step == 0:
                attn[a].kv_cache.copy_(kv)
            perm = torch.randperm(60, generator=g)   # disjoint KV blocks for every sequence of the rank
            for m in range(n_mb):
                ids = torch.randint(0, cfg.vocab_size, (B,), generator=g).int()
                ctx = torch.randint(3, 40, (B,), generator=g).int()
                rows = torch.arange(B, dtype=torch.int32) + m * B
                bt = perm[m * B * 4:(m + 1) * B * 4].view(B, 4).int()
                attn[a].block_tables[m * B:(m + 1) * B, :4] = bt.cuda()
                slots = torch.tensor([int(bt[i, int(ctx[i]) // 16]) * 16 + int(ctx[i]) % 16 for i in range(B)])
                d = attn[a].mb[m]
                d["ids"].copy_(ids); d["positions"].copy_(ctx); d["ctx_len"].copy_(ctx + 1)
                d["bt_row"].copy_(rows); d["slots"].copy_(slots)
                inputs[(a, m)] = (ids, ctx, slots, bt)
        for a in range(A):
            attn[a].kv_cache_before = attn[a].kv_cache.clone()
            for m in range(n_mb):
                attn[a].embed(m)
        for l in range(cfg.num_layers):
            for m in range(n_mb):
                for a in range(A):
                    attn[a].layer(l, m)
                for x in range(X):
                    exps[x].layer(l, m)
        for a in range(A):
            for m in range(n_mb):
                attn[a].head(m)
        torch.cuda.synchronize()
        assert gemm.check_status() == 0
        for (a, m), (ids, ctx, slots, bt) in inputs.items():
            if step == 0:
                ref.kv_cache.copy_(kv)
            else:
                ref.kv_cache.copy_(attn[a].kv_cache_before)
            ref.block_tables[:B, :4] = bt.cuda()
            _, lg = ref.decode(ids, ctx, slots, ctx + 1, torch.arange(B, dtype=torch.int32), want_logits=True)
            assert_close(attn[a].mb[m]["logits"], lg, f"rank {a} mb {m} step {step}")


@pytest.mark.parametrize("A,X,tp,n_mb,variant", [(2, 1, 2, 1, "mixtral"), (4, 2, 2, 2, "mixtral"),
                                                 (2, 3, 2, 2, "shared_dense"), (4, 1, 4, 1, "mixtral")])
def test_emulated_tensor_parallel_attention(A, X, tp, n_mb, variant):
    """Attention TP: all-gather of the normalised rows into the QKV GEMM, head-sharded QKV / attention / o_proj,
    reduce-scatter in the o_proj epilogue, row-sharded router / dispatch / LM head, id exchange at the end. B = 6 rows
    over tp = 4 gives shards of 2, 2, 2 and 0 rows: an empty shard still has to take part in every hand-shake."""
    cfg, sd, skew = _model(variant, 3 if variant == "shared_dense" else 2)
    B = 6 if tp == 4 else 4
    shape = DisaggShape(A, X, n_mb, B, cfg.top_k, cfg.hidden_size, cfg.num_experts, tp)
    layout = build_layout(shape)
    arenas = PeerArena.emulated(A + X, layout.size)
    attn = [AttentionRank(cfg, shape, arenas[a], layout, a, num_blocks=64, state_dict=sd) for a in range(A)]
    exps = [ExpertRank(cfg, shape, arenas[A + x], layout, x, state_dict=sd) for x in range(X)]
    ref = FusedModelExecutor(cfg, CacheConfig(block_size=16), device="cuda", max_batch_size=B, max_prefill_tokens=B,
                             state_dict=sd, num_blocks=64, enable_cuda_graph=False)
    for layer in [x for a in attn for x in a.layers] + list(ref.attn.values()):
        layer.set_route_skew(skew)
    g = torch.Generator().manual_seed(0)
    kv = torch.randn(ref.kv_cache.shape, generator=g).to(torch.bfloat16).cuda() * 0.5     # [L, 2, nb, bs, kvh, hd]
    kvh = cfg.num_kv_heads // tp
    inputs = {}
    for grp in range(A // tp):
        perm = torch.randperm(60, generator=g)
        for m in range(n_mb):
            ids = torch.randint(0, cfg.vocab_size, (B,), generator=g).int()
            ctx = torch.randint(3, 40, (B,), generator=g).int()
            bt = perm[m * B * 4:(m + 1) * B * 4].view(B, 4).int()
            slots = torch.tensor([int(bt[i, int(ctx[i]) // 16]) * 16 + int(ctx[i]) % 16 for i in range(B)])
            inputs[(grp, m)] = (ids, ctx, slots, bt)
            for r in range(tp):
                a = attn[grp * tp + r]
                a.kv_cache.copy_(kv[..., r * kvh:(r + 1) * kvh, :])
                a.block_tables[m * B:(m + 1) * B, :4] = bt.cuda()
                d = a.mb[m]
                d["ids"].copy_(ids); d["positions"].copy_(ctx); d["ctx_len"].copy_(ctx + 1)
                d["bt_row"].copy_(torch.arange(B, dtype=torch.int32) + m * B); d["slots"].copy_(slots)
    for a in attn:
        for m in range(n_mb):
            a.embed(m)
    # one stream, several ranks: every phase is launched for all ranks before the phase that waits for it
    for l in range(cfg.num_layers):
        for m in range(n_mb):
            for a in attn:
                a.layer_pre(l, m)
            for a in attn:
                a.layer_attn(l, m)
            for a in attn:
                a.layer_route_dispatch(l, m)
            for e in exps:
                e.layer(l, m)
    for a in attn:
        for m in range(n_mb):
            a.head(m)
    for a in attn:
        for m in range(n_mb):
            a.head_wait(m)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    per = (B + tp - 1) // tp
    for (grp, m), (ids, ctx, slots, bt) in inputs.items():
        ref.kv_cache.copy_(kv)
        ref.block_tables[:B, :4] = bt.cuda()
        nxt, lg = ref.decode(ids, ctx, slots, ctx + 1, torch.arange(B, dtype=torch.int32), want_logits=True)
        for r in range(tp):
            a = attn[grp * tp + r]
            lo, hi = min(B, r * per), min(B, (r + 1) * per)          # the rows this rank owns
            got = a.mb[m]["logits"][:hi - lo]
            assert_close(got, lg[lo:hi], f"group {grp} tp rank {r} mb {m}")
            # every member holds the sampled ids of the whole group after the id exchange
            own = a.mb[m]["next_local"][:hi - lo]
            assert torch.equal(a.mb[m]["next_ids"][lo:hi], own)
            assert torch.equal(a.mb[m]["next_ids"], attn[grp * tp].mb[m]["next_ids"])


def test_emulated_mixed_prompt_and_decode_rows():
    """A serving iteration: micro-batch 0 = one 12-token prompt + 2 decode tokens + padding rows, micro-batch 1 = 3 decode
    tokens (fewer active rows than the buffers hold). Rows that produce a token must match the colocated executor's
    prefill / decode logits."""
    cfg, sd, _ = _model("mixtral", 2)
    A, X, n_mb, cap = 1, 2, 2, 32
    shape = DisaggShape(A, X, n_mb, cap, cfg.top_k, cfg.hidden_size, cfg.num_experts)
    layout = build_layout(shape)
    arenas = PeerArena.emulated(A + X, layout.size)
    attn = AttentionRank(cfg, shape, arenas[0], layout, 0, num_blocks=64, state_dict=sd)
    exps = [ExpertRank(cfg, shape, arenas[A + x], layout, x, state_dict=sd) for x in range(X)]
    ref = FusedModelExecutor(cfg, CacheConfig(block_size=16), device="cuda", max_batch_size=8, max_prefill_tokens=32,
                             state_dict=sd, num_blocks=64, enable_cuda_graph=False)
    g = torch.Generator().manual_seed(1)
    kv = torch.randn(ref.kv_cache.shape, generator=g).to(torch.bfloat16).cuda() * 0.5
    attn.kv_cache.copy_(kv)
    ref.kv_cache.copy_(kv)
    bt = torch.arange(8 * 4, dtype=torch.int32).view(8, 4)          # sequence r owns blocks 4r .. 4r + 3
    bt[7] = 63                                                       # row 7: padding rows, scratch page
    attn.block_tables[:8, :4] = bt.cuda()
    ref.block_tables[:8, :4] = bt.cuda()
    slot = lambda r, p: int(bt[r, p // 16]) * 16 + p % 16
    prompt = torch.randint(0, cfg.vocab_size, (12,), generator=g).tolist()
    dec = {1: (int(torch.randint(0, cfg.vocab_size, (1,), generator=g)), 20), 2: (5, 9), 3: (6, 33), 4: (7, 1), 5: (8, 47)}
    mb_rows = [[(0, t, p) for p, t in enumerate(prompt)] + [(r, *dec[r]) for r in (1, 2)] + [(7, 0, 0)] * 2,
               [(r, *dec[r]) for r in (3, 4, 5)]]
    for m, rows in enumerate(mb_rows):
        T = len(rows)
        attn.set_active(m, T)
        d = attn.mb[m]
        d["ids"][:T] = torch.tensor([t for _, t, _ in rows], dtype=torch.int32)
        d["positions"][:T] = torch.tensor([p for _, _, p in rows], dtype=torch.int32)
        d["ctx_len"][:T] = torch.tensor([p + 1 for _, _, p in rows], dtype=torch.int32)
        d["bt_row"][:T] = torch.tensor([r for r, _, _ in rows], dtype=torch.int32)
        d["slots"][:T] = torch.tensor([slot(r, p) for r, _, p in rows])
    for m in range(n_mb):
        attn.embed(m)
    for l in range(cfg.num_layers):
        for m in range(n_mb):
            attn.layer(l, m)
            for e in exps:
                e.layer(l, m)
    for m in range(n_mb):
        attn.head(m)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    _, lg_p = ref.prefill(i32(prompt), i32(list(range(12))), torch.tensor([slot(0, p) for p in range(12)]),
                          i32([p + 1 for p in range(12)]), i32([0] * 12), want_logits=True)
    rs = [1, 2, 3, 4, 5]
    _, lg_d = ref.decode(i32([dec[r][0] for r in rs]), i32([dec[r][1] for r in rs]),
                         torch.tensor([slot(r, dec[r][1]) for r in rs]), i32([dec[r][1] + 1 for r in rs]), i32(rs),
                         want_logits=True)
    got = {"prompt": attn.mb[0]["logits"][11], 1: attn.mb[0]["logits"][12], 2: attn.mb[0]["logits"][13],
           3: attn.mb[1]["logits"][0], 4: attn.mb[1]["logits"][1], 5: attn.mb[1]["logits"][2]}
    want = {"prompt": lg_p[11], **{r: lg_d[i] for i, r in enumerate(rs)}}
    for k in got:
        assert_close(got[k], want[k], str(k))


@pytest.mark.parametrize("A,X,n_layers,variant", [(2, 2, 4, "mixtral"), (3, 1, 5, "mixtral"), (2, 3, 4, "shared_dense")])
def test_emulated_layer_striping_pipeline(A, X, n_layers, variant):
    """Layer striping on the fused path: the A attention ranks form one pipeline over the layers (rank g holds the
    weights and the KV cache of its block of layers only); the residual rows of a micro-batch are handed from stage to
    stage by peer stores, the experts return a stage's last layer to the next stage, the last stage runs the LM head.
    Two iterations (every stage's epochs carry over), two micro-batches, against the colocated executor."""
    cfg, sd, skew = _model(variant, n_layers)
    n_mb, B = 2, 4
    shape = DisaggShape(A, X, n_mb, B, cfg.top_k, cfg.hidden_size, cfg.num_experts, stripes=A, num_layers=n_layers)
    layout = build_layout(shape)
    arenas = PeerArena.emulated(A + X, layout.size)
    attn = [AttentionRank(cfg, shape, arenas[a], layout, a, num_blocks=64, state_dict=sd) for a in range(A)]
    exps = [ExpertRank(cfg, shape, arenas[A + x], layout, x, state_dict=sd) for x in range(X)]
    ref = FusedModelExecutor(cfg, CacheConfig(block_size=16), device="cuda", max_batch_size=B, max_prefill_tokens=B,
                             state_dict=sd, num_blocks=64, enable_cuda_graph=False)
    for layer in [x for a in attn for x in a.layers if x is not None] + list(ref.attn.values()):
        layer.set_route_skew(skew)
    assert [a.l1 - a.l0 for a in attn] == [len([l for l in range(n_layers) if shape.layer_owner(l) == g]) for g in range(A)]
    assert all(a.kv_cache.shape[0] == a.l1 - a.l0 for a in attn) and shape.layer_owner(n_layers) == A - 1
    g = torch.Generator().manual_seed(5)
    kv = torch.randn(ref.kv_cache.shape, generator=g).to(torch.bfloat16).cuda() * 0.5     # [L, 2, nb, bs, kvh, hd]
    for a in attn:
        a.kv_cache.copy_(kv[a.l0:a.l1])
    ref_kv = kv.clone()
    perm = torch.randperm(60, generator=g)
    for step in range(2):
        inputs = []
        for m in range(n_mb):
            ids = torch.randint(0, cfg.vocab_size, (B,), generator=g).int()
            ctx = torch.randint(3, 40, (B,), generator=g).int() + step
            bt = perm[m * B * 4:(m + 1) * B * 4].view(B, 4).int()
            slots = torch.tensor([int(bt[i, int(ctx[i]) // 16]) * 16 + int(ctx[i]) % 16 for i in range(B)])
            inputs.append((ids, ctx, slots, bt))
            for a in attn:      # every stage needs the positions and the block tables, the first one the ids
                a.block_tables[m * B:(m + 1) * B, :4] = bt.cuda()
                d = a.mb[m]
                d["ids"].copy_(ids); d["positions"].copy_(ctx); d["ctx_len"].copy_(ctx + 1)
                d["bt_row"].copy_(torch.arange(B, dtype=torch.int32) + m * B); d["slots"].copy_(slots)
        for a in attn:
            for m in range(n_mb):
                a.embed(m)
        # one stream, several ranks: a layer runs on its owner, then on the expert ranks, before anything waits for it
        for l in range(n_layers):
            for m in range(n_mb):
                attn[shape.layer_owner(l)].layer(l, m)
                for e in exps:
                    e.layer(l, m)
        for a in attn:
            for m in range(n_mb):
                a.head(m)
        torch.cuda.synchronize()
        assert gemm.check_status() == 0
        for m, (ids, ctx, slots, bt) in enumerate(inputs):
            ref.kv_cache.copy_(ref_kv)
            ref.block_tables[:B, :4] = bt.cuda()
            _, lg = ref.decode(ids, ctx, slots, ctx + 1, torch.arange(B, dtype=torch.int32), want_logits=True)
            # the step appended one K / V row per sequence: carry it into the next step's reference cache
            assert_close(attn[-1].mb[m]["logits"], lg, f"step {step} mb {m}")
            ref_kv.copy_(ref.kv_cache)
        # the stages' caches hold the rows the reference appended, layer block by layer block
        for a in attn:
            assert_close(a.kv_cache, ref_kv[a.l0:a.l1], f"KV cache of stage {a.a} after step {step}")
