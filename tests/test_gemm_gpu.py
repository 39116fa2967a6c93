"""tcgen05 GEMM kernel vs a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

from disagmoe_b200.ops import gemm

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["streamk", "whole_tiles"], autouse=True)
def work_distribution(request):
    """Every test of this file runs twice: with the stream-K distribution (the default: equal shares of K-block
    iterations per SM, partial tiles reduced through the workspace) and with whole tiles per CTA."""
    old = gemm.STREAM_K
    gemm.STREAM_K = request.param == "streamk"
    yield request.param
    gemm.STREAM_K = old


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _close(y, ref, tol=2 ** -7):
    """Every element within tol * |ref| + tol * rms(ref): a bf16 result of an fp32 accumulation is off by at most
    2^-9 relative, so a dropped K block or a wrong row shows up even where the reference is small."""
    y, ref = y.float(), ref.float()
    bound = ref.abs() * tol + ref.pow(2).mean().sqrt() * tol
    bad = int(((y - ref).abs() > bound).sum())
    assert bad == 0, f"{bad} of {ref.numel()} elements off; max err {(y - ref).abs().max().item():.4g}, " \
                     f"rms(ref) {ref.pow(2).mean().sqrt().item():.4g}"


@pytest.mark.parametrize("T,F,K,bn,splitk", [
    (7, 128, 64, 32, 1), (64, 256, 256, 64, 1), (200, 384, 512, 128, 1), (300, 256, 1024, 256, 1),
    (33, 512, 4096, 32, 4), (256, 6144, 4096, 0, 0), (16, 1024, 256, 0, 0), (130, 256, 200, 64, 2),
    (256, 4096, 14336, 256, 1),        # GEMM-2 shape of a Mixtral expert (K = 14336) at the widest token tile
    (96, 1024, 4096 + 64 + 8, 64, 5),  # split-K whose last split ends in a partial K block
])
def test_linear(T, F, K, bn, splitk):
    torch.manual_seed(0)
    x, w = _rand(T, K), _rand(F, K, scale=K ** -0.5)
    y = gemm.linear(x, w, bn=bn, splitk=splitk)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    _close(y, x.float() @ w.float().T)


def test_linear_residual_and_f32_out():
    torch.manual_seed(1)
    x, w, r = _rand(96, 512), _rand(256, 512, scale=0.05), _rand(96, 256)
    y = gemm.linear(x, w, residual=r)
    y32 = gemm.linear(x, w, out_dtype=torch.float32)
    torch.cuda.synchronize()
    ref = x.float() @ w.float().T
    _close(y, ref + r.float())
    _close(y32, ref, tol=2 ** -12)


def _offsets(counts):
    return torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("counts,I,K,bn", [
    ([5, 0, 40, 3], 128, 256, 32), ([64] * 8, 256, 512, 64), ([100, 7, 0, 0, 200, 1, 33, 64], 384, 256, 128),
    ([31, 33], 1408, 2048, 0),
])
def test_grouped_swiglu(counts, I, K, bn):
    torch.manual_seed(2)
    G, T = len(counts), sum(counts)
    x, w13 = _rand(T, K), _rand(G, 2 * I, K, scale=K ** -0.5)
    offs = _offsets(counts)
    y = gemm.grouped_swiglu(x, w13, offs, bn=bn, streamk=gemm.STREAM_K)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    _close(y, gemm._grouped_ref(x, w13, offs, True))


@pytest.mark.parametrize("counts,F,K,bn", [([5, 0, 40, 3], 256, 128, 32), ([64] * 8, 512, 1024, 64),
                                            ([300, 20], 256, 512, 256)])
def test_grouped_linear(counts, F, K, bn):
    torch.manual_seed(3)
    G, T = len(counts), sum(counts)
    x, w = _rand(T, K), _rand(G, F, K, scale=K ** -0.5)
    offs = _offsets(counts)
    y = gemm.grouped_linear(x, w, offs, bn=bn, streamk=gemm.STREAM_K)
    torch.cuda.synchronize()
    _close(y, gemm._grouped_ref(x, w, offs, False))


def test_grouped_combine_scatter():
    torch.manual_seed(4)
    counts, F, K = [10, 0, 25, 7], 256, 512
    G, T = len(counts), sum(counts)
    x, w = _rand(T, K), _rand(G, F, K, scale=K ** -0.5)
    offs = _offsets(counts)
    perm = torch.randperm(T, device="cuda")
    wts = torch.rand(T, device="cuda")
    recs = torch.zeros(T, 4, dtype=torch.int32, device="cuda")
    recs[:, 1] = perm.int()
    recs[:, 2] = wts.view(torch.int32)
    recs[3, 1] = -1  # dropped row
    out = torch.zeros(T, F, dtype=torch.bfloat16, device="cuda")
    bases = torch.tensor([out.data_ptr()], dtype=torch.int64, device="cuda")
    gemm.grouped_combine(x, w, offs, recs, bases, out.stride(0))
    torch.cuda.synchronize()
    ref = gemm._grouped_ref(x, w, offs, False) * wts[:, None]
    exp = torch.zeros(T, F, device="cuda")
    keep = recs[:, 1] >= 0
    exp[perm[keep]] = ref[keep]
    _close(out, exp)


def test_grouped_real_expert_shapes_bn256_and_empty_groups():
    """Mixtral expert shapes (H 4096, I 14336, 8 groups) with ragged, partly empty groups: SwiGLU up-projection at its
    widest tile and the down-projection at BN = 256."""
    torch.manual_seed(5)
    counts = [256, 0, 31, 300, 1, 0, 129, 64]
    G, T, H, I = len(counts), sum(counts), 4096, 14336
    x = _rand(T, H)
    w13 = _rand(G, 2 * I, H, scale=H ** -0.5)
    offs = _offsets(counts)
    act = gemm.grouped_swiglu(x, w13, offs, bn=128, streamk=gemm.STREAM_K)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    _close(act, gemm._grouped_ref(x, w13, offs, True))
    del w13
    w2 = _rand(G, H, I, scale=I ** -0.5)
    y = gemm.grouped_linear(act, w2, offs, bn=256, streamk=gemm.STREAM_K)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    _close(y, gemm._grouped_ref(act, w2, offs, False))


def test_grouped_multi_source_segments():
    """Expert-side input as the dispatch leaves it: S senders each packed their rows for the G groups into their own
    region (seg_cnt [S, G]); groups with no rows from some or all senders included."""
    torch.manual_seed(6)
    S, G, K, I, cap = 3, 4, 512, 256, 96
    cnt = torch.tensor([[10, 0, 33, 5], [0, 0, 64, 1], [7, 0, 0, 20]], dtype=torch.int32)
    x = _rand(S * cap, K)
    w13 = _rand(G, 2 * I, K, scale=K ** -0.5)
    out = torch.zeros(S * cap, I, dtype=torch.bfloat16, device="cuda")
    comm = gemm.GemmComm(seg_cnt=cnt.cuda(), S=S, seg_cap=cap)
    gemm.grouped_swiglu(x, w13, None, out=out, bn=32, comm=comm)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    for s in range(S):
        row = s * cap
        for g in range(G):
            n = int(cnt[s, g])
            if n:
                h = x[row:row + n].float() @ w13[g].float().T
                _close(out[row:row + n], torch.nn.functional.silu(h[:, :I]) * h[:, I:])
            row += n


@pytest.mark.parametrize("n_q,n_kv,hd,T,theta", [(8, 2, 128, 300, 1e6), (4, 4, 64, 77, 1e4), (2, 1, 64, 33, 1e4)])
def test_qkv_gemm_with_rope_and_kv_append_epilogue(n_q, n_kv, hd, T, theta):
    """The QKV GEMM whose epilogue rotates q / k and appends K / V to the paged cache, against the plain GEMM followed by
    the stand-alone RoPE + append kernel (same arithmetic, so the bf16 results agree to the last bit or nearly so), and
    against the fp32 reference of both ops."""
    from disagmoe_b200.ops import functional as F, reference
    torch.manual_seed(7)
    K, Fq = 512, (n_q + 2 * n_kv) * hd
    nb, bs = (T + 15) // 16 + 2, 16
    x, w = _rand(T, K), _rand(Fq, K, scale=K ** -0.5)
    pos = torch.randint(0, 4000, (T,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(nb * bs, device="cuda")[:T].long()
    slots[3] = -1
    mk = lambda: torch.zeros(nb, bs, n_kv, hd, dtype=torch.bfloat16, device="cuda")
    kc, vc, kc2, vc2 = mk(), mk(), mk(), mk()
    table = gemm.rope_table(4096, hd, theta, "cuda")
    rope = gemm.RopeAppend(table, pos, slots, kc, vc, n_q, n_kv, hd)
    for splitk in (1, 3):
        kc.zero_(); vc.zero_()
        qkv = gemm.linear(x, w, comm=gemm.GemmComm(rope=rope), splitk=splitk)
        ref = gemm.linear(x, w, splitk=splitk)
        F.rope_kv_append(ref, pos, slots, kc2, vc2, n_q, n_kv, hd, theta)
        torch.cuda.synchronize()
        assert gemm.check_status() == 0
        q = n_q * hd
        _close(qkv[:, :q], ref[:, :q], tol=2 ** -9)
        _close(kc, kc2, tol=2 ** -9)
        _close(vc, vc2, tol=2 ** -9)
    exact = (x.float() @ w.float().T).to(torch.bfloat16)
    kc3, vc3 = mk(), mk()
    reference.rope_kv_append(exact, pos, slots, kc3, vc3, n_q, n_kv, hd, theta)
    _close(qkv[:, :n_q * hd], exact[:, :n_q * hd])
    _close(kc, kc3)
    _close(vc, vc3)


def test_oproj_reduce_scatter_epilogue_and_shard_gated_prologue():
    """Tensor-parallel hooks of the dense GEMM on one GPU: (a) the reduce-scatter epilogue stores row t into slot
    rs_slot of the buffer of rank t // rs_rows and releases the peers' flags; (b) a GEMM whose X arrives in shards
    fetches token tiles only behind the shards' flags, and reports a timeout (status 2) instead of hanging when a
    shard's flag never comes."""
    from disagmoe_b200.ops import _lib
    torch.manual_seed(8)
    tp, T, K, Fo, per, cap = 4, 150, 256, 384, 40, 48      # shards of 40, 40, 40, 30 rows
    x, w = _rand(T, K), _rand(Fo, K, scale=K ** -0.5)
    bufs = [torch.zeros(tp, cap, Fo, dtype=torch.bfloat16, device="cuda") for _ in range(tp)]
    flags = [torch.zeros(tp, dtype=torch.int32, device="cuda") for _ in range(tp)]
    i64 = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device="cuda")
    z = lambda: torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = x.float() @ w.float().T
    for slot in (2, 0):
        comm = gemm.GemmComm(rs_bases=i64(bufs), rs_rows=per, rs_slot=slot, rs_cap=cap, signal_ptrs=i64(flags),
                             n_signal=tp, signal_slot=slot, signal_epoch=z(), done_ticket=z())
        gemm.linear(x, w, comm=comm, splitk=2 if slot == 0 else 1)
        torch.cuda.synchronize()
        for r in range(tp):
            lo, hi = r * per, min(T, (r + 1) * per)
            _close(bufs[r][slot, :hi - lo], ref[lo:hi])
            assert float(bufs[r][slot, hi - lo:].abs().max()) == 0.0     # nothing beyond the shard's rows
            assert int(flags[r][slot]) == 1
    # (b) shard-gated prologue: all flags at epoch 1 -> result as usual, epoch advanced
    sflags, epoch = torch.ones(tp, dtype=torch.int32, device="cuda"), z()
    y = gemm.linear(x, w, comm=gemm.GemmComm(shard_rows=per, wait_flags=sflags, n_wait=tp, wait_epoch=epoch,
                                             done_ticket=z()), bn=64)
    torch.cuda.synchronize()
    _close(y, ref)
    assert int(epoch) == 1 and gemm.check_status() == 0
    # shard 3's flag stays behind: the wait runs out (about 0.05 s), the kernel returns, the status word says so
    sflags[:3] = 2
    _lib.lib().dmoe_set_flag_wait_cycles(100_000_000)
    try:
        gemm.linear(x, w, comm=gemm.GemmComm(shard_rows=per, wait_flags=sflags, n_wait=tp, wait_epoch=epoch,
                                             done_ticket=z()), bn=64)
        torch.cuda.synchronize()
    finally:
        _lib.lib().dmoe_set_flag_wait_cycles(0)
    assert gemm.check_status() == 2
    y2 = gemm.linear(x, w)            # the context is intact
    torch.cuda.synchronize()
    _close(y2, ref)


@pytest.mark.parametrize("T,F,K", [(256, 6144, 4096), (64, 4096, 4096), (1024, 1536, 4096), (300, 384, 14336),
                                   (17, 128, 64), (512, 32000, 4096)])
def test_stream_k_linear_shapes(T, F, K, work_distribution):
    """Decode-size and TP-size dense GEMMs of the model (QKV, o_proj, LM head) with automatic tile and distribution:
    few tiles with long K loops (every tile shared by several CTAs) and many tiles (a boundary in every other tile)."""
    torch.manual_seed(9)
    x, w = _rand(T, K), _rand(F, K, scale=K ** -0.5)
    r = _rand(T, F)
    y = gemm.linear(x, w, residual=r)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    _close(y, x.float() @ w.float().T + r.float())
    y2 = gemm.linear(x, w, residual=r)       # the tile counters must be back at zero
    torch.cuda.synchronize()
    assert torch.equal(y, y2)


def test_stream_k_combine_matches_whole_tiles():
    """GEMM-2 with the combine epilogue (scaled scatter through records) at a shape where most tiles are shared
    between CTAs under stream-K: same result as with whole tiles."""
    torch.manual_seed(10)
    counts, F, K = [260, 250, 3, 0, 515], 512, 14336
    G, T = len(counts), sum(counts)
    x, w = _rand(T, K), _rand(G, F, K, scale=K ** -0.5)
    offs = _offsets(counts)
    perm = torch.randperm(T, device="cuda")
    wts = torch.rand(T, device="cuda")
    recs = torch.zeros(T, 4, dtype=torch.int32, device="cuda")
    recs[:, 1] = perm.int()
    recs[:, 2] = wts.view(torch.int32)
    outs = []
    for sk in (True, False):
        out = torch.zeros(T, F, dtype=torch.bfloat16, device="cuda")
        bases = torch.tensor([out.data_ptr()], dtype=torch.int64, device="cuda")
        gemm.grouped_combine(x, w, offs, recs, bases, out.stride(0), bn=256, streamk=sk)
        torch.cuda.synchronize()
        assert gemm.check_status() == 0
        outs.append(out)
    ref = gemm._grouped_ref(x, w, offs, False) * wts[:, None]
    exp = torch.zeros(T, F, device="cuda")
    exp[perm] = ref
    _close(outs[0], exp)
    _close(outs[1], exp)


@pytest.mark.parametrize("T,F,K,bn", [(256, 512, 512, 256), (100, 256, 256, 128), (300, 384, 1024, 256), (37, 128, 64, 128),
                                      (512, 6144, 4096, 256)])
def test_cta_pair_linear(T, F, K, bn):
    """Dense GEMM on CTA pairs (tcgen05.mma.cta_group::2: 256 weight rows per MMA, the token tile split between the two
    CTAs' shared memories): full and ragged token tiles, an odd number of 128-row weight tiles (F = 384: the second CTA
    of the last pair has no rows), residual add."""
    torch.manual_seed(11)
    x, w, r = _rand(T, K), _rand(F, K, scale=K ** -0.5), _rand(T, F)
    y = gemm.linear(x, w, residual=r, bn=bn, pair=True)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    _close(y, x.float() @ w.float().T + r.float())


@pytest.mark.parametrize("counts,I,K,bn", [([200, 0, 256, 31], 256, 512, 256), ([64] * 4, 384, 256, 128),
                                            ([255, 260], 1408, 2048, 256)])
def test_cta_pair_grouped_swiglu_and_combine(counts, I, K, bn):
    """Expert GEMMs on CTA pairs: SwiGLU up-projection with gate and up accumulators for 256 tokens filling TMEM
    (single-buffered), and the down-projection with the combine epilogue."""
    torch.manual_seed(12)
    G, T = len(counts), sum(counts)
    x, w13 = _rand(T, K), _rand(G, 2 * I, K, scale=K ** -0.5)
    offs = _offsets(counts)
    act = gemm.grouped_swiglu(x, w13, offs, bn=bn, pair=True)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    ref_act = gemm._grouped_ref(x, w13, offs, True)
    _close(act, ref_act)
    F = 256
    w2 = _rand(G, F, I, scale=I ** -0.5)
    perm = torch.randperm(T, device="cuda")
    wts = torch.rand(T, device="cuda")
    recs = torch.zeros(T, 4, dtype=torch.int32, device="cuda")
    recs[:, 1] = perm.int()
    recs[:, 2] = wts.view(torch.int32)
    out = torch.zeros(T, F, dtype=torch.bfloat16, device="cuda")
    bases = torch.tensor([out.data_ptr()], dtype=torch.int64, device="cuda")
    gemm.grouped_combine(act, w2, offs, recs, bases, out.stride(0), bn=bn, pair=True)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    exp = torch.zeros(T, F, device="cuda")
    exp[perm] = gemm._grouped_ref(act, w2, offs, False) * wts[:, None]
    _close(out, exp)


@pytest.mark.parametrize("counts,I,K,bn", [([64] * 8, 256, 512, 64), ([100, 7, 0, 0, 200, 1, 33, 64], 384, 256, 128),
                                            ([31, 300], 1408, 2048, 0)])
def test_blocked_weight_layout_swiglu_linear_and_combine(counts, I, K, bn):
    """Weights stored tile by tile (every 128 x 64 box contiguous) give the same results as the row-major stack: the
    SwiGLU up-projection (gate and up tiles of the fused stack), the grouped down-projection, and the combine epilogue."""
    torch.manual_seed(9)
    G, T = len(counts), sum(counts)
    x, w13 = _rand(T, K), _rand(G, 2 * I, K, scale=K ** -0.5)
    offs = _offsets(counts)
    act = gemm.grouped_swiglu(x, gemm.block_weight(w13), offs, bn=bn, streamk=gemm.STREAM_K, w_blocked=True)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    _close(act, gemm._grouped_ref(x, w13, offs, True))
    F2 = 256
    w2 = _rand(G, F2, I, scale=I ** -0.5)
    y = gemm.grouped_linear(act, gemm.block_weight(w2), offs, bn=bn, streamk=gemm.STREAM_K, w_blocked=True)
    ref = gemm._grouped_ref(act, w2, offs, False)
    _close(y, ref)
    wts = torch.rand(T, device="cuda")
    recs = torch.zeros(T, 4, dtype=torch.int32, device="cuda")
    perm = torch.randperm(T, device="cuda")
    recs[:, 1] = perm.int()
    recs[:, 2] = wts.view(torch.int32)
    out = torch.zeros(T, F2, dtype=torch.bfloat16, device="cuda")
    bases = torch.tensor([out.data_ptr()], dtype=torch.int64, device="cuda")
    gemm.grouped_combine(act, gemm.block_weight(w2), offs, recs, bases, out.stride(0), bn=bn, streamk=gemm.STREAM_K,
                         w_blocked=True)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    exp = torch.zeros(T, F2, device="cuda")
    exp[perm] = ref.float() * wts[:, None]
    _close(out, exp)
