"""Row / attention / routing kernels vs the PyTorch fp32 restatements of the same ops."""
import pytest
import torch

from disagmoe_b200.ops import functional as F
from disagmoe_b200.ops import gemm, reference

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def _close(a, b, tol=2 ** -7):
    """Every element within tol * |ref| + tol * rms(ref) (bf16 results of fp32 arithmetic are ~2^-9 relative)."""
    a, b = a.float(), b.float()
    bound = b.abs() * tol + b.pow(2).mean().sqrt() * tol
    bad = int(((a - b).abs() > bound).sum())
    assert bad == 0, f"{bad} of {b.numel()} elements off; max err {(a - b).abs().max().item():.4g}, " \
                     f"rms(ref) {b.pow(2).mean().sqrt().item():.4g}"


@pytest.mark.parametrize("T,H,P", [(5, 256, 0), (33, 4096, 2), (7, 2048, 6), (3, 8192, 1)])
def test_add_rmsnorm(T, H, P):
    torch.manual_seed(0)
    resid, w = _bf(T, H), _bf(H)
    add = _bf(T, P, H) if P else None
    new, y = F.add_rmsnorm(resid, add, w, 1e-5)
    rnew, ry = reference.add_rmsnorm(resid, [add[:, p] for p in range(P)] if P else [], w, 1e-5)
    _close(new, rnew)
    _close(y, ry)


def test_rmsnorm_no_resid():
    torch.manual_seed(0)
    add, w = _bf(9, 3, 512), _bf(512)
    new, y = F.add_rmsnorm(None, add, w, 1e-6)
    rnew, ry = reference.add_rmsnorm(None, [add[:, p] for p in range(3)], w, 1e-6)
    _close(new, rnew)
    _close(y, ry)


@pytest.mark.parametrize("n_q,n_kv,hd,theta", [(32, 8, 128, 1e6), (4, 4, 64, 1e4), (16, 16, 128, 1e4)])
def test_rope_kv_append(n_q, n_kv, hd, theta):
    torch.manual_seed(1)
    T, nb, bs = 37, 16, 16
    qkv = _bf(T, (n_q + 2 * n_kv) * hd)
    pos = torch.randint(0, 4000, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(nb * bs, device=DEV)[:T].long()
    slots[5] = -1
    kc, vc = torch.zeros(nb, bs, n_kv, hd, dtype=torch.bfloat16, device=DEV), torch.zeros(nb, bs, n_kv, hd, dtype=torch.bfloat16, device=DEV)
    q2, kc2, vc2 = qkv.clone(), kc.clone(), vc.clone()
    F.rope_kv_append(qkv, pos, slots, kc, vc, n_q, n_kv, hd, theta)
    reference.rope_kv_append(q2, pos, slots, kc2, vc2, n_q, n_kv, hd, theta)
    _close(qkv, q2)
    _close(kc, kc2)
    _close(vc, vc2)


@pytest.mark.parametrize("n_q,n_kv,hd,splits", [(32, 8, 128, 1), (32, 8, 128, 4), (4, 4, 64, 1), (16, 16, 128, 3),
                                                (8, 4, 64, 2), (16, 2, 128, 1)])
def test_paged_attention(n_q, n_kv, hd, splits):
    torch.manual_seed(2)
    T, nb, bs, maxb = 9, 64, 16, 12
    q = _bf(T, n_q * hd)
    kc, vc = _bf(nb, bs, n_kv, hd), _bf(nb, bs, n_kv, hd)
    nrows = 5
    bt = torch.stack([torch.randperm(nb, device=DEV)[:maxb] for _ in range(nrows)]).int()
    bt_row = torch.randint(0, nrows, (T,), device=DEV, dtype=torch.int32)
    ctx = torch.randint(1, maxb * bs, (T,), device=DEV, dtype=torch.int32)
    ctx[0], ctx[1] = 1, maxb * bs
    o = F.paged_attention(q, kc, vc, bt, bt_row, ctx, n_q, n_kv, hd, splits=splits)
    r = reference.paged_attention(q, kc, vc, bt, bt_row, ctx, n_q, n_kv, hd)
    _close(o, r)


@pytest.mark.parametrize("T,H,E,K,renorm,norm", [(64, 4096, 8, 2, True, True), (17, 2048, 60, 4, False, True),
                                                 (5, 256, 8, 2, True, False), (40, 2048, 64, 6, False, True)])
def test_route_and_dispatch(T, H, E, K, renorm, norm):
    torch.manual_seed(3)
    x, gw = _bf(T, H), _bf(E, H, scale=0.05)
    nw = _bf(H).abs() + 0.5 if norm else None
    buf = F.DispatchBuffers(T * K, H, E, DEV)
    y, ids, w, logits = F.route(x, nw, 1e-5, gw, K, renorm, counts=buf.counts, want_logits=True)
    ry, rids, rw, rlogits = reference.route(x, nw, 1e-5, gw, K, renorm)
    _close(y, ry)
    _close(logits, rlogits, 2 ** -6)
    # compare routing on the kernel's own logits (bf16 rounding can flip near ties)
    probs = torch.softmax(logits, -1)
    ew, eids = torch.topk(probs, K, dim=-1)
    if renorm:
        ew = ew / ew.sum(-1, keepdim=True)
    assert (eids.int() == ids).float().mean().item() > 0.98
    same = eids.int() == ids
    assert torch.allclose(w[same], ew[same], atol=1e-4)
    F.dispatch_local(y, ids, w, buf)
    torch.cuda.synchronize()
    assert gemm.check_status() == 0
    offs = buf.offs.tolist()
    assert offs == reference.expert_offsets(ids, E).tolist()
    assert int(buf.counts.sum()) == 0  # cleared for the next layer
    recs = buf.recs.cpu()
    seen = set()
    for e in range(E):
        for r in range(offs[e], offs[e + 1]):
            p = int(recs[r, 1])
            assert int(recs[r, 3]) == e and int(ids.view(-1)[p]) == e
            assert torch.equal(buf.xs[r], y[p // K])
            assert abs(recs[r, 2:3].view(torch.float32).item() - w.view(-1)[p].item()) < 1e-6
            seen.add(p)
    assert len(seen) == T * K


def test_embed_argmax_permute_gather():
    torch.manual_seed(4)
    V, H, T = 1000, 512, 50
    table = _bf(V, H)
    ids = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    assert torch.equal(F.embed(ids, table), table[ids.long()])
    logits = torch.randn(T, V, device=DEV)
    assert torch.equal(F.argmax(logits).long(), logits.argmax(-1))
    lb = logits.to(torch.bfloat16)
    am = F.argmax(lb).long()
    assert torch.equal(lb.float().gather(1, am[:, None]), lb.float().max(-1, keepdim=True).values)
    src = _bf(T, H)
    mp = torch.randperm(2 * T, device=DEV).int()
    out = F.permute_rows(src, mp, repeat=2)
    assert torch.equal(out, reference.permute_rows(src, mp, repeat=2))
    g = torch.randint(0, T, (77,), device=DEV, dtype=torch.int32)
    assert torch.equal(F.permute_rows(src, g, gather=True), src[g.long()])
    ptrs = torch.tensor([src[i].data_ptr() for i in g.tolist()], dtype=torch.int64, device=DEV)
    o2 = torch.empty(77, H, dtype=torch.bfloat16, device=DEV)
    assert torch.equal(F.gather_ptrs(ptrs, 77, H, o2), src[g.long()])


def test_flag_wait_gives_up_with_status_and_context_survives():
    """A wait on a flag that nothing sets runs out after its cycle budget, records kStatusFlagTimeout in the status
    word and returns; the context stays usable and later waits of the poisoned run return at once."""
    import ctypes
    import time
    from disagmoe_b200.ops import _lib
    lib = _lib.lib()
    lib.dmoe_set_flag_wait_cycles.argtypes = [ctypes.c_longlong]
    lib.dmoe_set_flag_wait_cycles(ctypes.c_longlong(200_000_000))       # ~0.1 s
    try:
        s = gemm.scratch("cuda")
        s.status.zero_()
        flags = torch.zeros(4, dtype=torch.int32, device=DEV)
        epoch = torch.zeros(1, dtype=torch.int32, device=DEV)
        vp = lambda t: ctypes.c_void_p(t.data_ptr())
        call = lambda: lib.dmoe_wait_flags(vp(flags), ctypes.c_int(4), vp(epoch), vp(s.status),
                                           ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        t0 = time.time()
        assert call() == 0
        torch.cuda.synchronize()
        assert time.time() - t0 < 3.0
        assert int(s.status.item()) == 2 and int(epoch.item()) == 1
        t0 = time.time()
        assert call() == 0                  # poisoned: no second wait
        torch.cuda.synchronize()
        assert time.time() - t0 < 0.05
        assert gemm.check_status() == 2     # read and cleared
        flags.fill_(3)
        assert call() == 0                  # flags already carry the epoch: passes without waiting
        torch.cuda.synchronize()
        assert gemm.check_status() == 0 and int(epoch.item()) == 3
        assert torch.allclose(torch.ones(4, device=DEV) * 2, torch.full((4,), 2.0, device=DEV))   # context still fine
    finally:
        lib.dmoe_set_flag_wait_cycles(ctypes.c_longlong(0))


def _ptrs(ts):
    return torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=DEV)


@pytest.mark.parametrize("T,H,P,n_dst", [(33, 4096, 2, 4), (5, 256, 0, 1), (0, 2048, 2, 2)])
def test_norm_gather_pushes_rows_waits_and_signals(T, H, P, n_dst):
    """add + RMSNorm with the normalised rows stored into several destination buffers at a row offset (the all-gather
    push of a TP group, emulated on one GPU), behind a wait on flags that are already set, followed by the release of
    one flag per destination; an empty shard (T = 0) still takes part in the hand-shake."""
    torch.manual_seed(10)
    row0, rows = 7, 64
    resid, w = _bf(max(T, 1), H)[:T], _bf(H)
    add = _bf(max(T, 1), max(P, 1), H)[:T] if P else None
    dsts = [torch.zeros(rows, H, dtype=torch.bfloat16, device=DEV) for _ in range(n_dst)]
    sflags = [torch.zeros(3, dtype=torch.int32, device=DEV) for _ in range(n_dst)]
    wflags = torch.full((5,), 4, dtype=torch.int32, device=DEV)
    z = lambda v=0: torch.full((1,), v, dtype=torch.int32, device=DEV)
    wait_epoch, sig_epoch, status = z(3), z(8), z()
    out = torch.zeros(max(T, 1), H, dtype=torch.bfloat16, device=DEV)[:T]
    F.norm_gather(resid, add, w, 1e-5, out if P else None, _ptrs(dsts), n_dst, row0, H, T, H, wait_flags=wflags,
                  n_wait=5, wait_epoch=wait_epoch, signal_ptrs=_ptrs(sflags), n_signal=n_dst, signal_slot=1,
                  signal_epoch=sig_epoch, ticket=z(), status=status)
    torch.cuda.synchronize()
    assert int(status) == 0 and int(wait_epoch) == 4 and int(sig_epoch) == 9
    assert all(f.tolist() == [0, 9, 0] for f in sflags)
    if T:
        rnew, ry = reference.add_rmsnorm(resid, [add[:, p] for p in range(P)] if P else [], w, 1e-5)
        if P:
            _close(out, rnew)
        for d in dsts:
            _close(d[row0:row0 + T], ry)
            assert float(d[:row0].abs().max()) == 0.0 and float(d[row0 + T:].abs().max()) == 0.0


@pytest.mark.parametrize("T,H,E,K,renorm,n_dst,n_add", [(64, 4096, 8, 2, True, 4, 0), (17, 2048, 60, 4, False, 6, 4),
                                                        (40, 2048, 64, 6, False, 3, 2), (0, 256, 8, 2, True, 2, 2)])
def test_route_dispatch_single_kernel(T, H, E, K, renorm, n_dst, n_add):
    """One launch: [reduce the TP partial slots into the residual] -> RMSNorm -> gate -> top-k -> per-pair row
    reservation in the expert's region of the owning "GPU" (buffers on this GPU) -> rows + records -> flags.
    Checked against the separate router kernel (same arithmetic) and by reading back every region."""
    torch.manual_seed(11)
    epr = (E + n_dst - 1) // n_dst
    if (n_dst - 1) * epr >= E:
        pytest.skip("an expert GPU would hold no expert")
    cap, my_rank, n_src = max(T * K, 1), 1, 3
    rows_cap = max(T, 1) + 3
    resid = _bf(rows_cap, H)
    resid0 = resid.clone()
    add = _bf(max(n_add, 1), rows_cap, H, scale=0.3)
    nw, gw = _bf(H).abs() + 0.5, _bf(E, H, scale=0.05)
    xs = [torch.zeros(epr * cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(n_dst)]
    recs = [torch.full((epr * cap, 4), -7, dtype=torch.int32, device=DEV) for _ in range(n_dst)]
    cnts = [torch.zeros(epr, dtype=torch.int32, device=DEV) for _ in range(n_dst)]
    flags = [torch.zeros(n_src, dtype=torch.int32, device=DEV) for _ in range(n_dst)]
    z = lambda v=0: torch.full((1,), v, dtype=torch.int32, device=DEV)
    disp_epoch, wait_epoch, status = z(5), z(2), z()
    oflags = torch.full((max(n_add, 1),), 3, dtype=torch.int32, device=DEV)
    y = torch.zeros(rows_cap, H, dtype=torch.bfloat16, device=DEV)
    ids = torch.zeros(rows_cap, K, dtype=torch.int32, device=DEV)
    wts = torch.zeros(rows_cap, K, dtype=torch.float32, device=DEV)
    kw = dict(add=add, n_add=n_add, add_slot_stride=rows_cap * H, ld_add=H, wait_flags=oflags, n_wait=n_add,
              wait_epoch=wait_epoch) if n_add else {}
    F.route_dispatch(resid, nw, 1e-5, gw, K, renorm, T, y=y, topk_ids=ids, topk_w=wts, x_bases=_ptrs(xs),
                     rec_bases=_ptrs(recs), cnt_bases=_ptrs(cnts), flag_bases=_ptrs(flags), ld_dst=H,
                     experts_per_rank=epr, n_dst=n_dst, my_rank=my_rank, region_cap=cap, disp_epoch=disp_epoch,
                     ticket=z(), status=status, **kw)
    torch.cuda.synchronize()
    assert int(status) == 0 and int(disp_epoch) == 6
    assert all(f.tolist() == [0, 6, 0] for f in flags)
    if n_add:
        assert int(wait_epoch) == 3
    if T == 0:
        assert all(int(c.sum()) == 0 for c in cnts)
        return
    # the reduced residual: ordered fp32 sum rounded once to bf16
    want_resid = resid0[:T].float()
    for s in range(n_add):
        want_resid = want_resid + add[s, :T].float()
    want_resid = want_resid.to(torch.bfloat16)
    if n_add:
        assert torch.equal(resid[:T], want_resid)
    assert torch.equal(resid[T:], resid0[T:])
    y2, ids2, w2, _ = F.route(want_resid, nw, 1e-5, gw, K, renorm)
    torch.cuda.synchronize()
    assert torch.equal(y[:T], y2) and torch.equal(ids[:T], ids2)
    assert torch.allclose(wts[:T], w2, atol=1e-6)
    seen = set()
    hist = torch.bincount(ids2.view(-1).long(), minlength=E).tolist()
    for d in range(n_dst):
        cnt = cnts[d].tolist()
        rc = recs[d].cpu()
        for le in range(epr):
            e = d * epr + le
            if e >= E:
                assert cnt[le] == 0
                continue
            assert cnt[le] == hist[e]
            for r in range(le * cap, le * cap + cnt[le]):
                p = int(rc[r, 1])
                assert int(rc[r, 0]) == my_rank and int(rc[r, 3]) == e and int(ids2.view(-1)[p]) == e
                assert torch.equal(xs[d][r], y2[p // K])
                assert abs(rc[r, 2:3].view(torch.float32).item() - w2.view(-1)[p].item()) < 1e-6
                seen.add(p)
            assert bool((rc[le * cap + cnt[le]:(le + 1) * cap, 1] == -7).all())      # the rest of the region is untouched
    assert len(seen) == T * K


def test_route_dispatch_without_gate_reduces_and_normalises_only():
    """A layer with a dense FFN has no router: the kernel sums the partial slots into the residual and writes the
    normalised rows; nothing is dispatched."""
    torch.manual_seed(12)
    T, H, tp = 9, 512, 2
    resid, add, nw = _bf(T, H), _bf(tp, T, H), _bf(H).abs() + 0.5
    r0 = resid.clone()
    y = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
    z = lambda v=0: torch.full((1,), v, dtype=torch.int32, device=DEV)
    of, we = torch.ones(tp, dtype=torch.int32, device=DEV), z()
    F.route_dispatch(resid, nw, 1e-5, None, 2, True, T, add=add, n_add=tp, add_slot_stride=T * H, ld_add=H, y=y,
                     wait_flags=of, n_wait=tp, wait_epoch=we, ticket=z(), status=z())
    torch.cuda.synchronize()
    want = (r0.float() + add[0].float() + add[1].float()).to(torch.bfloat16)
    assert torch.equal(resid, want) and int(we) == 1
    _, ry = reference.add_rmsnorm(want, [], nw, 1e-5)
    _close(y, ry)


def test_ids_gather():
    src = torch.arange(10, dtype=torch.int32, device=DEV) + 100
    dsts = [torch.zeros(32, dtype=torch.int32, device=DEV) for _ in range(3)]
    flags = [torch.zeros(4, dtype=torch.int32, device=DEV) for _ in range(3)]
    ep = torch.full((1,), 6, dtype=torch.int32, device=DEV)
    F.ids_gather(src, 10, _ptrs(dsts), 3, 8, _ptrs(flags), 2, ep)
    torch.cuda.synchronize()
    for d, f in zip(dsts, flags):
        assert d[8:18].tolist() == list(range(100, 110)) and int(d.sum()) == sum(range(100, 110))
        assert f.tolist() == [0, 0, 7, 0]
    assert int(ep) == 7


@pytest.mark.parametrize("n_q,n_kv,hd", [(32, 8, 128), (4, 4, 64), (16, 2, 128), (8, 4, 64), (2, 2, 128)])
def test_prefill_attention_tiled_causal(n_q, n_kv, hd):
    """The tiled causal kernel on a mixed batch: whole prompts of 1 ... 300 tokens, a chunk that continues a cached
    prefix (chunked prefill), short runs and decode rows that stay with the per-token kernel. Reference: the fp32
    restatement of paged attention with ctx_len = position + 1 for every row."""
    torch.manual_seed(20)
    bs, maxb = 16, 40
    segs = [(0, 0, 300), (1, 0, 64), (2, 137, 70), (3, 500, 1), (4, 0, 5), (5, 90, 1), (6, 0, 17), (7, 31, 129)]   # (bt row, first pos, tokens)
    rows, pos = [], []
    for r, p0, n in segs:
        rows += [r] * n
        pos += list(range(p0, p0 + n))
    T = len(rows)
    nb = 8 * maxb
    q = _bf(T, n_q * hd)
    kc, vc = _bf(nb, bs, n_kv, hd), _bf(nb, bs, n_kv, hd)
    bt = torch.randperm(nb, device=DEV)[:8 * maxb].view(8, maxb).int()
    bt_row = torch.tensor(rows, dtype=torch.int32, device=DEV)
    ctx = torch.tensor([p + 1 for p in pos], dtype=torch.int32, device=DEV)
    tiles, covered = F.build_prefill_tiles(rows, pos, F.prefill_tile_tokens(n_q, n_kv))
    assert int(covered.sum()) == 300 + 64 + 70 + 17 + 129 and not covered[434:435].any()      # runs of 1 and 5 rows stay
    ctx_dec = ctx.clone()
    ctx_dec[covered.to(DEV)] = 0
    out = F.paged_attention(q, kc, vc, bt, bt_row, ctx_dec, n_q, n_kv, hd)
    F.prefill_attention(q, kc, vc, bt, tiles.to(DEV), len(tiles), n_q, n_kv, hd, out)
    ref = reference.paged_attention(q, kc, vc, bt, bt_row, ctx, n_q, n_kv, hd)
    torch.cuda.synchronize()
    # probabilities are rounded to bf16 before P V and the output once more: a handful of elements in millions land two
    # bf16 steps from the fp32 reference
    _close(out, ref, tol=2 ** -6)
    # and the per-token kernel agrees with both (it is what the tiled kernel replaces for these rows)
    _close(F.paged_attention(q, kc, vc, bt, bt_row, ctx, n_q, n_kv, hd), ref, tol=2 ** -6)


def test_debug_add_one_kernel_and_multi_launch():
    """The debug kernel of the launch / overlap experiments, and the native module's test that chains hundreds of its
    launches on two streams at once (counterpart of the reference's test_multi_launch)."""
    import ctypes
    from disagmoe_b200 import disagmoe_c as C
    from disagmoe_b200.ops import _lib
    x = torch.randn(1000, device=DEV)
    y = torch.empty_like(x)
    rc = _lib.lib().dmoe_add_one(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr()), ctypes.c_longlong(1000),
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(y, x + 1)
    assert C.test_multi_launch(0, 300, 4096)
