"""Row / attention / routing kernels vs the PyTorch fp32 restatements of the same ops."""
import pytest
import torch

from disagmoe_b200.ops import functional as F
from disagmoe_b200.ops import gemm, reference

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def _close(a, b, tol=2e-2):
    err = (a.float() - b.float()).abs().max().item()
    mag = b.float().abs().max().item() + 1e-6
    assert err / mag < tol, f"max err {err} vs {mag}"


@pytest.mark.parametrize("T,H,P", [(5, 256, 0), (33, 4096, 2), (7, 2048, 6), (3, 8192, 1)])
def test_add_rmsnorm(T, H, P):
    torch.manual_seed(0)
    resid, w = _bf(T, H), _bf(H)
    add = _bf(T, P, H) if P else None
    new, y = F.add_rmsnorm(resid, add, w, 1e-5)
    rnew, ry = reference.add_rmsnorm(resid, [add[:, p] for p in range(P)] if P else [], w, 1e-5)
    _close(new, rnew, 1e-2)
    _close(y, ry)


def test_rmsnorm_no_resid():
    torch.manual_seed(0)
    add, w = _bf(9, 3, 512), _bf(512)
    new, y = F.add_rmsnorm(None, add, w, 1e-6)
    rnew, ry = reference.add_rmsnorm(None, [add[:, p] for p in range(3)], w, 1e-6)
    _close(new, rnew, 1e-2)
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
    _close(logits, rlogits, 3e-2)
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
