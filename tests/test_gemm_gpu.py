"""tcgen05 GEMM kernel vs a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

from disagmoe_b200.ops import gemm

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _close(y, ref, tol=2e-2):
    err = (y.float() - ref).abs().max().item()
    mag = ref.abs().max().item() + 1e-6
    assert err / mag < tol, f"max err {err} vs magnitude {mag}"


@pytest.mark.parametrize("T,F,K,bn,splitk", [
    (7, 128, 64, 32, 1), (64, 256, 256, 64, 1), (200, 384, 512, 128, 1), (300, 256, 1024, 256, 1),
    (33, 512, 4096, 32, 4), (256, 6144, 4096, 0, 0), (16, 1024, 256, 0, 0), (130, 256, 200, 64, 2),
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
    _close(y32, ref, tol=1e-3)


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
    y = gemm.grouped_swiglu(x, w13, offs, bn=bn)
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
    y = gemm.grouped_linear(x, w, offs, bn=bn)
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
