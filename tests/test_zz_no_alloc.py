"""The allocation-free GEMM entry point (``dmoe_linear_noalloc``, declared in csrc/kernels/dmoe_noalloc.h).

Some users of the kernel library cannot allocate device memory when they need a GEMM: an engine that has already
given all free HBM to its KV cache, or a runtime helper thread that must not call cudaMalloc (it synchronises the
device) or touch the framework's allocator. For them the library keeps the split-K scratch in a built-in device
array. This test calls the entry point through its exported C symbol, twice in a row (the second call reuses the
array with the first call's leftovers in it), and checks the result against the regular entry point
(``disagmoe_b200.ops.gemm.linear``) within the tolerance the other GEMM tests use. It also checks that an oversized
problem is refused with a readable message. The file sorts last so that a ``-x`` run has finished every other test
before this one starts; it passes on its own in a fresh process as well.
"""
import ctypes

import pytest
import torch

from disagmoe_b200.ops import _lib, gemm

pytestmark = pytest.mark.gpu


def _call(lib, w, x, y, bn, splitk):
    T, K = x.shape
    F = w.shape[0]
    return lib.dmoe_linear_noalloc(ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(x.data_ptr()),
                                   ctypes.c_void_p(y.data_ptr()), ctypes.c_int(T), ctypes.c_int(F), ctypes.c_int(K),
                                   ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(y.stride(0)), ctypes.c_int(bn),
                                   ctypes.c_int(splitk), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_linear_matches_regular_entry_point_twice():
    lib = ctypes.CDLL(_lib.lib_path())     # the exported C symbol, not the Python wrapper of the regular path
    lib.dmoe_linear_noalloc.restype = ctypes.c_int
    lib.dmoe_noalloc_last_error.restype = ctypes.c_char_p
    torch.manual_seed(0)
    for call, (T, F, K, bn, sk) in enumerate([(200, 1024, 4096, 128, 4), (64, 512, 2048, 64, 3)]):
        x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
        w = (torch.randn(F, K, device="cuda") * K ** -0.5).to(torch.bfloat16)
        y = torch.zeros(T, F, dtype=torch.bfloat16, device="cuda")
        mem_before = torch.cuda.memory_allocated()
        rc = _call(lib, w, x, y, bn, sk)
        assert rc == 0, lib.dmoe_noalloc_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == mem_before
        st = ctypes.c_int(-1)
        assert lib.dmoe_noalloc_last_status(ctypes.byref(st)) == 0 and st.value == 0
        ref = gemm.linear(x, w, bn=bn, splitk=sk)            # existing entry point (caller-owned scratch)
        torch.cuda.synchronize()
        err = (y.float() - ref.float()).abs().max().item()
        mag = ref.float().abs().max().item() + 1e-6
        assert err / mag < 2e-2, f"call {call}: max err {err} vs magnitude {mag}"
        exact = x.float() @ w.float().T
        assert (y.float() - exact).abs().max().item() / exact.abs().max().item() < 2e-2


def test_noalloc_rejects_oversized_problem():
    lib = ctypes.CDLL(_lib.lib_path())
    lib.dmoe_linear_noalloc.restype = ctypes.c_int
    lib.dmoe_noalloc_last_error.restype = ctypes.c_char_p
    T, F, K = 1024, 8192, 4096          # 64 x 4 tiles x 8 splits x 128 KB of partials = 256 MB > 16 MB
    x = torch.zeros(T, K, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(F, K, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(T, F, dtype=torch.bfloat16, device="cuda")
    rc = _call(lib, w, x, y, 256, 8)
    assert rc == -30
    msg = lib.dmoe_noalloc_last_error().decode()
    assert "too large" in msg and "16777216" in msg
