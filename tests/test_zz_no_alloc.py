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
    # (T, F, K, token tile, splits): explicit choices, the library's own picks (0), and a single split
    cases = [(200, 1024, 4096, 128, 4), (64, 512, 2048, 64, 3), (96, 768, 4096, 0, 0), (40, 256, 1024, 32, 1)]
    gemm.scratch("cuda")                                     # the regular path's scratch exists before the probes
    for call, (T, F, K, bn, sk) in enumerate(cases):
        x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
        w = (torch.randn(F, K, device="cuda") * K ** -0.5).to(torch.bfloat16)
        y = torch.zeros(T, F, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        mem_before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]           # the driver's view: a cudaMalloc inside the library shows here
        rc = _call(lib, w, x, y, bn, sk)
        assert rc == 0, lib.dmoe_noalloc_last_error().decode()
        st = ctypes.c_int(-1)
        assert lib.dmoe_noalloc_last_status(ctypes.byref(st)) == 0 and st.value == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == mem_before
        if call > 0:                                         # the first call may load the module's lazy parts
            assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated behind the call"
        ref = gemm.linear(x, w, bn=bn, splitk=sk)            # existing entry point (caller-owned scratch)
        torch.cuda.synchronize()
        _close(y, ref, f"call {call} vs the regular entry point")
        _close(y, x.float() @ w.float().T, f"call {call} vs fp32")


def _close(got, ref, what):
    """|err| <= 2^-7 |ref| + 2^-7 rms(ref) for every element (bf16 output of an fp32 accumulation)."""
    got, ref = got.float(), ref.float()
    bound = ref.abs() * 2 ** -7 + ref.pow(2).mean().sqrt() * 2 ** -7
    bad = ((got - ref).abs() > bound).sum().item()
    assert bad == 0, f"{what}: {bad} elements outside the bound, max err {(got - ref).abs().max().item()}"


def test_noalloc_strided_views_on_a_side_stream():
    """X and Y are column slices of wider buffers (row strides larger than K and F) and the call runs on a
    non-blocking side stream: the status read has to be ordered behind the kernel on that stream."""
    lib = ctypes.CDLL(_lib.lib_path())
    lib.dmoe_linear_noalloc.restype = ctypes.c_int
    lib.dmoe_noalloc_last_error.restype = ctypes.c_char_p
    torch.manual_seed(1)
    T, F, K = 72, 384, 2048
    xw = torch.randn(T, K + 64, device="cuda").to(torch.bfloat16)
    yw = torch.zeros(T, F + 128, dtype=torch.bfloat16, device="cuda")
    x, y = xw[:, :K], yw[:, :F]
    w = (torch.randn(F, K, device="cuda") * K ** -0.5).to(torch.bfloat16)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        rc = _call(lib, w, x, y, 0, 0)
        assert rc == 0, lib.dmoe_noalloc_last_error().decode()
        st = ctypes.c_int(-1)
        assert lib.dmoe_noalloc_last_status(ctypes.byref(st)) == 0 and st.value == 0
    side.synchronize()
    _close(y, x.float() @ w.float().T, "strided call")
    assert float(yw[:, F:].abs().max()) == 0.0               # nothing was written outside the [T, F] view
    # a row stride smaller than K is refused with a message, before any launch
    rc = lib.dmoe_linear_noalloc(ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(x.data_ptr()),
                                 ctypes.c_void_p(y.data_ptr()), T, F, K, ctypes.c_longlong(K - 8),
                                 ctypes.c_longlong(y.stride(0)), 0, 0, ctypes.c_void_p(0))
    assert rc == -31 and b"stride" in lib.dmoe_noalloc_last_error()


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
