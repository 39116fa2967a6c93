"""In-tree build of the native parts.

* ``lib/libdmoe_kernels.so`` -- every ``csrc/kernels/*.cu`` compiled by nvcc for sm_100a (C ABI, loaded with ctypes).
* ``disagmoe_c*.so``         -- the host runtime (``csrc/runtime/*.cpp``, pybind11 + libtorch).

Both are rebuilt only when a source is newer than the product. nvcc cross-compiles without a GPU.
Run ``python -m disagmoe_b200.build`` or call :func:`build_all`.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys
import sysconfig

ROOT = os.path.dirname(os.path.abspath(__file__))
KERNEL_DIR = os.path.join(ROOT, "csrc", "kernels")
RUNTIME_DIR = os.path.join(ROOT, "csrc", "runtime")
LIB_DIR = os.path.join(ROOT, "lib")
OBJ_DIR = os.path.join(ROOT, "build")
KERNEL_LIB = os.path.join(LIB_DIR, "libdmoe_kernels.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _newer(srcs, product):
    if not os.path.exists(product):
        return True
    t = os.path.getmtime(product)
    return any(os.path.getmtime(s) > t for s in srcs)


def _run(cmd, log=None):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + proc.stdout)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    return proc.stdout


def nvcc_path():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def build_kernels(force=False, verbose=False):
    """Compile csrc/kernels/*.cu into lib/libdmoe_kernels.so for sm_100a."""
    srcs = sorted(glob.glob(os.path.join(KERNEL_DIR, "*.cu")))
    hdrs = sorted(glob.glob(os.path.join(KERNEL_DIR, "*.cuh")) + glob.glob(os.path.join(KERNEL_DIR, "*.h")))
    if not force and not _newer(srcs + hdrs, KERNEL_LIB):
        return KERNEL_LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = nvcc_path()
    objs = []
    jobs = []
    for s in srcs:
        o = os.path.join(OBJ_DIR, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer([s] + hdrs, o):
            jobs.append(([nvcc] + NVCC_FLAGS + ["-I", KERNEL_DIR, "-c", s, "-o", o], o + ".log"))
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for out in ex.map(lambda j: _run(j[0], j[1]), jobs):
            if verbose:
                print(out)
    # link next to the product and rename: a reader (or a snapshot of the tree) never sees a half-written library
    _run([nvcc, "-shared", "-o", KERNEL_LIB + ".tmp"] + objs + ["-lcudart"])
    os.replace(KERNEL_LIB + ".tmp", KERNEL_LIB)
    return KERNEL_LIB


def runtime_lib_path():
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(ROOT, "disagmoe_c" + suffix)


def variant_lib_path(sanitize):
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(ROOT, "_variants", sanitize, "disagmoe_c" + suffix)


def sanitizer_runtime(sanitize):
    """Path of gcc's runtime library of a sanitizer (to be LD_PRELOADed into the Python process), or None."""
    name = {"address": "libasan.so", "thread": "libtsan.so"}[sanitize]
    p = subprocess.run(["gcc", "-print-file-name=" + name], capture_output=True, text=True).stdout.strip()
    return p if os.path.isabs(p) and os.path.exists(p) else None


def build_runtime(force=False, verbose=False, sanitize=None):
    """Compile csrc/runtime/*.cpp into the pybind11 module disagmoe_b200.disagmoe_c. ``sanitize`` = "address" or
    "thread" builds an instrumented copy under _variants/<sanitize>/ instead (-fsanitize=..., -O1 -g), which the
    package loads in place of the normal module when DMOE_RUNTIME_VARIANT=<sanitize> is set."""
    srcs = sorted(glob.glob(os.path.join(RUNTIME_DIR, "*.cpp")))
    hdrs = sorted(glob.glob(os.path.join(RUNTIME_DIR, "*.h")) + glob.glob(os.path.join(RUNTIME_DIR, "*.hpp")))
    out = variant_lib_path(sanitize) if sanitize else runtime_lib_path()
    os.makedirs(os.path.dirname(out), exist_ok=True)
    if not srcs:
        return None
    if not force and not _newer(srcs + hdrs, out):
        return out
    import pybind11
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OBJ_DIR, exist_ok=True)
    inc = ["-I" + p for p in ce.include_paths()] + ["-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"],
                                                    "-I" + RUNTIME_DIR, "-I" + KERNEL_DIR]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cflags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-DTORCH_EXTENSION_NAME=disagmoe_c",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi, "-DTORCH_API_INCLUDE_EXTENSION_H", "-Wno-unused-variable"]
    san_flags = []
    if sanitize:
        san_flags = ["-fsanitize=" + sanitize, "-fno-omit-frame-pointer", "-g"]
        cflags = ["-O1" if f == "-O2" else f for f in cflags] + san_flags
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(OBJ_DIR, ("rt_%s_" % sanitize if sanitize else "rt_") + os.path.basename(s)[:-4] + ".o")
        objs.append(o)
        if force or _newer([s] + hdrs, o):
            jobs.append((["g++"] + cflags + inc + ["-c", s, "-o", o], o + ".log"))
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for res in ex.map(lambda j: _run(j[0], j[1]), jobs):
            if verbose:
                print(res)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    _run(["g++", "-shared", "-o", out + ".tmp"] + san_flags + objs + ["-L" + torch_lib, "-Wl,-rpath," + torch_lib, "-ltorch",
                                                           "-ltorch_cpu", "-lc10", "-ltorch_python", "-lpthread", "-ldl"])
    os.replace(out + ".tmp", out)
    return out


def build_all(force=False, verbose=False):
    k = build_kernels(force=force, verbose=verbose)
    r = build_runtime(force=force, verbose=verbose)
    return k, r


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_all(force=force, verbose="-v" in sys.argv))
