"""The native runtime (pools, schedulers, dispatchers, sockets, block manager, sampler) under AddressSanitizer and
ThreadSanitizer: an instrumented copy of the extension is built next to the normal one and a subset of the CPU tests
that drive its threads runs in a child process with the sanitizer runtime preloaded. A report makes the child exit
non-zero. (The GPU pool offers no compute-sanitizer; kernels carry their own index checks and status words.)"""
import os
import subprocess
import sys

import pytest

from disagmoe_b200 import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TARGETS = ["tests/test_runtime_cpu.py",
           "tests/test_disagg_cpu.py::test_disaggregated_in_process_1attn_1expert",
           "tests/test_disagg_cpu.py::test_colocated_in_process",
           "tests/test_fused_serving_cpu.py::test_mixed_prefill_decode_micro_batches",
           "tests/test_fault_and_resume_cpu.py::test_duplicated_or_delayed_message_does_not_change_the_result",
           # worker processes inherit the preloaded sanitizer: TCP sockets between processes, the TP group, recovery
           "tests/test_disagg_cpu.py::test_three_processes_attention_tp2",
           "tests/test_fault_and_resume_cpu.py::test_recover_restarts_workers_and_readmits_unfinished_requests"]


@pytest.mark.parametrize("kind", ["address", "thread"])
def test_runtime_under_sanitizer(kind):
    rt = build.sanitizer_runtime(kind)
    if rt is None:
        pytest.skip(f"gcc has no {kind} sanitizer runtime on this machine")
    build.build_runtime(sanitize=kind)
    stdcpp = subprocess.run(["gcc", "-print-file-name=libstdc++.so.6"], capture_output=True, text=True).stdout.strip()
    env = dict(os.environ, DMOE_RUNTIME_VARIANT=kind, LD_PRELOAD=f"{rt} {stdcpp}", PYTHONPATH=ROOT)
    if kind == "address":
        # leak checking would report the interpreter's and libtorch's intentional process-lifetime allocations
        env["ASAN_OPTIONS"] = "detect_leaks=0:verify_asan_link_order=0:exitcode=66"
    else:
        supp = os.path.join(ROOT, "disagmoe_b200", "csrc", "runtime", "tsan.supp")
        env["TSAN_OPTIONS"] = f"report_signal_unsafe=0 exitcode=66 suppressions={supp}"
    out = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider"] + TARGETS, cwd=ROOT,
                         env=env, capture_output=True, text=True, timeout=900)
    tail = (out.stdout + out.stderr)[-3000:]
    assert out.returncode == 0, tail
    assert "Sanitizer" not in out.stderr, tail
    assert " passed" in out.stdout, tail
