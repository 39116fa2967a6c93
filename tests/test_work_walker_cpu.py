"""The GEMM's work partition (split-K and stream-K unit lists, workspace slots) checked on the host: the header is
plain C++, so a small g++ harness enumerates random problems and verifies exact coverage of every tile's K blocks."""
import os
import subprocess
import tempfile


def test_work_partition_covers_every_tile_exactly_once():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = os.path.join(tempfile.mkdtemp(), "work_walker_check")
    subprocess.run(["g++", "-O1", "-std=c++17", "-I", os.path.join(root, "disagmoe_b200", "csrc", "kernels"),
                    os.path.join(root, "tests", "native", "work_walker_check.cpp"), "-o", exe], check=True)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and out.stdout.startswith("ok"), out.stdout + out.stderr
