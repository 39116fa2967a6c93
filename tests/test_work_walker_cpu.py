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


def test_dense_tile_and_split_choice_is_launchable_and_follows_the_measured_order():
    """The (token tile, split-K) picker of decode-size dense GEMMs: every choice is one the launcher accepts (no empty
    split, at least 8 K blocks per split) and it prefers what the tile / split sweep on B200 measured as fastest."""
    from disagmoe_b200.ops import gemm
    for F, K in ((6144, 4096), (4096, 4096), (1536, 4096), (4096, 1024), (32000, 4096), (512, 128)):
        for T in (1, 7, 16, 64, 100, 128, 256, 512, 1000):
            bn, sk = gemm.pick_dense(T, F, K, 148)
            kblocks = (K + 63) // 64
            per = (kblocks + sk - 1) // sk
            assert bn in (32, 64, 128, 256) and sk >= 1
            assert sk == 1 or (per >= 8 and (kblocks + per - 1) // per == sk)
    # measured: QKV (F 6144) at 256 tokens is fastest on 128-token tiles, o_proj (F 4096) at 256 tokens with a split
    assert gemm.pick_dense(256, 6144, 4096, 148)[0] == 128
    assert gemm.pick_dense(256, 4096, 4096, 148) == (128, 2)
    assert gemm.pick_dense(64, 4096, 4096, 148)[1] >= 2


def test_tile_blocked_weight_layout_round_trip_and_box_order():
    """block_weight puts every 128-row x 64-column box of a K-contiguous stack into one contiguous run, boxes ordered
    (group, row tile, K block) as the GEMM's blocked tensor map addresses them; unblock_weight inverts it."""
    import torch
    from disagmoe_b200.ops import gemm
    w = torch.arange(2 * 256 * 192, dtype=torch.float32).view(2, 256, 192)
    b = gemm.block_weight(w)
    assert b.shape == w.shape and torch.equal(gemm.unblock_weight(b), w)
    flat, KB = b.reshape(-1), 192 // 64
    for g, m, kb in ((0, 0, 0), (0, 1, 2), (1, 0, 1), (1, 1, 2)):
        box = flat[((g * 2 + m) * KB + kb) * 128 * 64:][:128 * 64].view(128, 64)
        assert torch.equal(box, w[g, m * 128:(m + 1) * 128, kb * 64:(kb + 1) * 64])
    w2 = torch.randn(128, 64)
    assert torch.equal(gemm.block_weight(w2), w2)       # a single box is already in order


def test_stream_k_policy_follows_the_measured_operating_points():
    """want_streamk: never for the SwiGLU up-projection (two accumulators per partial tile); for the down-projection
    only where the expected tiles fill the last wave badly (2 local experts at decode sizes), not at 8 experts x 64."""
    from disagmoe_b200.ops import gemm
    H, I, sms = 4096, 14336, 148
    assert not gemm.want_streamk(gemm.EPI_SWIGLU, I, 2, 128, 128, sms)
    assert gemm.want_streamk(gemm.EPI_COMBINE, H, 2, 128, 128, sms)        # 64 tiles on 148 SMs
    assert gemm.want_streamk(gemm.EPI_COMBINE, H, 2, 512, 256, sms)
    assert not gemm.want_streamk(gemm.EPI_COMBINE, H, 8, 512, 128, sms)    # 256 tiles: 0.86 of two waves
    old = gemm.STREAM_K
    try:
        gemm.STREAM_K = False
        assert not gemm.want_streamk(gemm.EPI_COMBINE, H, 2, 128, 128, sms)
    finally:
        gemm.STREAM_K = old
