"""Host-side batch preparation cost (reference: benchmark/benchmark_preprocess.py): how long the native runtime needs to
build the attention metadata of a decode batch -- block-table growth, slots, rows -- as the batch grows. No GPU needed."""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from disagmoe_b200 import disagmoe_c as C


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=200)
    a = ap.parse_args(argv)
    out = []
    for bs in (8, 32, 128, 256, 512, 1024):
        bm = C.BlockManager(16, bs * 80, 0, bs)
        lens = [100 + (i * 37) % 900 for i in range(bs)]
        for i, l in enumerate(lens):
            bm.allocate(i, l + 1)
        ids = list(range(bs))
        t0 = time.perf_counter()
        for it in range(a.iters):
            bm.step_decode(ids, lens)
            bm.drain_updates()
            lens = [l + 1 for l in lens]
        us = (time.perf_counter() - t0) / a.iters * 1e6
        m = C.Metadata([bs * 2, 4096])
        m.req_ids = [i // 2 for i in range(bs * 2)]
        m.exp_ids = [(i * 7) % 8 for i in range(bs * 2)]
        m.attn_dp_ranks = [0] * (bs * 2)
        t0 = time.perf_counter()
        for it in range(a.iters):
            C.Metadata.merge_by_exp_ids([m])
        us_sort = (time.perf_counter() - t0) / a.iters * 1e6
        print(f"batch {bs}: decode block-table step {us:.1f} us, expert counting sort of {bs * 2} rows {us_sort:.1f} us")
        out.append((bs, us, us_sort))
    return out


if __name__ == "__main__":
    main()
