"""Dispatch / combine microbenchmark between an attention GPU group and an expert GPU group.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmark/dispatch_combine.py --attn A --tokens 64,256,1024,4096,16384

One MoE layer round trip for bf16 tokens of hidden 4096, top-2 over 8 experts with uniform random routing:
router top-k -> dispatch -> expert GEMM-1 + SwiGLU -> GEMM-2 -> weighted combine back at the attention GPUs.
``--tokens`` is per attention GPU. Ranks [0, A) are attention GPUs, ranks [A, N) expert GPUs (N - A must divide 8).

Variants:
  fused   peer-memory kernels of this package: route_dispatch_kernel (norm + gate + top-k + row reservation + remote
          stores + records + release flag in one launch), gated grouped tcgen05 GEMM-1, GEMM-2 with the combine
          epilogue (remote stores into the owner's partial buffer + completion flag), and norm_gather_kernel (bounded
          flag wait + add + RMSNorm in one launch) at the consumer: 4 launches per round trip.
  nccl    the reference-style path restated with library pieces: torch.topk, argsort + row permute, NCCL all-to-all of
          counts and rows (rows + metadata), torch._grouped_mm / SiLU-mul / torch._grouped_mm, NCCL all-to-all back,
          un-permute + weighted sum.

Per size it prints one JSON line: device time (CUDA events, max over ranks, median of --iters), and the achieved
fraction of the roofline = slower of FLOPs / measured bf16 peak and NVLink bytes / 770 GB/s per direction per GPU, plus an
HBM-inclusive bound that adds the expert weights every expert GPU has to stream once.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from disagmoe_b200.config import mixtral_config
from disagmoe_b200.models.experts import MoEExperts
from disagmoe_b200.ops import _lib, gemm
from disagmoe_b200.ops import functional as F
from disagmoe_b200.parallel.disagg import DisaggShape, ExpertRank, build_layout
from disagmoe_b200.parallel.peer import PeerArena

c_int, c_ll, c_vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
NVLINK_GBS = 770.0


def _vp(t):
    return c_vp(0 if t is None else t.data_ptr())


def load_peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["bf16_tflops"], d["hbm_gbs"], "measured"
    return 1590.0, 6650.0, "fallback"


class FusedAttnSide:
    """Router + dispatch (one kernel) and wait + add + RMSNorm (one kernel) of one attention GPU."""

    def __init__(self, cfg, shape, arena, layout, a, x, gate_w, norm_w):
        self.cfg, self.S, self.a, self.x, self.gate_w, self.norm_w = cfg, shape, a, x, gate_w, norm_w
        dev = x.device
        z = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        ex = [shape.n_attn + i for i in range(shape.n_expert)]
        self.disp_epoch, self.wait_epoch, self.ticket = z(1), z(1), z(1)
        self.parts = arena.view(layout.offset("parts0"), (shape.batch, cfg.top_k, cfg.hidden_size), torch.bfloat16)
        self.comb_flag = arena.view(layout.offset("comb_flag0"), (shape.n_expert,), torch.int32)
        self.tables = [arena.ptr_table(ex, layout.offset(n)) for n in ("recv_rows0", "recv_recs0", "recv_cnt0", "disp_flag0")]
        self.status = gemm.scratch(dev).status
        self.resid = x.clone()
        self.y = torch.empty_like(x)
        self.out = torch.empty_like(x)
        self.y_ptr = torch.tensor([self.y.data_ptr()], dtype=torch.int64, device=dev)

    def run(self):
        cfg, S = self.cfg, self.S
        H = cfg.hidden_size
        F.route_dispatch(self.resid, self.norm_w, 1e-5, self.gate_w, cfg.top_k, True, S.batch, x_bases=self.tables[0],
                         rec_bases=self.tables[1], cnt_bases=self.tables[2], flag_bases=self.tables[3], ld_dst=H,
                         experts_per_rank=S.experts_per_rank, n_dst=S.n_expert, my_rank=self.a,
                         region_cap=S.region_cap, disp_epoch=self.disp_epoch, ticket=self.ticket, status=self.status)
        F.norm_gather(self.x, self.parts, self.norm_w, 1e-5, self.out, self.y_ptr, 1, 0, H, S.batch, H,
                      wait_flags=self.comb_flag, n_wait=S.n_expert, wait_epoch=self.wait_epoch, ticket=self.ticket,
                      status=self.status)
        return self.out


class NcclPath:
    """Reference-style restatement with NCCL collectives and library GEMMs (all ranks call run())."""

    def __init__(self, cfg, A, X, rank, T, x, gate_w, norm_w, experts):
        self.cfg, self.A, self.X, self.rank, self.T = cfg, A, X, rank, T
        self.x, self.gate_w, self.norm_w, self.experts = x, gate_w, norm_w, experts
        self.is_attn = rank < A
        self.epr = (cfg.num_experts + X - 1) // X          # contiguous blocks; the last expert GPU may hold fewer
        self.dev = torch.device("cuda", torch.cuda.current_device())
        # the library GEMM wants row-major stacks; the fused path keeps its own copies tile-blocked
        self.w13, self.w2 = experts.logical_weights() if experts is not None else (None, None)

    def run(self):
        cfg, A, X, k, H = self.cfg, self.A, self.X, self.cfg.top_k, self.cfg.hidden_size
        W = A + X
        dev = self.dev
        send_counts = torch.zeros(W, self.epr, dtype=torch.int64, device=dev)
        if self.is_attn:
            h = torch.nn.functional.rms_norm(self.x.float(), (H,), self.norm_w.float(), 1e-5).to(torch.bfloat16)
            logits = h.float() @ self.gate_w.float().T      # fp32 router logits, as the fused router computes them
            wts, ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
            wts = wts / wts.sum(-1, keepdim=True)
            flat = ids.reshape(-1)
            order = torch.argsort(flat, stable=True)
            rows = h.index_select(0, order // k)                      # permute + duplicate
            per_expert = torch.bincount(flat, minlength=cfg.num_experts)
            send_counts[A:] = torch.nn.functional.pad(per_expert, (0, X * self.epr - cfg.num_experts)).view(X, self.epr)
            meta = torch.stack([order.float(), wts.reshape(-1)[order]], 1)   # per-row metadata travelling with the rows
        else:
            rows = torch.empty(0, H, dtype=torch.bfloat16, device=dev)
            meta = torch.empty(0, 2, device=dev)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts)
        in_split = send_counts.sum(1).tolist()
        out_split = recv_counts.sum(1).tolist()              # host sync: sizes must be known before receiving
        got = torch.empty(sum(out_split), H, dtype=torch.bfloat16, device=dev)
        dist.all_to_all_single(got, rows, out_split, in_split)
        got_meta = torch.empty(sum(out_split), 2, device=dev)
        dist.all_to_all_single(got_meta, meta, out_split, in_split)
        if not self.is_attn:
            # rows arrive grouped by source, each source's rows sorted by expert: merge into expert order
            cnt = recv_counts[:A]                             # [A, epr]
            eid = torch.cat([torch.repeat_interleave(torch.arange(self.epr, device=dev), cnt[a]) for a in range(A)])
            perm = torch.argsort(eid, stable=True)
            xs = got.index_select(0, perm)
            e = self.experts
            offs = cnt.sum(0).cumsum(0).int()[:e.num_experts]
            up = torch._grouped_mm(xs, self.w13.transpose(1, 2), offs=offs)
            I = up.shape[1] // 2
            act = torch.nn.functional.silu(up[:, :I]) * up[:, I:]
            down = torch._grouped_mm(act, self.w2.transpose(1, 2), offs=offs)
            down = down * got_meta.index_select(0, perm)[:, 1:2].to(torch.bfloat16)
            back = torch.empty_like(down)
            back[perm] = down
        else:
            back = torch.empty(0, H, dtype=torch.bfloat16, device=dev)
        ret = torch.empty(sum(in_split), H, dtype=torch.bfloat16, device=dev)
        dist.all_to_all_single(ret, back, in_split, out_split)
        if self.is_attn:
            un = torch.empty_like(ret)
            un[order] = ret
            return self.x + un.view(self.T, k, H).sum(1)
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--attn", type=int, default=0, help="attention GPUs (default: half of the world)")
    ap.add_argument("--tokens", default="64,256,1024,4096,16384")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--variants", default="fused,nccl")
    ap.add_argument("--check", action="store_true", help="compare the fused result with the NCCL path once per size")
    args = ap.parse_args()
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    A = args.attn or world // 2
    X = world - A
    cfg = mixtral_config.clone(num_layers=1)
    EPR = (cfg.num_experts + X - 1) // X
    assert (X - 1) * EPR < cfg.num_experts, "an expert GPU would hold no expert"
    peak_tf, hbm_gbs, src = load_peaks()
    is_attn = rank < A
    H, I, E, k = cfg.hidden_size, cfg.intermediate_size, cfg.num_experts, cfg.top_k
    gate_w = (torch.randn(E, H, generator=torch.Generator().manual_seed(1)) * 0.05).to(torch.bfloat16).to(dev)
    norm_w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    sizes = [int(t) for t in args.tokens.split(",")]
    tmax = max(sizes)
    big_shape = DisaggShape(A, X, 1, tmax, k, H, E)
    layout_bytes = build_layout(big_shape).size
    arena = PeerArena.create(layout_bytes, device=dev)
    experts_mod = None
    if not is_attn:
        experts_mod = MoEExperts(cfg, 0, (rank - A) * EPR, min((rank - A + 1) * EPR, E), device=dev, dtype=torch.bfloat16)
        experts_mod.init_weights()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for T in sizes:
        shape = DisaggShape(A, X, 1, T, k, H, E)
        layout = build_layout(shape)
        arena.local.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(100 + rank)).to(torch.bfloat16).to(dev)
        fused = None
        if is_attn:
            fused = FusedAttnSide(cfg, shape, arena, layout, rank, x, gate_w, norm_w)
        else:
            er = ExpertRank.__new__(ExpertRank)
            er.cfg, er.shape, er.arena, er.layout, er.x, er.device = cfg, shape, arena, layout, rank - A, dev
            er.layers = [experts_mod]
            rows = EPR * shape.region_cap
            z = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
            er.act = torch.zeros(rows, I, dtype=torch.bfloat16, device=dev)
            er.ticket = z(1)
            er.mb = [dict(rows=arena.view(layout.offset("recv_rows0"), (rows, H), torch.bfloat16),
                          recs=arena.view(layout.offset("recv_recs0"), (rows, 4), torch.int32),
                          cnt=arena.view(layout.offset("recv_cnt0"), (EPR,), torch.int32),
                          flag=arena.view(layout.offset("disp_flag0"), (A,), torch.int32),
                          wait_epoch=z(1), signal_epoch=z(1),
                          parts_bases=arena.ptr_table(list(range(A)), layout.offset("parts0")),
                          signal_ptrs=arena.ptr_table(list(range(A)), layout.offset("comb_flag0")))]
            er.bn = gemm.pick_bn(gemm._group_hint(A * T * k, E), gemm.EPI_SWIGLU)
            er.bn2 = gemm.pick_bn(gemm._group_hint(A * T * k, E), gemm.EPI_COMBINE)
            er.sk2 = gemm.want_streamk(gemm.EPI_COMBINE, H, EPR, A * T * k * EPR // E, er.bn2, gemm.num_sms(dev))
            fused = er
        nccl = NcclPath(cfg, A, X, rank, T, x, gate_w, norm_w, experts_mod)

        def run_fused():
            return fused.run() if is_attn else fused.layer(0, 0)

        results = {}
        for name, fn in (("fused", run_fused), ("nccl", nccl.run)):
            if name not in args.variants:
                continue
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            times = []
            for _ in range(args.iters):
                flush.zero_()
                torch.cuda.synchronize()
                dist.barrier()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                fn()
                e.record()
                torch.cuda.synchronize()
                t = torch.tensor([s.elapsed_time(e)], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                times.append(float(t))
            times.sort()
            results[name] = times[len(times) // 2]
        err = None
        if args.check and "fused" in results and "nccl" in results:
            a_out = run_fused()
            b_out = nccl.run()
            torch.cuda.synchronize()
            if is_attn:
                # row-wise: a token whose top-2 set flipped on a near tie differs entirely, so report the share of
                # rows that disagree by more than 5 % next to the worst error of the agreeing rows
                d = (a_out.float() - b_out.float()).abs().amax(1) / b_out.float().abs().amax(1)
                bad = (d > 0.05).float().mean().item()
                err = float(d[d <= 0.05].max()) if (d <= 0.05).any() else 1.0
                if bad > 0.02:
                    err = 1.0
            t = torch.tensor([err or 0.0], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            err = float(t)
        st = torch.tensor([float(gemm.check_status(dev))], device=dev)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        if rank == 0:
            pairs = A * T * k
            flops = 2.0 * pairs * 3 * H * I                        # whole job
            t_compute = flops * EPR / E / (peak_tf * 1e12)         # the fullest expert GPU (EPR of E experts), even routing
            nv_bytes = max(T * k * H * 2.0, pairs * H * 2.0 * EPR / E)   # per direction: what one attention GPU sends / one expert GPU receives
            t_link = nv_bytes / (NVLINK_GBS * 1e9)
            t_hbm = EPR * 3 * H * I * 2.0 / (hbm_gbs * 1e9)
            roof = max(t_compute, t_link)
            roof_hbm = max(roof, t_hbm)
            line = {"tokens_per_attn_gpu": T, "split": f"{A}+{X}", "peaks": src, "kernel_status": int(st),
                    "roofline_us": round(roof * 1e6, 1), "roofline_with_hbm_us": round(roof_hbm * 1e6, 1)}
            for name, ms in results.items():
                line[name + "_us"] = round(ms * 1e3, 1)
                line[name + "_frac_of_roofline"] = round(roof / (ms / 1e3), 3)
                line[name + "_frac_of_hbm_roofline"] = round(roof_hbm / (ms / 1e3), 3)
            if err is not None:
                line["fused_vs_nccl_rel_err"] = round(err, 4)
            print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
