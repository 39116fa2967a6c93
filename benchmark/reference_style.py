"""Reference-style decode step: the data path of USC-NSL/DisagMoE restated with library pieces, as a baseline.

The reference cannot be built on this image, so this module re-creates what one of its decode iterations executes, on
the same model shape, batch, context lengths and GPU count as the product path, using none of this package's kernels:

    attention GPUs   torch RMSNorm, cuBLAS linears (``F.linear``), RoPE with torch ops, KV append by index copy, a
                     library paged-attention kernel (vLLM's flash-attention fork, else flash-attn, else SDPA over
                     gathered pages), ``torch.topk`` routing                 -- disagmoe/models/attention.py:202-233
    dispatch         stable sort by expert + row permute, NCCL all-to-all of counts (host sync: the receiver has to
                     learn the sizes first, as the reference's ZMQ metadata message does) and of rows + metadata
                                                                             -- csrc/muhelper/muhelper.cpp:189-228,485-515
    expert GPUs      merge by expert, ``torch._grouped_mm`` -> SiLU * mul -> ``torch._grouped_mm``, router-weight scale
                                                                             -- disagmoe/models/experts.py:81-96
    combine          NCCL all-to-all back, un-permute, top-k sum, residual   -- disagmoe/frontend/engine.py:624-628,731-734

N = 1 runs everything on one GPU (no collectives, the whole step in one CUDA graph, which is more than the reference
captures). N >= 2 uses N/2 data-parallel attention GPUs and N/2 expert GPUs with two micro-batches in flight, so the
two sides overlap the way they do in the product path. Random weights, synthetic KV history.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as tF


def _pick_attention(device, n_q, n_kv, hd):
    """Returns (name, page_size, fn(q [B, n_q, hd], kcache, vcache, block_table [B, nblk] int32, ctx [B] int32))."""
    B = 2
    q = torch.randn(B, n_q, hd, device=device, dtype=torch.bfloat16)
    ctx = torch.tensor([5, 17], dtype=torch.int32, device=device)

    def probe(page, fn):
        kc = torch.randn(4, page, n_kv, hd, device=device, dtype=torch.bfloat16)
        bt = torch.tensor([[0, 1], [2, 3]], dtype=torch.int32, device=device)
        out = fn(q, kc, kc, bt, ctx)
        torch.cuda.synchronize()
        assert out.shape == (B, n_q, hd) and bool(torch.isfinite(out.float()).all())

    try:
        from vllm.vllm_flash_attn import flash_attn_varlen_func as vfa

        def f_vllm(q, kc, vc, bt, ctx):
            cu = torch.arange(q.shape[0] + 1, dtype=torch.int32, device=q.device)
            return vfa(q, kc, vc, max_seqlen_q=1, cu_seqlens_q=cu, max_seqlen_k=int(bt.shape[1] * kc.shape[1]),
                       seqused_k=ctx, block_table=bt, causal=True, fa_version=2)
        probe(16, f_vllm)
        return "vllm flash-attention fork (paged, page 16)", 16, f_vllm
    except Exception:
        pass
    try:
        from flash_attn import flash_attn_with_kvcache as fa

        def f_fa(q, kc, vc, bt, ctx):
            return fa(q.unsqueeze(1), kc, vc, cache_seqlens=ctx, block_table=bt, causal=True).squeeze(1)
        probe(256, f_fa)
        return "flash-attn 2 flash_attn_with_kvcache (paged, page 256: its minimum)", 256, f_fa
    except Exception:
        pass

    def f_sdpa(q, kc, vc, bt, ctx):
        Bq, page = q.shape[0], kc.shape[1]
        k = kc[bt.long()].reshape(Bq, -1, n_kv, hd).transpose(1, 2)
        v = vc[bt.long()].reshape(Bq, -1, n_kv, hd).transpose(1, 2)
        mask = torch.arange(k.shape[2], device=q.device)[None, :] < ctx[:, None]
        o = tF.scaled_dot_product_attention(q.unsqueeze(2), k, v, attn_mask=mask[:, None, None, :], enable_gqa=True)
        return o.squeeze(2)
    probe(16, f_sdpa)
    return "torch SDPA over gathered pages (no paged library kernel importable)", 16, f_sdpa


class ReferenceStyleDecode:
    def __init__(self, cfg, world: int, rank: int, local_rank: int, batch: int, ctx_min: int, ctx_max: int,
                 total_steps: int, gen: torch.Generator, n_mb: int = 2):
        self.cfg, self.world, self.rank = cfg, world, rank
        dev = self.device = torch.device("cuda", local_rank)
        dt = torch.bfloat16
        self.A = A = 1 if world == 1 else world // 2
        self.X = X = 1 if world == 1 else world - A
        self.colocated = world == 1
        self.is_attn = self.colocated or rank < A
        self.is_expert = self.colocated or rank >= A
        self.n_mb = 1 if self.colocated else n_mb
        self.B = B = batch
        H, E, I, L = cfg.hidden_size, cfg.num_experts, cfg.intermediate_size, cfg.num_layers
        self.epr = (E + X - 1) // X
        self.h2d_bytes_last = self.d2h_bytes_last = 0
        self.profile_events, self.event_pairs = False, []
        self.launches = 0
        rnd = lambda *s, std=0.02: torch.randn(*s, device=dev, dtype=torch.float32).mul_(std).to(dt)
        if self.is_attn:
            n_q, n_kv, hd = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
            self.attn_name, self.page, self.attn_fn = _pick_attention(dev, n_q, n_kv, hd)
            self.qkv_w = [rnd((n_q + 2 * n_kv) * hd, H) for _ in range(L)]
            self.o_w = [rnd(H, n_q * hd) for _ in range(L)]
            self.gate_w = [rnd(E, H) for _ in range(L)]
            self.ln1 = [torch.ones(H, device=dev, dtype=dt) for _ in range(L)]
            self.ln2 = [torch.ones(H, device=dev, dtype=dt) for _ in range(L)]
            self.embed_w, self.lm_w, self.norm_w = rnd(cfg.vocab_size, H), rnd(cfg.vocab_size, H), torch.ones(H, device=dev, dtype=dt)
            n = self.n_mb * B
            self.ctx = torch.randint(ctx_min, ctx_max + 1, (n,), generator=gen)
            page = self.page
            nblk = [(int(c) + total_steps + 2 + page - 1) // page for c in self.ctx]
            self.max_blocks = max(nblk)
            self.block_table = torch.zeros(n, self.max_blocks, dtype=torch.int32)
            nxt = 0
            for i, b in enumerate(nblk):
                self.block_table[i, :b] = torch.arange(nxt, nxt + b, dtype=torch.int32)
                nxt += b
            self.block_table = self.block_table.to(dev)
            self.kv = torch.empty(L, 2, nxt, page, n_kv, hd, device=dev, dtype=dt).normal_(0, 0.5)
            self.ids = torch.randint(0, cfg.vocab_size, (n,), generator=gen).to(dev)
            self.h_ids = torch.zeros(n, dtype=torch.int64).pin_memory()
            self.h_ctx = torch.zeros(n, dtype=torch.int32).pin_memory()
            self.h_out = torch.zeros(n, dtype=torch.int64).pin_memory()
            self.d_ids = torch.zeros(n, dtype=torch.int64, device=dev)
            self.d_ctx = torch.zeros(n, dtype=torch.int32, device=dev)
            self.d_out = torch.zeros(n, dtype=torch.int64, device=dev)
            self.last = self.ids.cpu()
            inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd))
            pos = torch.arange(cfg.max_seq_len, device=dev, dtype=torch.float32)
            self.cos, self.sin = torch.cos(pos[:, None] * inv[None]), torch.sin(pos[:, None] * inv[None])
        if self.is_expert:
            x = 0 if self.colocated else rank - A
            self.e_lo, self.e_hi = x * self.epr, min((x + 1) * self.epr, E)
            ne = self.e_hi - self.e_lo
            self.w13 = [rnd(ne, H, 2 * I) for _ in range(L)]      # [in, out]: what torch._grouped_mm multiplies by
            self.w2 = [rnd(ne, I, H) for _ in range(L)]
        self.graph = None
        torch.cuda.synchronize()
        if self.colocated:
            self._stage(0)
            for _ in range(2):
                self._colocated_step()
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._colocated_step()
            torch.cuda.synchronize()

    # ---- pieces ----------------------------------------------------------------------------------------------
    def _attention(self, l: int, x: torch.Tensor, sl: slice) -> torch.Tensor:
        cfg = self.cfg
        n_q, n_kv, hd = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        ctx = self.d_ctx[sl]                                  # tokens cached before this step = position of the new token
        h = tF.rms_norm(x, (cfg.hidden_size,), self.ln1[l], cfg.rms_norm_eps)
        qkv = tF.linear(h, self.qkv_w[l])
        q, k, v = qkv.split([n_q * hd, n_kv * hd, n_kv * hd], dim=-1)
        q, k = q.view(-1, n_q, hd), k.view(-1, n_kv, hd)
        cos, sin = self.cos[ctx.long()][:, None, :], self.sin[ctx.long()][:, None, :]

        def rot(t):
            t1, t2 = t[..., :hd // 2].float(), t[..., hd // 2:].float()
            return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], -1).to(t.dtype)
        q, k = rot(q), rot(k)
        bt = self.block_table[sl]
        blk = bt.gather(1, (ctx // self.page).long()[:, None]).squeeze(1).long()
        kc, vc = self.kv[l, 0], self.kv[l, 1]
        kc[blk, (ctx % self.page).long()] = k
        vc[blk, (ctx % self.page).long()] = v.view(-1, n_kv, hd)
        o = self.attn_fn(q, kc, vc, bt, ctx + 1)
        return x + tF.linear(o.reshape(-1, n_q * hd), self.o_w[l])

    def _route(self, l: int, x: torch.Tensor):
        cfg = self.cfg
        h = tF.rms_norm(x, (cfg.hidden_size,), self.ln2[l], cfg.rms_norm_eps)
        logits = tF.linear(h, self.gate_w[l]).float()
        wts, ids = torch.topk(torch.softmax(logits, -1), cfg.top_k, dim=-1)
        wts = wts / wts.sum(-1, keepdim=True)
        flat = ids.reshape(-1)
        order = torch.argsort(flat, stable=True)              # the reference's counting sort by expert id
        rows = h.index_select(0, order // cfg.top_k)          # permute + duplicate (its permute_tokens kernel)
        counts = (flat[:, None] == torch.arange(cfg.num_experts, device=flat.device)[None, :]).sum(0)   # capture-safe histogram
        return rows, order, wts.reshape(-1)[order], counts

    def _experts(self, l: int, xs: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        offs = counts.cumsum(0).int()
        up = torch._grouped_mm(xs, self.w13[l], offs=offs)
        I = up.shape[1] // 2
        act = tF.silu(up[:, :I]) * up[:, I:]
        return torch._grouped_mm(act, self.w2[l], offs=offs)

    def _head(self, x: torch.Tensor, sl: slice) -> None:
        h = tF.rms_norm(x, (self.cfg.hidden_size,), self.norm_w, self.cfg.rms_norm_eps)
        self.d_out[sl] = tF.linear(h, self.lm_w).argmax(-1)

    # ---- one GPU -----------------------------------------------------------------------------------------------
    def _colocated_step(self) -> None:
        cfg, k = self.cfg, self.cfg.top_k
        sl = slice(0, self.B)
        x = self.embed_w[self.d_ids[sl]]
        for l in range(cfg.num_layers):
            x = self._attention(l, x, sl)
            rows, order, w, counts = self._route(l, x)
            down = self._experts(l, rows, counts) * w[:, None].to(rows.dtype)
            un = torch.empty_like(down)
            un[order] = down
            x = x + un.view(-1, k, cfg.hidden_size).sum(1)
        self._head(x, sl)

    # ---- N >= 2 -----------------------------------------------------------------------------------------------
    def _a2a(self, out_rows: int, src: torch.Tensor, out_split: List[int], in_split: List[int]) -> torch.Tensor:
        got = torch.empty(out_rows, *src.shape[1:], dtype=src.dtype, device=self.device)
        dist.all_to_all_single(got, src, out_split, in_split)
        return got

    def _moe_hop(self, l: int, x: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Dispatch -> experts -> combine of one micro-batch; every rank calls it (NCCL all-to-all over all ranks)."""
        cfg, A, X, W, dev = self.cfg, self.A, self.X, self.world, self.device
        H, k = cfg.hidden_size, cfg.top_k
        send_counts = torch.zeros(W, self.epr, dtype=torch.int64, device=dev)
        if self.is_attn:
            rows, order, w, per_expert = self._route(l, x)
            send_counts[A:] = tF.pad(per_expert, (0, X * self.epr - cfg.num_experts)).view(X, self.epr)
            meta = w.float()[:, None]
        else:
            rows = torch.empty(0, H, dtype=torch.bfloat16, device=dev)
            meta = torch.empty(0, 1, device=dev)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts)
        in_split = send_counts.sum(1).tolist()
        out_split = recv_counts.sum(1).tolist()               # host sync: sizes are needed before the rows can be received
        got = self._a2a(sum(out_split), rows, out_split, in_split)
        got_w = self._a2a(sum(out_split), meta, out_split, in_split)
        if not self.is_attn:
            cnt = recv_counts[:A]                              # [A, epr]: rows per (source, local expert)
            eid = torch.cat([torch.repeat_interleave(torch.arange(self.epr, device=dev), cnt[a]) for a in range(A)])
            perm = torch.argsort(eid, stable=True)             # merge the sources' expert-sorted runs (its gather kernel)
            ne = self.e_hi - self.e_lo
            down = self._experts(l, got.index_select(0, perm), cnt.sum(0)[:ne])
            down = down * got_w.index_select(0, perm).to(torch.bfloat16)
            back = torch.empty_like(down)
            back[perm] = down
        else:
            back = torch.empty(0, H, dtype=torch.bfloat16, device=dev)
        ret = self._a2a(sum(in_split), back, in_split, out_split)
        if self.is_attn:
            un = torch.empty_like(ret)
            un[order] = ret
            return x + un.view(-1, k, H).sum(1)
        return None

    def _disagg_step(self) -> None:
        cfg, B = self.cfg, self.B
        xs: List[Optional[torch.Tensor]] = [None] * self.n_mb
        if self.is_attn:
            for m in range(self.n_mb):
                xs[m] = self.embed_w[self.d_ids[m * B:(m + 1) * B]]
        for l in range(cfg.num_layers):
            for m in range(self.n_mb):
                if self.is_attn:
                    xs[m] = self._attention(l, xs[m], slice(m * B, (m + 1) * B))
                xs[m] = self._moe_hop(l, xs[m])
        if self.is_attn:
            for m in range(self.n_mb):
                self._head(xs[m], slice(m * B, (m + 1) * B))

    # ---- bench protocol -----------------------------------------------------------------------------------------
    def _stage(self, step: int) -> int:
        if not self.is_attn:
            return 0
        self.h_ids.copy_(self.last)
        self.h_ctx.copy_(self.ctx + step)
        self.d_ids.copy_(self.h_ids, non_blocking=True)
        self.d_ctx.copy_(self.h_ctx, non_blocking=True)
        return self.h_ids.numel() * 12

    _step_no = 0

    def step(self) -> None:
        ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) if self.profile_events else None
        if ev:
            ev[0].record()
        self.h2d_bytes_last = self._stage(self._step_no)
        self._step_no += 1
        if self.graph is not None:
            self.graph.replay()
        else:
            self._disagg_step()
        self.d2h_bytes_last = 0
        if self.is_attn:
            self.h_out.copy_(self.d_out, non_blocking=True)
            self.d2h_bytes_last = self.h_out.numel() * 8
        if ev:
            ev[1].record()
        torch.cuda.current_stream().synchronize()
        if self.is_attn:
            self.last = self.h_out.clone()
        if ev:
            self.event_pairs.append(ev)

    def tokens_per_step(self) -> int:
        return self.n_mb * self.B if self.is_attn else 0

    @property
    def parallelism(self) -> str:
        if self.colocated:
            return f"reference-style colocated1 (library kernels, one CUDA graph); attention: {self.attn_name}"
        name = self.attn_name if self.is_attn else "n/a"
        return (f"reference-style attn dp{self.A} + expert ep{self.X}, NCCL all-to-all dispatch/combine with host-synced "
                f"sizes, torch._grouped_mm experts, {self.n_mb} micro-batches; attention: {name}")
