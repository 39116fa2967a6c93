"""Single-GPU serving engine: every layer's attention and experts colocated on one device.

The in-process counterpart of a one-worker ``ColocatePlacement`` deployment (reference: disagmoe/utils/placement.py:
467-508, disagmoe/frontend/engine.py:873-904): continuous batching over the whole-iteration executor
(:class:`disagmoe_b200.executor.fused.FusedModelExecutor`), the native paged-KV ``BlockManager`` with a
device-resident block table that is patched incrementally, pinned host staging for the per-step inputs and a
device->host read of the sampled ids (the sampler lives on the host, as in the reference).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .. import disagmoe_c as C
from ..config import CacheConfig, ModelConfig
from ..executor.fused import FusedModelExecutor
from ..utils.constants import EOS_TOKEN_ID


@dataclass
class _Seq:
    req_id: int
    prompt: List[int]
    max_new_tokens: int
    length: int = 0                 # tokens whose K/V are cached
    last_token: int = 0             # next input token
    outputs: List[int] = field(default_factory=list)
    t_arrival: float = 0.0
    t_tokens: List[float] = field(default_factory=list)


class ColocatedEngine:
    def __init__(self, cfg: ModelConfig, cache_cfg: Optional[CacheConfig] = None, device="cuda", max_batch_size: int = 256,
                 max_prefill_tokens: int = 4096, state_dict=None, num_blocks: Optional[int] = None,
                 enable_cuda_graph: bool = True, ignore_eos: bool = True, dtype=None):
        self.cfg = cfg
        self.cache_cfg = cache_cfg or CacheConfig()
        self.device = torch.device(device)
        self.max_batch_size = max_batch_size
        self.ignore_eos = ignore_eos
        self.executor = FusedModelExecutor(cfg, self.cache_cfg, device=device, dtype=dtype, max_batch_size=max_batch_size,
                                           max_prefill_tokens=max_prefill_tokens, state_dict=state_dict,
                                           num_blocks=num_blocks, enable_cuda_graph=enable_cuda_graph)
        self.block_size = self.cache_cfg.block_size
        self.block_mgr = C.BlockManager(self.block_size, self.executor.num_blocks - self.cache_cfg.num_reserved_blocks,
                                        self.cache_cfg.num_reserved_blocks, max_batch_size)
        self.waiting: List[_Seq] = []
        self.running: Dict[int, _Seq] = {}    # insertion ordered
        self.finished: Dict[int, _Seq] = {}
        pin = self.device.type == "cuda"
        B = max(max_batch_size, max_prefill_tokens)
        mk = lambda dt: torch.zeros(B, dtype=dt, pin_memory=pin)
        self._h_ids, self._h_pos, self._h_ctx, self._h_row = mk(torch.int32), mk(torch.int32), mk(torch.int32), mk(torch.int32)
        self._h_slots = mk(torch.int64)
        self._h_out = torch.zeros(B, dtype=torch.int32, pin_memory=pin)
        self._h_patch = torch.zeros(3, 4 * B + 1024, dtype=torch.int64, pin_memory=pin)
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0
        self.steps = 0
        self._last_was_prefill = False
        self.profile_events = False     # when set, every decode step appends a (start, end) CUDA event pair
        self.event_pairs = []

    # ---- requests -----------------------------------------------------------------------------------------------
    def add_request(self, req_id: int, prompt_ids: List[int], max_new_tokens: int) -> None:
        assert len(prompt_ids) >= 1 and len(prompt_ids) + max_new_tokens <= self.cfg.max_seq_len
        self.waiting.append(_Seq(req_id, list(prompt_ids), max_new_tokens, t_arrival=time.time()))

    def add_synthetic_request(self, req_id: int, context_len: int, next_token: int, max_new_tokens: int) -> None:
        """A sequence that already has ``context_len`` cached tokens (whatever the KV cache holds at its blocks):
        used by benchmarks that measure decode throughput at a given context length without running the prefill."""
        assert len(self.running) < self.max_batch_size
        s = _Seq(req_id, [], max_new_tokens, length=context_len, last_token=next_token, t_arrival=time.time())
        self.block_mgr.allocate(req_id, context_len + 1)
        self.running[req_id] = s
        self._apply_block_table_patches()

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- block table --------------------------------------------------------------------------------------------
    def _apply_block_table_patches(self) -> int:
        ups = self.block_mgr.drain_updates()
        if not ups:
            return 0
        n = len(ups)
        if n > self._h_patch.shape[1]:
            self._h_patch = torch.zeros(3, 2 * n, dtype=torch.int64, pin_memory=self._h_patch.is_pinned())
        t = torch.tensor(ups, dtype=torch.int64)          # [n, 3] rows, cols, blocks
        self._h_patch[:, :n] = t.T
        d = self._h_patch[:, :n].to(self.device, non_blocking=True)
        self.executor.block_tables.index_put_((d[0], d[1]), d[2].int())
        return 3 * 8 * n

    # ---- steps --------------------------------------------------------------------------------------------------
    def _blocks(self, tokens: int) -> int:
        return (tokens + self.block_size - 1) // self.block_size

    def _prefill(self) -> List[Tuple[int, int]]:
        ex = self.executor
        batch: List[_Seq] = []
        total = 0
        # blocks the running sequences will still take before they finish stay free: a decode step never finds the
        # pool empty (there is no preemption)
        reserve = sum(max(0, self._blocks(max(len(s.prompt), s.length) + s.max_new_tokens - len(s.outputs)) -
                          len(self.block_mgr.get_seq_block_list(s.req_id))) for s in self.running.values())
        while self.waiting and len(self.running) + len(batch) < self.max_batch_size:
            s = self.waiting[0]
            need = self._blocks(len(s.prompt) + s.max_new_tokens)
            if total + len(s.prompt) > ex.prefill_buf.cap or self.block_mgr.num_free_blocks() - reserve < need:
                break
            reserve += need - self._blocks(len(s.prompt) + 1)
            self.waiting.pop(0)
            self.block_mgr.allocate(s.req_id, len(s.prompt) + 1)
            batch.append(s)
            total += len(s.prompt)
        if not batch:
            return []
        h2d = self._apply_block_table_patches()
        i = 0
        ends = []
        for s in batch:
            row = self.block_mgr.row_of(s.req_id)
            for p, tok in enumerate(s.prompt):
                self._h_ids[i], self._h_pos[i], self._h_ctx[i], self._h_row[i] = tok, p, p + 1, row
                self._h_slots[i] = self.block_mgr.slot_of(s.req_id, p)
                i += 1
            ends.append(i - 1)
        T = i
        nxt, _ = ex.prefill(self._h_ids[:T], self._h_pos[:T], self._h_slots[:T], self._h_ctx[:T], self._h_row[:T])
        out = nxt.cpu()
        res = []
        now = time.time()
        for s, e in zip(batch, ends):
            s.length = len(s.prompt)
            tok = int(out[e])
            self._record(s, tok, now)
            res.append((s.req_id, tok))
        self.h2d_bytes_last += h2d + T * 24
        self.d2h_bytes_last += T * 4
        return res

    def _record(self, s: _Seq, tok: int, now: float) -> None:
        s.outputs.append(tok)
        s.t_tokens.append(now)
        s.last_token = tok
        done = len(s.outputs) >= s.max_new_tokens or (not self.ignore_eos and tok == EOS_TOKEN_ID)
        if done:
            self.block_mgr.release(s.req_id)
            self.finished[s.req_id] = s
            self.running.pop(s.req_id, None)
        else:
            self.running[s.req_id] = s

    def _decode(self) -> List[Tuple[int, int]]:
        seqs = list(self.running.values())
        B = len(seqs)
        if B == 0:
            return []
        lens = [s.length for s in seqs]
        rs = self.block_mgr.step_decode([s.req_id for s in seqs], lens)
        self._h_ids.numpy()[:B] = [s.last_token for s in seqs]
        self._h_pos.numpy()[:B] = lens
        self._h_ctx.numpy()[:B] = [l + 1 for l in lens]
        self._h_row.numpy()[:B] = rs[:B]
        self._h_slots.numpy()[:B] = rs[B:]
        ev = None
        if self.profile_events and self.device.type == "cuda":
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        h2d = self._apply_block_table_patches()
        nxt, _ = self.executor.decode(self._h_ids[:B], self._h_pos[:B], self._h_slots[:B], self._h_ctx[:B], self._h_row[:B])
        self._h_out[:B].copy_(nxt, non_blocking=True)
        if ev is not None:
            ev[1].record()
            self.event_pairs.append(ev)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        toks = self._h_out[:B].tolist()
        now = time.time()
        res = []
        for s, tok in zip(seqs, toks):
            s.length += 1
            self._record(s, tok, now)
            res.append((s.req_id, tok))
        self.h2d_bytes_last += h2d + B * 24
        self.d2h_bytes_last += B * 4
        return res

    def step(self) -> List[Tuple[int, int]]:
        """One engine iteration: prefill newly admitted requests (if any), else one decode token for every running
        sequence. Returns (req_id, token) pairs produced by this step."""
        self.h2d_bytes_last = self.d2h_bytes_last = 0
        self.steps += 1
        # prefill and decode steps alternate while both have work, so a burst of arrivals cannot stall the running
        # sequences for more than one prefill step (bounds the inter-token latency tail)
        want_prefill = self.waiting and len(self.running) < self.max_batch_size
        if want_prefill and not (self._last_was_prefill and self.running):
            out = self._prefill()
            if out:
                self._last_was_prefill = True
                return out
        self._last_was_prefill = False
        return self._decode()

    # ---- serving-state snapshot ----------------------------------------------------------------------------------
    def save_state(self, path: str) -> None:
        """Writes the request table and the KV pages of every live sequence (between two steps). A new engine with the
        same weights continues from it with :meth:`load_state` and produces the same tokens."""
        seqs = []
        for s in self.running.values():
            blocks = self.block_mgr.get_seq_block_list(s.req_id)
            pages = self.executor.kv_cache[:, :, torch.tensor(blocks, device=self.device)].cpu()
            seqs.append(dict(req_id=s.req_id, prompt=s.prompt, max_new_tokens=s.max_new_tokens, length=s.length,
                             last_token=s.last_token, outputs=list(s.outputs), pages=pages))
        waiting = [dict(req_id=s.req_id, prompt=s.prompt, max_new_tokens=s.max_new_tokens) for s in self.waiting]
        finished = {r: list(s.outputs) for r, s in self.finished.items()}
        tmp = path + ".tmp"
        torch.save(dict(running=seqs, waiting=waiting, finished=finished, block_size=self.block_size), tmp)
        import os
        os.replace(tmp, path)

    def load_state(self, path: str) -> None:
        st = torch.load(path, map_location="cpu", weights_only=True)   # plain containers + tensors only
        assert st["block_size"] == self.block_size and not self.running and not self.waiting
        for d in st["running"]:
            s = _Seq(d["req_id"], d["prompt"], d["max_new_tokens"], length=d["length"], last_token=d["last_token"],
                     outputs=list(d["outputs"]), t_arrival=time.time())
            self.block_mgr.allocate(s.req_id, s.length + 1)
            blocks = self.block_mgr.get_seq_block_list(s.req_id)
            n = d["pages"].shape[2]
            self.executor.kv_cache[:, :, torch.tensor(blocks[:n], device=self.device)] = d["pages"].to(self.device)
            self.running[s.req_id] = s
        for d in st["waiting"]:
            self.add_request(d["req_id"], d["prompt"], d["max_new_tokens"])
        for r, outs in st["finished"].items():
            self.finished[r] = _Seq(r, [], len(outs), outputs=list(outs))
        self._apply_block_table_patches()

    def launch_count(self) -> int:
        from ..ops import _lib
        return _lib.LAUNCHES

    def tokens_per_step(self) -> int:
        return len(self.running)

    def run_until_done(self, max_steps: int = 1 << 30) -> Dict[int, List[int]]:
        n = 0
        while self.has_unfinished() and n < max_steps:
            self.step()
            n += 1
        return {r: s.outputs for r, s in self.finished.items()}
