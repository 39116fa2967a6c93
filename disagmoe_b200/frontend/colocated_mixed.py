"""Single-GPU serving engine with mixed batches: every step carries one decode token per running sequence plus prompt
tokens up to a budget, and long prompts are prefilled in chunks over several steps.

Same executor, block manager and staging buffers as :class:`ColocatedEngine`; the scheduling is the
:class:`disagmoe_b200.parallel.serving.FusedScheduler` of the multi-GPU serving path with one micro-batch. Compared
with alternating whole-prompt prefill steps and decode steps, a burst of arrivals delays the running sequences by at
most ``prefill_budget`` prompt rows per step. Steps without prompt rows replay the decode CUDA graph; steps with prompt
rows launch eagerly through the executor's general token path.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Tuple

import torch

from ..config import CacheConfig, ModelConfig
from ..parallel.serving import FusedScheduler, PyFusedScheduler, ServeSeq, make_seq
from .colocated import ColocatedEngine


class MixedBatchEngine(ColocatedEngine):
    def __init__(self, cfg: ModelConfig, cache_cfg: Optional[CacheConfig] = None, device="cuda", max_batch_size: int = 256,
                 max_prefill_tokens: int = 4096, prefill_budget: int = 512, **kw):
        super().__init__(cfg, cache_cfg, device=device, max_batch_size=max_batch_size,
                         max_prefill_tokens=max_prefill_tokens, **kw)
        self.row_cap = self.executor.prefill_buf.cap          # rows of one step: decode rows + prompt rows
        assert self.row_cap > max_batch_size, "max_prefill_tokens must leave room for prompt rows next to the decode rows"
        self.sched = FusedScheduler(self.block_mgr, self.block_size, 1, max_batch_size, self.row_cap,
                                    min(prefill_budget, self.row_cap - max_batch_size), ignore_eos=self.ignore_eos)

    # ---- requests -----------------------------------------------------------------------------------------------
    def add_request(self, req_id: int, prompt_ids: List[int], max_new_tokens: int) -> None:
        assert len(prompt_ids) >= 1 and len(prompt_ids) + max_new_tokens <= self.cfg.max_seq_len
        self.sched.add_request(req_id, prompt_ids, max_new_tokens, time.time())

    def add_synthetic_request(self, *a, **kw):
        raise NotImplementedError("synthetic KV histories belong to the decode benchmark engine (ColocatedEngine)")

    def has_unfinished(self) -> bool:
        return self.sched.num_unfinished() > 0

    @property
    def finished(self) -> Dict[int, ServeSeq]:
        return self.sched.finished

    @finished.setter
    def finished(self, value) -> None:       # the base constructor assigns an empty dict
        pass

    def tokens_per_step(self) -> int:
        return sum(len(r) for r in self.sched.running)

    # ---- one step -----------------------------------------------------------------------------------------------
    def step(self) -> List[Tuple[int, int]]:
        self.h2d_bytes_last = self.d2h_bytes_last = 0
        self.steps += 1
        plans = self.sched.build(time.time())
        p = plans[0]
        T = len(p)
        if T == 0:
            return []
        h2d = self._apply_block_table_patches()
        self._h_ids.numpy()[:T] = p.ids
        self._h_pos.numpy()[:T] = p.pos
        self._h_ctx.numpy()[:T] = [x + 1 for x in p.pos]
        self._h_row.numpy()[:T] = p.rows
        self._h_slots.numpy()[:T] = p.slots
        decode_only = all(row >= 0 and grown == 1 and s.length >= len(s.prompt) for row, s, grown in p.emit)
        args = (self._h_ids[:T], self._h_pos[:T], self._h_slots[:T], self._h_ctx[:T], self._h_row[:T])
        nxt, _ = self.executor.decode(*args) if decode_only else self.executor.prefill(*args)
        self._h_out[:T].copy_(nxt[:T], non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        out = self.sched.commit(plans, [self._h_out[:T].tolist()], time.time())
        self.h2d_bytes_last += h2d + T * 24
        self.d2h_bytes_last += T * 4
        return out

    def run_until_done(self, max_steps: int = 1 << 30) -> Dict[int, List[int]]:
        n = 0
        while self.has_unfinished() and n < max_steps:
            self.step()
            n += 1
        return {r: s.outputs for r, s in self.sched.finished.items()}

    # ---- serving-state snapshot ----------------------------------------------------------------------------------
    def save_state(self, path: str) -> None:
        """Request table (running sequences with their prefill progress, waiting and finished requests) and the KV
        pages of every running sequence, taken between two steps. ``load_state`` on a fresh engine with the same weights
        continues with identical tokens."""
        import os
        running = []
        for s in self.sched.running[0].values():
            blocks = self.block_mgr.get_seq_block_list(s.req_id)
            pages = self.executor.kv_cache[:, :, torch.tensor(blocks, device=self.device)].cpu()
            running.append(dict(req_id=s.req_id, prompt=s.prompt, max_new_tokens=s.max_new_tokens, length=s.length,
                                last_token=s.last_token, outputs=list(s.outputs), t_arrival=s.t_arrival, pages=pages))
        waiting = [dict(req_id=s.req_id, prompt=s.prompt, max_new_tokens=s.max_new_tokens, t_arrival=s.t_arrival)
                   for s in self.sched.waiting]
        finished = {r: list(s.outputs) for r, s in self.sched.finished.items()}
        tmp = path + ".tmp"
        torch.save(dict(running=running, waiting=waiting, finished=finished, block_size=self.block_size), tmp)
        os.replace(tmp, path)

    def load_state(self, path: str) -> None:
        st = torch.load(path, map_location="cpu", weights_only=True)   # plain containers + tensors only
        assert st["block_size"] == self.block_size and self.sched.num_unfinished() == 0
        for d in st["running"]:
            native = not isinstance(self.sched, PyFusedScheduler)
            s = make_seq(d["req_id"], d["prompt"], d["max_new_tokens"], d["t_arrival"], native=native, mb=0,
                         length=d["length"], last_token=d["last_token"], outputs=list(d["outputs"]))
            # the same reservation a fresh admission makes: room for the whole prompt, the rest grows step by step
            self.block_mgr.allocate(s.req_id, max(len(s.prompt), s.length) + 1)
            blocks = self.block_mgr.get_seq_block_list(s.req_id)
            n = min(d["pages"].shape[2], len(blocks))
            self.executor.kv_cache[:, :, torch.tensor(blocks[:n], device=self.device)] = d["pages"][:, :, :n].to(self.device)
            self.sched.restore_running(0, s)
        for d in st["waiting"]:
            self.sched.add_request(d["req_id"], d["prompt"], d["max_new_tokens"], d["t_arrival"])
        for r, outs in st["finished"].items():
            native = not isinstance(self.sched, PyFusedScheduler)
            self.sched.restore_finished(make_seq(r, [], len(outs), 0.0, native=native, outputs=list(outs)))
        self._apply_block_table_patches()
