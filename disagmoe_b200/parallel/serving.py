"""Continuous-batching serving on the fused disaggregated data plane (attention GPUs + expert GPUs, peer memory).

One process per GPU. Ranks [0, A) are attention GPUs in TP groups of ``tp`` consecutive ranks; ranks [A, world) hold
the routed experts. Every iteration of the job is one pass of two micro-batches through all layers
(:class:`disagmoe_b200.parallel.disagg.AttentionRank` / ``ExpertRank``):

* the **leader** of every attention group (its first rank) owns the group's requests: it admits arrivals, keeps the
  paged-KV block manager, and builds the iteration's two micro-batches as flat token lists. A running sequence
  contributes its next decode token; a newly admitted request contributes prompt tokens, all of them or, under the
  per-iteration prompt budget, one chunk per iteration (position p attends to the first p + 1 cached tokens of its own
  block-table row, so prompt and decode tokens share one kernel and one batch: prefill never stalls the sequences that
  are decoding, and a long prompt never waits for a micro-batch to empty);
* the other members of a TP group receive the leader's plan (token ids, positions, slots, block-table patches) over a
  host-side broadcast and run the same launches on their head shard;
* the expert GPUs replay one CUDA graph per iteration whatever the attention side scheduled: row counts travel with
  the data (per-expert cursors in peer memory), so the expert side has no shape to agree on.

Iterations are kept in lock step by one tiny host all-reduce per iteration (work left? any device status set?); token
rows, router decisions and expert outputs never touch the host. Decode-sized iterations replay a CUDA graph captured
for the padded micro-batch size; larger (prefill-heavy) iterations launch eagerly.

The reference's counterpart is the whole host-scheduled loop: disagmoe/frontend/engine.py:614-871 (attention / expert
loops), csrc/muhelper/muhelper.cpp (pools and dispatchers), disagmoe/frontend/controller.py:276-330 (request
admission and results).
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..config import ModelConfig
from ..frontend.datatypes import SloStat
from ..utils.constants import EOS_TOKEN_ID


# ------------------------------------------------------------------------------------------------ scheduling (host)
@dataclass
class ServeSeq:
    req_id: int
    prompt: List[int]
    max_new_tokens: int
    t_arrival: float
    mb: int = -1
    length: int = 0                 # tokens whose K/V are cached
    last_token: int = 0
    outputs: List[int] = field(default_factory=list)
    t_tokens: List[float] = field(default_factory=list)


@dataclass
class MicroBatchPlan:
    ids: List[int] = field(default_factory=list)
    pos: List[int] = field(default_factory=list)
    rows: List[int] = field(default_factory=list)
    slots: List[int] = field(default_factory=list)
    # (row in the micro-batch or -1, sequence, tokens this step adds to its cache): row >= 0 produces the sequence's next
    # token; row == -1 is a prompt chunk that is not the last one (cache grows, nothing is sampled)
    emit: List[Tuple[int, ServeSeq, int]] = field(default_factory=list)

    def __len__(self):
        return len(self.ids)


class PyFusedScheduler:
    """Admission + micro-batch construction of one attention group (pure host logic, no GPU). This is the Python
    statement of the policy; the serving path runs its C++ twin ``disagmoe_c.FusedScheduler``
    (csrc/runtime/fused_scheduler.cpp) through :func:`FusedScheduler`, and a CPU test holds the two to identical plans.

    Every iteration a micro-batch holds one decode token per running sequence plus prompt tokens up to two budgets:
    ``max_tokens_per_mb`` rows in total and ``max_prefill_tokens_per_mb`` prompt rows. A prompt that does not fit is
    processed in chunks over several iterations (chunk i attends to the K/V the earlier chunks cached; only the last
    chunk samples a token), so long prompts neither starve behind decode tokens nor stall them."""

    MIN_CHUNK = 16      # do not start or continue a prompt with fewer rows than this unless that finishes it

    def __init__(self, block_mgr, block_size: int, n_mb: int, max_seqs_per_mb: int, max_tokens_per_mb: int,
                 max_prefill_tokens_per_mb: Optional[int] = None, ignore_eos: bool = True):
        self.bm, self.block_size, self.n_mb = block_mgr, block_size, n_mb
        self.ignore_eos = ignore_eos          # False: a sampled EOS token (id 2) ends the request early
        self.max_seqs, self.max_tokens = max_seqs_per_mb, max_tokens_per_mb
        self.max_prefill = max_prefill_tokens_per_mb or max_tokens_per_mb
        assert self.max_tokens > self.max_seqs, "a micro-batch must have room for prompt rows next to its decode rows"
        self.waiting: List[ServeSeq] = []                     # arrival order
        self.running: List[Dict[int, ServeSeq]] = [dict() for _ in range(n_mb)]
        self.finished: Dict[int, ServeSeq] = {}
        self.pool_blocks = block_mgr.num_free_blocks()        # the scheduler is created on an empty pool

    def add_request(self, req_id: int, prompt: Sequence[int], max_new_tokens: int, t_arrival: float) -> None:
        assert len(prompt) >= 1 and max_new_tokens >= 1
        if self._blocks(len(prompt) + max_new_tokens) > self.pool_blocks:
            raise ValueError(f"request {req_id} needs more KV blocks than the pool has")
        self.waiting.append(ServeSeq(req_id, list(prompt), max_new_tokens, t_arrival))

    def num_unfinished(self) -> int:
        return len(self.waiting) + sum(len(r) for r in self.running)

    def has_work(self, now: float) -> bool:
        return any(len(r) for r in self.running) or bool(self.waiting and self.waiting[0].t_arrival <= now)

    def _blocks(self, tokens: int) -> int:
        return (tokens + self.block_size - 1) // self.block_size

    def _growth_reserve(self) -> int:
        """KV blocks the running sequences will still take before they finish. Admission leaves them free, so that a
        decode step can never find the pool empty (there is no preemption)."""
        return sum(max(0, self._blocks(len(s.prompt) + s.max_new_tokens) - len(self.bm.get_seq_block_list(s.req_id)))
                   for r in self.running for s in r.values())

    def _add_prompt_rows(self, p: MicroBatchPlan, s: ServeSeq, budget: int) -> int:
        """Appends the next prompt rows of ``s`` (at most ``budget``) to the plan; returns how many."""
        n, done = len(s.prompt), s.length
        take = min(n - done, budget)
        if take <= 0 or (take < self.MIN_CHUNK and take < n - done):
            return 0
        row = self.bm.row_of(s.req_id)
        blocks = self.bm.get_seq_block_list(s.req_id)
        bs = self.block_size
        p.ids.extend(s.prompt[done:done + take])
        p.pos.extend(range(done, done + take))
        p.rows.extend([row] * take)
        p.slots.extend(blocks[i // bs] * bs + i % bs for i in range(done, done + take))
        last = done + take == n
        p.emit.append((len(p.ids) - 1 if last else -1, s, take))
        return take

    def build(self, now: float) -> List[MicroBatchPlan]:
        plans = [MicroBatchPlan() for _ in range(self.n_mb)]
        prefill = [0] * self.n_mb
        budget = lambda m: min(self.max_tokens - len(plans[m]), self.max_prefill - prefill[m])
        for m in range(self.n_mb):
            seqs = [s for s in self.running[m].values() if s.length >= len(s.prompt)]      # fully prefilled
            if seqs:
                lens = [s.length for s in seqs]
                rs = self.bm.step_decode([s.req_id for s in seqs], lens)
                n = len(seqs)
                p = plans[m]
                p.ids = [s.last_token for s in seqs]
                p.pos = lens
                p.rows = [int(r) for r in rs[:n]]
                p.slots = [int(r) for r in rs[n:]]
                p.emit = [(i, q, 1) for i, q in enumerate(seqs)]
            # prompts that are part-way through, oldest first
            for s in [s for s in self.running[m].values() if s.length < len(s.prompt)]:
                prefill[m] += self._add_prompt_rows(plans[m], s, budget(m))
        # admission in arrival order; a request goes to the micro-batch with more room this iteration
        while self.waiting and self.waiting[0].t_arrival <= now:
            s = self.waiting[0]
            n = len(s.prompt)
            order = sorted(range(self.n_mb), key=lambda m: (-budget(m), len(plans[m]), len(self.running[m])))
            m = next((m for m in order if len(self.running[m]) < self.max_seqs
                      and budget(m) >= min(n, self.MIN_CHUNK)), None)
            if m is None or self.bm.num_free_blocks() - self._growth_reserve() < self._blocks(n + s.max_new_tokens):
                break
            self.waiting.pop(0)
            self.bm.allocate(s.req_id, n + 1)
            s.mb = m
            self.running[m][s.req_id] = s
            prefill[m] += self._add_prompt_rows(plans[m], s, budget(m))
        return plans

    def commit(self, plans: List[MicroBatchPlan], next_ids: List[Sequence[int]], now: float) -> List[Tuple[int, int]]:
        out = []
        for m, p in enumerate(plans):
            for row, s, grown in p.emit:
                s.length += grown
                if row < 0:
                    continue
                tok = int(next_ids[m][row])
                s.outputs.append(tok)
                s.t_tokens.append(now)
                s.last_token = tok
                out.append((s.req_id, tok))
                if len(s.outputs) >= s.max_new_tokens or (not self.ignore_eos and tok == EOS_TOKEN_ID):
                    self.bm.release(s.req_id)
                    self.running[m].pop(s.req_id, None)
                    self.finished[s.req_id] = s
        return out


    def restore_running(self, mb: int, s: ServeSeq) -> None:
        s.mb = mb
        self.running[mb][s.req_id] = s

    def restore_finished(self, s: ServeSeq) -> None:
        self.finished[s.req_id] = s


def FusedScheduler(block_mgr, block_size: int, n_mb: int, max_seqs_per_mb: int, max_tokens_per_mb: int,
                   max_prefill_tokens_per_mb: Optional[int] = None, ignore_eos: bool = True, native: Optional[bool] = None):
    """The serving scheduler of one attention group: the native implementation (C++, next to the block manager it
    drives) unless ``native=False`` or DMOE_PY_SCHEDULER=1 asks for the Python one. Both expose ``add_request``,
    ``has_work``, ``num_unfinished``, ``build``, ``commit``, ``restore_running`` / ``restore_finished`` and the
    ``waiting`` / ``running`` / ``finished`` views."""
    if native is None:
        native = os.environ.get("DMOE_PY_SCHEDULER", "") != "1"
    if native:
        from .. import disagmoe_c as C
        return C.FusedScheduler(block_mgr, block_size, n_mb, max_seqs_per_mb, max_tokens_per_mb,
                                max_prefill_tokens_per_mb or 0, ignore_eos)
    return PyFusedScheduler(block_mgr, block_size, n_mb, max_seqs_per_mb, max_tokens_per_mb, max_prefill_tokens_per_mb,
                            ignore_eos)


def make_seq(req_id: int, prompt, max_new_tokens: int, t_arrival: float = 0.0, native: bool = True, **kw):
    """A sequence record for ``restore_running`` / ``restore_finished`` of the scheduler flavour in use."""
    if native:
        from .. import disagmoe_c as C
        return C.FusedSeq(req_id, list(prompt), max_new_tokens, t_arrival, **kw)
    return ServeSeq(req_id, list(prompt), max_new_tokens, t_arrival, **kw)


# ------------------------------------------------------------------------------------------------ host-only stand-ins
class HostOnlyAttention:
    """Stands in for the GPU side of an attention rank in host-only runs (CPU processes, no kernels): the same buffers
    as ``AttentionRank``; the "model" maps (token, position) to the next token deterministically."""

    def __init__(self, srv: "FusedServingRank", vocab: int):
        z = lambda n, dt=torch.int32: torch.zeros(n, dtype=dt)
        self.mb = [dict(ids=z(srv.cap), positions=z(srv.cap), ctx_len=z(srv.cap), bt_row=z(srv.cap),
                        slots=z(srv.cap, torch.int64), next_ids=z(srv.cap)) for _ in range(srv.n_mb)]
        self.block_tables = torch.zeros(2 * srv.cap + 8, 64, dtype=torch.int32)
        self.layers: List = []
        self.active = [srv.cap] * srv.n_mb
        self.vocab = vocab

    @staticmethod
    def next_token(token: int, position: int, vocab: int) -> int:
        return (token * 7 + position * 3 + 1) % vocab

    def set_active(self, m: int, T: int) -> None:
        self.active[m] = T

    def iteration(self) -> None:
        for m, d in enumerate(self.mb):
            T = self.active[m]
            d["next_ids"][:T] = (d["ids"][:T] * 7 + d["positions"][:T] * 3 + 1) % self.vocab


class HostOnlyExpert:
    def iteration(self) -> None:
        pass


def host_only_runner(vocab: int):
    """``host_only_runner`` argument of :class:`FusedServingRank` for dry runs of the host protocol on CPU."""
    return lambda role, srv: HostOnlyAttention(srv, vocab) if role == "attention" else HostOnlyExpert()


# ------------------------------------------------------------------------------------------------ one rank of the job
class FusedServingRank:
    """One process of the fused disaggregated serving job (see the module docstring for the roles)."""

    def __init__(self, cfg: ModelConfig, world: int, rank: int, local_rank: int, n_attn: int, tp: int = 1,
                 max_seqs_per_mb: int = 128, max_tokens_per_mb: int = 2048, num_blocks: int = 8192,
                 graph_sizes: Sequence[int] = (8, 32, 64, 128, 256), n_mb: int = 2, route_skew: float = 0.0,
                 max_prefill_tokens_per_mb: Optional[int] = None, state_dict=None, host_only_runner=None,
                 ignore_eos: bool = True):
        """``host_only_runner(role, server)`` replaces the GPU side (peer arena, attention / expert ranks, CUDA graphs)
        with a stand-in that offers the same buffers and ``iteration()``: the host protocol (control all-reduce, plan
        sharing inside a TP group, scheduling, result collection) then runs as plain CPU processes."""
        import torch.distributed as dist
        from .. import disagmoe_c as C
        from ..ops import _lib, gemm
        from .disagg import AttentionRank, DisaggShape, ExpertRank, build_layout
        from .peer import PeerArena
        self.dist, self._lib, self._gemm = dist, _lib, gemm
        A, X = n_attn, world - n_attn
        assert 1 <= A < world and A % tp == 0
        self.cfg, self.world, self.rank, self.A, self.X, self.tp, self.n_mb = cfg, world, rank, A, X, tp, n_mb
        self.host_only = host_only_runner is not None
        self.device = torch.device("cpu") if self.host_only else torch.device("cuda", local_rank)
        self.is_attn = rank < A
        self.is_leader = self.is_attn and rank % tp == 0
        self.cap = max_tokens_per_mb
        self.block_size = 16
        self.shape = DisaggShape(A, X, n_mb, self.cap, cfg.top_k, cfg.hidden_size, cfg.num_experts, tp)
        self.layout = build_layout(self.shape)
        self.arena = None if self.host_only else PeerArena.create(self.layout.size, device=self.device)
        # host control plane: gloo (keeps the CUDA streams free of control collectives). Every rank calls it at least
        # every iteration (idle ranks poll), so a collective that waits two minutes means a rank is gone: the others
        # then fail with a timeout instead of waiting forever
        import datetime
        self.ctl = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=120))
        self.leader_rank = rank // tp * tp if self.is_attn else -1
        self.graph_sizes = [] if self.host_only else sorted(g for g in graph_sizes if g <= self.cap)
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.iterations = 0
        self.graph_iterations = 0
        # per iteration: (start s, end s, rows of every micro-batch, graph size or 0 for an eager launch)
        self.step_log: List[Tuple[float, float, Tuple[int, ...], int]] = []
        if self.is_attn:
            # one block beyond the manager's range is the scratch page the padding rows write to
            self.runner = host_only_runner("attention", self) if self.host_only else \
                AttentionRank(cfg, self.shape, self.arena, self.layout, rank, num_blocks + 1, state_dict=state_dict)
            for layer in self.runner.layers:
                layer.set_route_skew(route_skew)
            self.scratch_block = num_blocks
            self.max_rows = n_mb * max_seqs_per_mb
            self.dummy_row = self.max_rows                      # a block-table row that only names the scratch page
            assert self.runner.block_tables.shape[0] > self.dummy_row
            self.runner.block_tables[self.dummy_row].fill_(self.scratch_block)
            self.sched = None
            if self.is_leader:
                self.bm = C.BlockManager(self.block_size, num_blocks, 0, self.max_rows)
                self.sched = FusedScheduler(self.bm, self.block_size, n_mb, max_seqs_per_mb, self.cap,
                                            max_prefill_tokens_per_mb, ignore_eos)
            n = n_mb * self.cap
            pin = lambda dt: torch.zeros(n, dtype=dt) if self.host_only else torch.zeros(n, dtype=dt).pin_memory()
            self.h_ids, self.h_pos, self.h_ctx, self.h_row = (pin(torch.int32) for _ in range(4))
            self.h_slots = pin(torch.int64)
            self.h_out = pin(torch.int32)
        else:
            self.runner = host_only_runner("expert", self) if self.host_only else \
                ExpertRank(cfg, self.shape, self.arena, self.layout, rank - A, state_dict=state_dict)
        self._last_status = 0
        self._sync()
        dist.barrier()
        self._debug = bool(os.environ.get("DMOE_SERVE_DEBUG"))
        self._log("set-up done")
        self._warm_up_and_capture()
        self._log("graphs captured")

    def _sync(self) -> None:
        if not self.host_only:
            torch.cuda.synchronize()

    def _status_word(self) -> int:
        return 0 if self.host_only else int(self._gemm.scratch(self.device).status.item())

    def _log(self, msg: str) -> None:
        if self._debug:
            print(f"[serve rank {self.rank} it {self.iterations}] {msg}", file=sys.stderr, flush=True)

    # ---- set-up ------------------------------------------------------------------------------------------------
    def _fill_padding(self, m: int, start: int, end: int) -> None:
        """Rows [start, end) of micro-batch m become padding: token 0 at position 0 of the scratch page."""
        sl = slice(m * self.cap + start, m * self.cap + end)
        self.h_ids[sl] = 0
        self.h_pos[sl] = 0
        self.h_ctx[sl] = 1
        self.h_row[sl] = self.dummy_row
        self.h_slots[sl] = self.scratch_block * self.block_size

    def _upload(self, m: int, T: int) -> None:
        d = self.runner.mb[m]
        sl = slice(m * self.cap, m * self.cap + T)
        d["ids"][:T].copy_(self.h_ids[sl], non_blocking=True)
        d["positions"][:T].copy_(self.h_pos[sl], non_blocking=True)
        d["ctx_len"][:T].copy_(self.h_ctx[sl], non_blocking=True)
        d["bt_row"][:T].copy_(self.h_row[sl], non_blocking=True)
        d["slots"][:T].copy_(self.h_slots[sl], non_blocking=True)

    def _warm_up_and_capture(self) -> None:
        dist = self.dist
        g0 = self.graph_sizes[0] if self.graph_sizes else 1
        # eager iterations in lock step (scratch buffers, kernel attributes), then capture; capture runs no kernel,
        # so the ranks need not agree on how many graphs each of them captures
        # the first one runs at full capacity so that every scratch buffer reaches its final size before any capture
        for size in (self.cap, g0):
            if self.is_attn:
                for m in range(self.n_mb):
                    self._fill_padding(m, 0, size)
                    self._upload(m, size)
                    self.runner.set_active(m, size)
            self.runner.iteration()
            self._sync()
            self._log(f"eager warm-up iteration done, status {self._status_word()}")
            dist.barrier()
        if self.host_only:
            self.launches_per_graph = 0
            return
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream())
        n0 = self._lib.LAUNCHES
        if self.is_attn:
            for g in self.graph_sizes:
                for m in range(self.n_mb):
                    self.runner.set_active(m, g)
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=side):
                    self.runner.iteration()
                self.graphs[g] = gr
            self.launches_per_graph = (self._lib.LAUNCHES - n0) // max(1, len(self.graph_sizes))
        else:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=side):
                self.runner.iteration()
            self.graphs[0] = gr
            self.launches_per_graph = self._lib.LAUNCHES - n0
        torch.cuda.synchronize()
        dist.barrier()

    # ---- requests (leaders) --------------------------------------------------------------------------------------
    def add_request(self, req_id: int, prompt: Sequence[int], max_new_tokens: int, t_arrival: float) -> None:
        assert self.is_leader
        if len(prompt) + max_new_tokens > self.cfg.max_seq_len:
            # the block table has max_seq_len / block_size columns: a longer sequence must be refused here, on the host
            raise ValueError(f"request {req_id}: {len(prompt)} prompt + {max_new_tokens} new tokens exceed "
                             f"max_seq_len {self.cfg.max_seq_len}")
        self.sched.add_request(req_id, prompt, max_new_tokens, t_arrival)

    # ---- one iteration -------------------------------------------------------------------------------------------
    def _pack_plan(self, Ts: List[int], patches: Optional[torch.Tensor]) -> torch.Tensor:
        n_patch = 0 if patches is None else patches.shape[1]
        buf = torch.empty(5 * sum(Ts) + 3 * n_patch, dtype=torch.int64)
        o = 0
        for m, T in enumerate(Ts):
            sl = slice(m * self.cap, m * self.cap + T)
            for h in (self.h_ids, self.h_pos, self.h_ctx, self.h_row, self.h_slots):
                buf[o:o + T] = h[sl]
                o += T
        if n_patch:
            buf[o:] = patches.reshape(-1)
        return buf

    def _unpack_plan(self, buf: torch.Tensor, Ts: List[int], n_patch: int) -> Optional[torch.Tensor]:
        o = 0
        for m, T in enumerate(Ts):
            sl = slice(m * self.cap, m * self.cap + T)
            for h in (self.h_ids, self.h_pos, self.h_ctx, self.h_row, self.h_slots):
                h[sl] = buf[o:o + T].to(h.dtype)
                o += T
        return buf[o:].reshape(3, n_patch) if n_patch else None

    def _plan_to_host(self, plans: List[MicroBatchPlan]) -> List[int]:
        Ts = []
        for m, p in enumerate(plans):
            T = len(p)
            o = m * self.cap
            if T and hasattr(p, "copy_to"):
                p.copy_to(self.h_ids, self.h_pos, self.h_ctx, self.h_row, self.h_slots, o)   # native plan: one pass in C++
            elif T:
                self.h_ids.numpy()[o:o + T] = p.ids
                self.h_pos.numpy()[o:o + T] = p.pos
                self.h_ctx.numpy()[o:o + T] = np.asarray(p.pos, dtype=np.int32) + 1
                self.h_row.numpy()[o:o + T] = p.rows
                self.h_slots.numpy()[o:o + T] = p.slots
            Ts.append(T)
        return Ts

    def step(self, now: float) -> Optional[List[Tuple[int, int]]]:
        """One lock-step iteration of the whole job. Returns None when the job is over (no request left anywhere, or
        a device-side wait gave up), [] when nothing was ready to run, else the (request, token) pairs this rank's
        group produced (leaders only).

        Host protocol, all over one gloo group of every rank (sub-groups are avoided on purpose: creating a gloo
        sub-group under an eagerly initialised NCCL world blocked its members): one all-gather of a small header per
        rank [requests unfinished, work ready now, device status set, rows of every micro-batch, block-table patches],
        then, with tensor parallelism, one broadcast per TP group of the leader's staged token arrays, which the
        members of that group keep and everybody else drops."""
        n_mb = self.n_mb
        hdr = torch.zeros(4 + n_mb, dtype=torch.int64)
        plans, Ts, patches = None, [0] * n_mb, None
        if self.is_leader:
            hdr[0] = self.sched.num_unfinished()
            hdr[1] = int(self.sched.has_work(now))
            if hdr[1]:
                plans = self.sched.build(now)
                Ts = self._plan_to_host(plans)
                ups = self.bm.drain_updates()
                if ups:
                    patches = torch.tensor(ups, dtype=torch.int64).T.contiguous()
                hdr[3:3 + n_mb] = torch.tensor(Ts)
                hdr[3 + n_mb] = 0 if patches is None else patches.shape[1]
        hdr[2] = int(self._last_status != 0)
        every = [torch.zeros_like(hdr) for _ in range(self.world)]
        self.dist.all_gather(every, hdr, group=self.ctl)
        unfinished = sum(int(h[0]) for h in every)
        ready = sum(int(h[1]) for h in every)
        bad = sum(int(h[2]) for h in every)
        if unfinished == 0 or bad:
            return None
        if ready == 0:
            time.sleep(0.0005)
            return []
        self.iterations += 1
        if self._debug and self.iterations <= 3:
            self._log(f"iteration starts (unfinished {unfinished}, ready {ready})")
        if self.tp > 1:
            for lead in range(0, self.A, self.tp):
                h = every[lead]
                lTs, n_patch = [int(x) for x in h[3:3 + n_mb]], int(h[3 + n_mb])
                size = 5 * sum(lTs) + 3 * n_patch
                if size == 0:
                    continue
                buf = self._pack_plan(Ts, patches) if self.rank == lead else torch.empty(size, dtype=torch.int64)
                self.dist.broadcast(buf, src=lead, group=self.ctl)
                if self.leader_rank == lead and not self.is_leader:
                    Ts = lTs
                    patches = self._unpack_plan(buf, lTs, n_patch)
        if not self.is_attn:
            if self.host_only:
                self.runner.iteration()
            else:
                self.graphs[0].replay()
                self._lib.add_launches(self.launches_per_graph)
                torch.cuda.current_stream().synchronize()
                self._last_status = self._status_word()
            return []
        if patches is not None:
            t = patches if self.host_only else patches.pin_memory().to(self.device, non_blocking=True)
            self.runner.block_tables.index_put_((t[0], t[1]), t[2].int())
        t_begin = time.time()
        # decode-sized iterations replay the graph of the padded size; bigger ones launch eagerly at the exact size
        tmax = max(max(Ts), 1)
        g = next((s for s in self.graph_sizes if s >= tmax), None)
        for m, T in enumerate(Ts):
            size = g if g is not None else min(self.cap, (max(T, 1) + 15) // 16 * 16)
            self._fill_padding(m, T, size)
            self._upload(m, size)
            self.runner.set_active(m, size)
            if not self.host_only:
                # eager (prefill-heavy) iterations send their prompt segments through the tiled causal attention
                # kernel; graph replays were captured without it
                sl = slice(m * self.cap, m * self.cap + size)
                if g is None:
                    self.runner.set_prefill_tiles(m, self.h_row[sl], self.h_pos[sl], self.h_ctx[sl])
                else:
                    self.runner.set_prefill_tiles(m, None, None, None)
        if g is not None:
            self.graphs[g].replay()
            self._lib.add_launches(self.launches_per_graph)
            self.graph_iterations += 1
        else:
            self.runner.iteration()
        for m, T in enumerate(Ts):
            if T:
                self.h_out[m * self.cap:m * self.cap + T].copy_(self.runner.mb[m]["next_ids"][:T], non_blocking=True)
        if not self.host_only:
            torch.cuda.current_stream().synchronize()
            self._last_status = self._status_word()
        self.step_log.append((t_begin, time.time(), tuple(Ts), g or 0))
        if not self.is_leader:
            return []
        if plans is None:
            return []
        outs = [self.h_out[m * self.cap:m * self.cap + T].tolist() for m, T in enumerate(Ts)]
        return self.sched.commit(plans, outs, time.time())

    def kernel_status(self) -> int:
        return 0 if self.host_only else (self._gemm.check_status(self.device) or self._last_status)

    # ---- a whole workload ----------------------------------------------------------------------------------------
    def serve(self, requests: Sequence[Tuple[int, Sequence[int], int, float]], time_limit: float = 600.0
              ) -> Dict[str, object]:
        """Runs until every request of every group is finished. ``requests``: (req_id, prompt ids, output length,
        arrival offset in seconds) of THIS rank's group (leaders; ignored elsewhere). Returns this rank's results."""
        dist = self.dist
        dist.barrier(group=self.ctl)
        t0 = time.time()
        problem = ""
        if self.is_leader:
            try:
                for rid, prompt, n_out, at in requests:
                    self.add_request(rid, prompt, n_out, t0 + at)
            except ValueError as e:
                problem = str(e)
        # a request one leader has to refuse ends the job on every rank, before anybody waits for anybody
        flag = torch.tensor([1 if problem else 0], dtype=torch.int64)
        dist.all_reduce(flag, group=self.ctl)
        if int(flag) > 0:
            raise ValueError(problem or "another attention group refused one of its requests")
        tokens = 0
        while True:
            now = time.time()
            if now - t0 > time_limit:
                raise TimeoutError("serving run exceeded its time limit")
            out = self.step(now)
            if out is None:
                break
            tokens += len(out)
        self._sync()
        dt = time.time() - t0
        res = {"rank": self.rank, "duration": dt, "tokens": tokens, "iterations": self.iterations,
               "graph_iterations": self.graph_iterations, "kernel_status": self.kernel_status(), "slo": [], "arrivals": {},
               "step_log": list(self.step_log)}
        if self.is_leader:
            for s in self.sched.finished.values():
                res["slo"].append(SloStat(s.req_id, s.t_tokens[0], 0.0, s.t_tokens[-1], list(s.t_tokens)))
                res["arrivals"][s.req_id] = s.t_arrival
            res["outputs"] = {s.req_id: list(s.outputs) for s in self.sched.finished.values()}
        return res
