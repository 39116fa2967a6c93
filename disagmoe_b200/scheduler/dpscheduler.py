"""Admission control across attention DP replicas (reference: disagmoe/scheduler/dpscheduler.py:16-150).

A request is admitted to one replica and stays there (its KV cache is private to the replica). Every admitted
sequence reserves ``delta = ceil(seq_len / block_size)`` KV blocks on its replica until it is deleted. Policy
``max`` picks the replica with the most free blocks and makes the request wait while none has ``delta`` free;
``RR`` is round robin. Requests wait in FIFO order in an asyncio queue served by :meth:`waiting_loop`.
"""
from __future__ import annotations

import asyncio
from dataclasses import dataclass
from typing import Callable, Dict, List, Tuple

from ..utils.logger import get_logger


@dataclass
class RequestItem:
    func: Callable
    req_id: int
    args: Tuple


class DPScheduler:
    def __init__(self, dp_size: int, seq_len: int, block_size: int):
        self.dp_size = dp_size
        self.seq_len = seq_len
        self.block_size = block_size
        self.delta = (seq_len + block_size - 1) // block_size
        self.kv_cache_stats: List[int] = [0] * dp_size
        self.seq_ranks: Dict[int, int] = {}
        self._logger = get_logger("DPScheduler")
        self._loop_task = None
        self.reset()

    def reset(self) -> None:
        self.end_flag = False
        self.end_event = asyncio.Event()
        self.sch_event = asyncio.Event()
        self.waiting_queue: asyncio.Queue = asyncio.Queue()
        self._blocked = 0

    def start(self, stats: Dict[int, int]) -> None:
        """Must be called from a running event loop; ``stats`` maps replica rank -> free KV blocks."""
        self.init_kv_cache_stats(stats)
        self.reset()
        self._loop_task = asyncio.create_task(self.waiting_loop())

    async def terminate(self) -> None:
        self.end_flag = True
        self.end_event.set()
        if self._loop_task is not None:
            await self._loop_task

    def put_request(self, func: Callable, req_id: int, *args) -> None:
        """Queues ``func(req_id, *args, rank)`` to be called once a replica has room."""
        self.waiting_queue.put_nowait(RequestItem(func, req_id, args))

    async def waiting_loop(self) -> None:
        end_wait = asyncio.ensure_future(self.end_event.wait())
        try:
            while not self.end_flag:
                getter = asyncio.ensure_future(self.waiting_queue.get())
                await asyncio.wait([getter, end_wait], return_when=asyncio.FIRST_COMPLETED)
                if self.end_event.is_set():
                    getter.cancel()
                    break
                item: RequestItem = getter.result()
                rank = self.schedule([item.req_id])[0]
                while rank < 0 and not self.end_flag:
                    self._blocked += 1
                    waiter = asyncio.ensure_future(self.sch_event.wait())
                    await asyncio.wait([waiter, end_wait], return_when=asyncio.FIRST_COMPLETED)
                    self._blocked -= 1
                    waiter.cancel()
                    self.sch_event.clear()
                    if self.end_event.is_set():
                        return
                    rank = self.schedule([item.req_id])[0]
                item.func(item.req_id, *item.args, rank)
        finally:
            end_wait.cancel()

    def init_kv_cache_stats(self, stats: Dict[int, int]) -> None:
        for rank, blocks in stats.items():
            self.kv_cache_stats[rank] = blocks

    def add_seq(self, seq_id: int, rank: int) -> None:
        self.kv_cache_stats[rank] -= self.delta
        self.seq_ranks[seq_id] = rank

    def del_seq(self, seq_id: int) -> None:
        rank = self.seq_ranks.pop(seq_id)
        self.kv_cache_stats[rank] += self.delta
        if self._blocked > 0:
            self.sch_event.set()

    def _schedule(self) -> int:
        raise NotImplementedError

    def schedule(self, req_ids: List[int]) -> List[int]:
        ranks = []
        for rid in req_ids:
            r = self._schedule()
            ranks.append(r)
            if r >= 0:
                self.add_seq(rid, r)
        return ranks


class DPSchedulerMax(DPScheduler):
    """Most free KV blocks first; -1 (wait) when no replica can hold another sequence."""

    def _schedule(self) -> int:
        best = max(range(self.dp_size), key=lambda r: (self.kv_cache_stats[r], -r))
        return best if self.kv_cache_stats[best] >= self.delta else -1


class DPSChedulerRR(DPScheduler):
    def __init__(self, dp_size: int, seq_len: int, block_size: int):
        super().__init__(dp_size, seq_len, block_size)
        self.cur_rank = 0

    def _schedule(self) -> int:
        r = self.cur_rank
        self.cur_rank = (r + 1) % self.dp_size
        return r


_policies = {"RR": DPSChedulerRR, "max": DPSchedulerMax}


def get_dp_scheduler(dp_size: int, seq_len: int, block_size: int, policy: str) -> DPScheduler:
    return _policies[policy](dp_size, seq_len, block_size)
