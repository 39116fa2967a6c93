"""Cluster controller: spawns one worker process per device, wires them up from a ``ModelPlacement`` and drives
requests through the tokenizer / sampler pair.

Counterpart of disagmoe/frontend/controller.py:46-432 and ray_helper.py. Ray is replaced by plain processes
(``multiprocessing`` spawn) with a pipe-based RPC: ``worker.call("method", *args)``. The tokenizer and the sampler are
native objects living in the controller process. NCCL unique ids are minted per edge only when the workers are CUDA
devices; CPU workers use the socket transport (the tensor bytes ride in the control message).
"""
from __future__ import annotations

import multiprocessing as mp
import os
import random
import threading
import time
import traceback
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

from .. import disagmoe_c as C
from ..config import CacheConfig, ModelConfig, SamplingConfig
from ..scheduler.dpscheduler import get_dp_scheduler
from ..utils.constants import SAMPLER_DEV_ID, TOKENIZER_DEV_ID
from ..utils.logger import get_logger
from ..utils.placement import ModelPlacement
from .datatypes import SloStat
from .engine import Engine, InitCoreArgs, SamplerEngine, TokenizerEngine


def _worker_main(conn, device_id: int, device: str, env: Dict[str, str]) -> None:
    os.environ.update(env)
    eng = Engine(device_id, device)
    while True:
        try:
            msg = conn.recv()
        except EOFError:
            break
        if msg is None:
            break
        method, args, kwargs = msg
        try:
            res = getattr(eng, method)(*args, **kwargs)
            conn.send(("ok", res))
        except Exception:
            conn.send(("err", traceback.format_exc()))
    try:
        eng.terminate()
    except Exception:
        pass


class ConnWorker:
    """Method-call stub over a ``multiprocessing`` connection: one request in flight at a time (``call_async`` takes
    the lock, ``wait`` returns it). Sub-classes say how the worker was started and how to tell whether it is alive."""

    device_id: int

    def _init_conn(self, conn) -> None:
        self.conn = conn
        self.lock = threading.Lock()
        self._dead = False

    def call_async(self, method: str, *args, **kwargs) -> None:
        self.lock.acquire()
        try:
            self.conn.send((method, args, kwargs))
        except (OSError, ValueError) as e:
            self.lock.release()
            self._dead = True
            raise RuntimeError(f"worker {self.device_id} is gone: {e}")

    def wait(self, timeout: float = 300.0):
        try:
            if not self.conn.poll(timeout):
                raise TimeoutError(f"worker {self.device_id} did not answer within {timeout} s")
            try:
                status, res = self.conn.recv()
            except (EOFError, OSError) as e:
                self._dead = True
                raise RuntimeError(f"worker {self.device_id} is gone: {e}")
        finally:
            self.lock.release()
        if status != "ok":
            raise RuntimeError(f"worker {self.device_id} failed:\n{res}")
        return res

    def call(self, method: str, *args, timeout: float = 300.0, **kwargs):
        self.call_async(method, *args, **kwargs)
        return self.wait(timeout)

    def _send_stop(self) -> None:
        try:
            if self.lock.acquire(timeout=5):
                try:
                    self.conn.send(None)
                finally:
                    self.lock.release()
        except Exception:
            pass


class WorkerHandle(ConnWorker):
    """A worker process on this machine, reached through a pipe."""

    def __init__(self, device_id: int, device: str, env: Optional[Dict[str, str]] = None):
        ctx = mp.get_context("spawn")
        self.device_id = device_id
        conn, child = ctx.Pipe()
        self.proc = ctx.Process(target=_worker_main, args=(child, device_id, device, env or {}), daemon=True)
        self.proc.start()
        self._init_conn(conn)

    def alive(self) -> bool:
        return self.proc.is_alive()

    def stop(self) -> None:
        self._send_stop()
        self.proc.join(timeout=10)
        if self.proc.is_alive():
            self.proc.terminate()


class LocalWorker:
    """Same interface as ``WorkerHandle`` for an engine living in the controller process (single-process runs)."""

    def __init__(self, device_id: int, device: str):
        self.device_id = device_id
        self.engine = Engine(device_id, device)
        self._res = None

    def call_async(self, method, *args, **kwargs):
        self._res = getattr(self.engine, method)(*args, **kwargs)

    def wait(self, timeout: float = 300.0):
        return self._res

    def call(self, method, *args, timeout: float = 300.0, **kwargs):
        return getattr(self.engine, method)(*args, **kwargs)

    def alive(self) -> bool:
        return True

    def stop(self) -> None:
        self.engine.terminate()


@dataclass
class AsyncResult:
    req_id: int
    event: threading.Event
    slo: Optional[SloStat] = None
    tokens: Optional[List[int]] = None

    def get(self, timeout: Optional[float] = None) -> SloStat:
        if not self.event.wait(timeout):
            raise TimeoutError(f"request {self.req_id} did not finish")
        return self.slo


class Controller:
    def __init__(self, n_node: int, n_gpu_per_node: int, device: str = "cuda", in_process: bool = False,
                 heartbeat_timeout_s: float = 30.0, dp_policy: str = "max",
                 worker_addresses: Optional[Dict[int, Tuple[str, int]]] = None):
        self.n_node, self.n_gpu_per_node = n_node, n_gpu_per_node
        self.device_kind = device
        self.in_process = in_process
        self.workers: Dict[int, object] = {}
        self.tokenizer: Optional[TokenizerEngine] = None
        self.sampler: Optional[SamplerEngine] = None
        self.placement: Optional[ModelPlacement] = None
        self.model_config: Optional[ModelConfig] = None
        self.req_counter = 0
        self.results: Dict[int, AsyncResult] = {}
        self.dp_scheduler = None
        self.dp_policy = dp_policy          # "max": replica with the most free KV blocks (waits for room); "RR"
        # device id -> (host, port) of the node agent that hosts that device's worker (multi-node deployments);
        # devices not listed get a worker process on this machine
        self.worker_addresses = dict(worker_addresses or {})
        self.controller_host = "127.0.0.1"   # the address workers on other nodes use to reach tokenizer / sampler
        self.port_shift = random.randint(0, 400) * 16 * 4 % 6000
        self.heartbeat_timeout_s = heartbeat_timeout_s
        self.suspect_workers: List[int] = []
        self._poll_thread: Optional[threading.Thread] = None
        self._end = False
        self._logger = get_logger("controller")
        self._free_blocks: Dict[int, int] = {}
        self._req_rank: Dict[int, int] = {}
        self._lock = threading.Lock()
        self._init_args = None                       # arguments of init_engine, kept for recover()
        self._req_info: Dict[int, Tuple[List[int], int]] = {}   # request -> (original prompt, output length)
        self._prefix: Dict[int, List[int]] = {}      # tokens a request had produced before a recovery
        self._pending_args: Dict[int, InitCoreArgs] = {}
        self._progress: Dict[int, Tuple[int, float]] = {}   # request -> (tokens seen, time of the last new token)

    # ---- workers --------------------------------------------------------------------------------------------
    def _device_of(self, device_id: int) -> str:
        if self.device_kind == "cpu":
            return "cpu"
        # a worker process sees exactly one GPU (CUDA_VISIBLE_DEVICES), so every native helper thread is on the right
        # device without a cudaSetDevice of its own -- the arrangement the reference gets from Ray
        return f"cuda:{device_id % self.n_gpu_per_node}" if self.in_process else "cuda:0"

    def _create_engines(self, placement: ModelPlacement) -> None:
        for d in placement.device_ids():
            if self.in_process:
                self.workers[d] = LocalWorker(d, self._device_of(d))
            elif d in self.worker_addresses:
                from .node_agent import RemoteWorkerHandle
                env = {"CUDA_VISIBLE_DEVICES": str(d % self.n_gpu_per_node)} if self.device_kind == "cuda" else {}
                self.workers[d] = RemoteWorkerHandle(d, self._device_of(d), self.worker_addresses[d], env)
            else:
                env = {}
                if self.device_kind == "cuda":
                    env["CUDA_VISIBLE_DEVICES"] = str(d % self.n_gpu_per_node)
                self.workers[d] = WorkerHandle(d, self._device_of(d), env)

    def _all(self, method: str, *args, **kwargs) -> Dict[int, object]:
        for w in self.workers.values():
            w.call_async(method, *args, **kwargs)
        return {d: w.wait() for d, w in self.workers.items()}

    def _get_nccl_ids(self, placement: ModelPlacement) -> Dict[Tuple[int, int], bytes]:
        ids = {}
        if self.device_kind != "cuda":
            return ids
        for src, outs in placement.out_device_ids.items():
            for dst in outs:
                if C.is_embedding_node(src) or C.is_embedding_node(dst) or src == dst:
                    continue
                ids[(src, dst)] = C.get_nccl_unique_id()
        return ids

    # ---- init -----------------------------------------------------------------------------------------------
    def init_engine(self, placement: ModelPlacement, model_config: ModelConfig, cache_config: Optional[CacheConfig] = None,
                    sampling_config: Optional[SamplingConfig] = None, state_dict_path: Optional[str] = None,
                    keep_logits: bool = False, dtype=None, ignore_eos: bool = True) -> None:
        self.placement, self.model_config = placement, model_config
        self._init_args = (placement, model_config, cache_config, sampling_config, state_dict_path, keep_logits, dtype,
                           ignore_eos)
        self._pending_args = {}
        cache_config = cache_config or CacheConfig()
        sampling_config = sampling_config or SamplingConfig(1, 2)
        L = model_config.num_layers
        C.set_port_base(self.port_shift)
        C.set_inproc_transport(self.in_process)
        self._create_engines(placement)
        nccl = self._get_nccl_ids(placement)
        # who runs attention layer l for dp rank r (layer L = the LM-head step, hosted where layer 0 runs)
        attn_peer: Dict[int, Dict[int, int]] = {}
        for l in range(L):
            for d in placement.attn_devices_of_layer(l):
                if placement.is_worker_device(d):
                    continue
                attn_peer.setdefault(l, {})[placement.attn_dp_rank_at(d)] = d
        attn_peer[L] = dict(attn_peer[0])
        expert_ranks = [(l, e, r) for (l, e), r in placement.expert_ranks.items()]
        # every worker learns where every other one lives; tokenizer and sampler live with the controller
        hosts = {d: self.worker_addresses.get(d, (self.controller_host, 0))[0]
                 for d in list(self.workers) + [TOKENIZER_DEV_ID, SAMPLER_DEV_ID]}
        C.set_hosts(os.getpid(), hosts)
        self._all("setup_engine", model_config, cache_config, dtype, self.in_process)
        # attention TP: only the driver of a group is part of the token flow; it broadcasts its batches to the workers
        tp_workers = {d for d in self.workers if placement.is_worker_device(d)}
        assert not (tp_workers and self.in_process), "attention TP needs one process per device"
        for d, w in self.workers.items():
            group = (placement.device_groups or {}).get(d, [d]) if placement.has_attn(d) else [d]
            tp = dict(tp_rank=group.index(d), tp_size=len(group),
                      tp_master_port=20000 + (self.port_shift + 97 * group[0]) % 20000)
            if d in tp_workers:
                self._pending_args[d] = InitCoreArgs(
                    layer_ids=placement.layer_ids_at(d), in_device_ids=[], out_device_ids=[], out_channel_infos=[],
                    attn_peer=attn_peer, expert_ranks=expert_ranks, hosts=hosts, port_shift=self.port_shift,
                    state_dict_path=state_dict_path, **tp)
                continue
            outs = [o for o in placement.out_device_ids.get(d, []) if o not in tp_workers]
            ins = [i for i in placement.in_device_ids.get(d, []) if i not in tp_workers]
            if placement.has_attn(d):
                # the residual stream goes to the attention worker of the next layer; the head step reports to the sampler
                dp = placement.attn_dp_rank_at(d)
                for l in placement.attn_layer_ids_at(d):
                    nxt = attn_peer[l + 1].get(dp, next(iter(attn_peer[l + 1].values())))
                    if nxt not in outs:
                        outs.append(nxt)
                if attn_peer[L].get(dp) == d and SAMPLER_DEV_ID not in outs:
                    outs.append(SAMPLER_DEV_ID)
            if placement.has_expert(d):
                # experts of the last layer return to the LM-head step instead of the sampler
                outs = [o for o in outs if o != SAMPLER_DEV_ID or placement.has_attn(d)]
                for r, dev in attn_peer[L].items():
                    if any(l == L - 1 for l, _ in placement.expert_ids_at(d)) and dev not in outs:
                        outs.append(dev)
            infos = []
            for o in outs:
                infos.append((list(placement.expert.get(o, [])), list(placement.attn.get(o, [])),
                              placement.attn_dp_rank_at(o) if o in placement.attn else 0))
            # every device that may send to d
            senders = set(ins)
            for s in self.workers:
                if s == d:
                    continue
            args = InitCoreArgs(
                layer_ids=placement.layer_ids_at(d), in_device_ids=[], out_device_ids=outs, out_channel_infos=infos,
                in_nccl_ids={}, out_nccl_ids={o: nccl[(d, o)] for o in outs if (d, o) in nccl},
                attn_peer=attn_peer, expert_ranks=expert_ranks,
                local_attn_dp_rank=placement.attn_dp_rank_at(d) if d in placement.attn else 0,
                expert_ids=list(placement.expert_ids_at(d)), hosts=hosts, port_shift=self.port_shift,
                state_dict_path=state_dict_path, keep_logits=keep_logits, **tp)
            self._pending_args[d] = args
        # in-edges are the transpose of the (extended) out-edges
        for d, a in self._pending_args.items():
            for o in a.out_device_ids:
                if o in self._pending_args and d not in self._pending_args[o].in_device_ids:
                    self._pending_args[o].in_device_ids.append(d)
                    if (d, o) in nccl:
                        self._pending_args[o].in_nccl_ids[d] = nccl[(d, o)]
        # mailboxes are bound in init_core, NCCL communicators need both ends at once: run it on all workers together
        for d, w in self.workers.items():
            w.call_async("init_core", self._pending_args[d], placement)
        for w in self.workers.values():
            w.wait()
        layer0 = attn_peer[0]
        self.tokenizer = TokenizerEngine(TOKENIZER_DEV_ID, list(layer0.values()), layer0)
        self.sampler = SamplerEngine(SAMPLER_DEV_ID, list(layer0.values()), layer0, sampling_config.min_output_len,
                                     sampling_config.max_output_len, model_config.top_k, ignore_eos)
        self.sampling_config = sampling_config
        self.cache_config = cache_config
        self.dp_size = len(layer0)
        self.dp_scheduler = get_dp_scheduler(self.dp_size, model_config.max_seq_len, cache_config.block_size,
                                             self.dp_policy)
        self._free_blocks = {r: self.workers[dev].call("num_free_blocks") for r, dev in layer0.items()}
        self.attn_peer = attn_peer

    def start_engine(self) -> None:
        self._all("start")
        self.tokenizer.start()
        self.sampler.start()
        self._end = False
        self._poll_thread = threading.Thread(target=self._poll_loop, daemon=True, name="controller-poll")
        self._poll_thread.start()

    # ---- requests -------------------------------------------------------------------------------------------
    def get_new_req_id(self) -> int:
        self.req_counter += 1
        return self.req_counter

    def _pick_dp_rank(self, need_blocks: int) -> int:
        if self.dp_policy == "RR":
            with self._lock:
                r = self.dp_scheduler._schedule()
                self._free_blocks[r] -= need_blocks
                return r
        # admission by free KV blocks (the "max" policy of the DP scheduler, with the request's own block need
        # instead of a fixed worst case); waits while no replica has room
        while True:
            with self._lock:
                r = max(self._free_blocks, key=lambda k: (self._free_blocks[k], -k))
                if self._free_blocks[r] >= need_blocks:
                    self._free_blocks[r] -= need_blocks
                    return r
            time.sleep(0.005)

    def put_single_request(self, prompt, output_len: Optional[int] = None, req_id: Optional[int] = None) -> AsyncResult:
        """``prompt`` is a list of token ids or an int (a prompt of that many pseudo-random ids)."""
        cfg = self.model_config
        if isinstance(prompt, int):
            rnd = random.Random(self.req_counter + 1)
            prompt = [rnd.randrange(3, cfg.vocab_size) for _ in range(prompt)]
        rid = req_id if req_id is not None else self.get_new_req_id()
        max_out = output_len if output_len is not None else self.sampling_config.max_output_len
        if len(prompt) + max_out > cfg.max_seq_len:
            raise ValueError(f"{len(prompt)} prompt + {max_out} new tokens exceed max_seq_len {cfg.max_seq_len}")
        res = AsyncResult(rid, threading.Event())
        with self._lock:
            self.results[rid] = res
            self._req_info[rid] = (list(prompt), max_out)
        self._submit(rid, list(prompt), max_out, explicit_len=output_len is not None)
        return res

    def _submit(self, rid: int, prompt: List[int], max_out: int, explicit_len: bool = True) -> None:
        need = (len(prompt) + max_out + self.cache_config.block_size - 1) // self.cache_config.block_size
        rank = self._pick_dp_rank(need)
        with self._lock:
            self._req_rank[rid] = (rank, need)
        if explicit_len:
            self.sampler.set_request_output_len(rid, max_out)
        self.tokenizer.put_single_request(rid, prompt, rank)

    def put_requests(self, prompts: List, output_lens: Optional[List[int]] = None) -> List[AsyncResult]:
        return [self.put_single_request(p, None if output_lens is None else output_lens[i])
                for i, p in enumerate(prompts)]

    def _poll_loop(self) -> None:
        last_beat = time.time()
        while not self._end:
            try:
                self.process_finished_results(self.sampler.fetch_finished_results())
            except Exception:
                self._logger.error(traceback.format_exc())
            if time.time() - last_beat > max(1.0, self.heartbeat_timeout_s / 3):
                last_beat = time.time()
                self.check_workers()
            self._note_progress()
            time.sleep(0.002)

    def _note_progress(self, period_s: float = 0.05) -> None:
        now = time.time()
        if now - getattr(self, "_last_progress_scan", 0.0) < period_s:
            return
        self._last_progress_scan = now
        with self._lock:
            pending = [rid for rid, r in self.results.items() if not r.event.is_set()]
        for rid in pending:
            n = len(self.sampler.get_output_tokens(rid))
            seen = self._progress.get(rid)
            if seen is None or seen[0] != n:
                self._progress[rid] = (n, now)

    def stalled_requests(self, deadline_s: float) -> List[int]:
        """Unfinished requests that have produced no token for ``deadline_s`` seconds (a lost message leaves the
        tokens of a request waiting for a part that never comes; nothing else in the system would notice)."""
        now = time.time()
        with self._lock:
            pending = [rid for rid, r in self.results.items() if not r.event.is_set()]
        return [rid for rid in pending if rid in self._progress and now - self._progress[rid][1] > deadline_s]

    def process_finished_results(self, stats) -> None:
        if not stats:
            return
        done = [s.req_id for s in stats]
        self.release_kv_cache(done)
        for s in stats:
            with self._lock:
                res = self.results.get(s.req_id)
                rank_need = self._req_rank.pop(s.req_id, None)
                if rank_need is not None:
                    self._free_blocks[rank_need[0]] += rank_need[1]
            if res is not None:
                res.slo = SloStat.from_c(s)
                res.tokens = self._prefix.get(s.req_id, []) + list(self.sampler.get_output_tokens(s.req_id))
                res.event.set()

    # ---- names of the reference controller (controller.py:131-136, 323-358, 388-390) ------------------------------
    @property
    def all_workers(self) -> List[object]:
        return list(self.workers.values()) + [self.sampler, self.tokenizer]

    @property
    def all_device_ids(self) -> List[int]:
        from ..utils.constants import SAMPLER_DEV_ID, TOKENIZER_DEV_ID
        return list(self.workers) + [SAMPLER_DEV_ID, TOKENIZER_DEV_ID]

    def determine_worker_type(self, device_id: int) -> str:
        from ..utils.constants import SAMPLER_DEV_ID, TOKENIZER_DEV_ID
        if device_id == SAMPLER_DEV_ID:
            return "sampler"
        if device_id == TOKENIZER_DEV_ID:
            return "tokenizer"
        if self.placement.is_hybrid:
            return "hybrid"
        return "attention" if self.placement.has_attn(device_id) else "expert"

    def fetch_queueing_delays(self) -> Tuple[List[List[float]], List[List[float]]]:
        """Per-step queueing delays (ms) of every attention worker and of every expert worker."""
        attn, exp = [], []
        for d, res in self._all("fetch_queueing_delays").items():
            if self.placement.is_worker_device(d):
                continue                      # a TP worker has no queue: it runs what its driver broadcasts
            (attn if self.placement.has_attn(d) else exp).append(res)
        return attn, exp

    def fetch_submitted_time(self) -> Dict[int, float]:
        return self.tokenizer.fetch_submitted_time()

    def reset_workers(self) -> None:
        self._all("reset")

    def start_polling_results(self) -> None:
        if self._poll_thread is None or not self._poll_thread.is_alive():
            self._end = False
            self._poll_thread = threading.Thread(target=self._poll_loop, daemon=True, name="controller-poll")
            self._poll_thread.start()

    def release_kv_cache(self, req_ids: List[int]) -> None:
        for d, w in self.workers.items():
            if self.placement.has_attn(d) and d not in self.suspect_workers and w.alive():
                w.call("release_seqs", req_ids)

    def wait_for_requests(self, n_request: int, timeout: float = 600.0) -> Dict[int, SloStat]:
        t0 = time.time()
        while time.time() - t0 < timeout:
            with self._lock:
                done = {r: a.slo for r, a in self.results.items() if a.event.is_set()}
            if len(done) >= n_request:
                return done
            err = self.first_worker_error()
            if err:
                raise RuntimeError(err)
            time.sleep(0.01)
        raise TimeoutError(f"{n_request} requests did not finish within {timeout} s")

    # ---- failure detection ----------------------------------------------------------------------------------
    def check_workers(self) -> List[int]:
        """Marks workers whose process died (or whose RPC no longer answers) as suspect; returns their ids."""
        bad = []
        for d, w in self.workers.items():
            if not w.alive():
                bad.append(d)
        for d in bad:
            if d not in self.suspect_workers:
                self.suspect_workers.append(d)
                self._logger.error(f"worker {d} is not alive")
        return bad

    def first_worker_error(self) -> Optional[str]:
        for d, w in self.workers.items():
            if d in self.suspect_workers:
                return f"worker {d} died"
            if isinstance(w, LocalWorker):
                e = w.engine.check_error()
                if e:
                    return e
        # worker processes are asked over RPC, at most once a second
        now = time.time()
        if now - getattr(self, "_last_remote_check", 0.0) >= 1.0:
            self._last_remote_check = now
            for d, w in self.workers.items():
                if not isinstance(w, LocalWorker) and d not in self.suspect_workers:
                    try:
                        e = w.call("check_error")
                    except Exception as ex:     # the RPC itself failed: the worker is gone
                        return f"worker {d}: {ex}"
                    if e:
                        return f"worker {d}: {e}"
        return None

    def recover(self) -> List[int]:
        """Recovery after a worker failure by full restart and re-admission: every worker is torn down and rebuilt
        with the placement / configuration of the last ``init_engine`` (fresh ports, fresh channels), and every
        request that had not finished is submitted again as prompt + the tokens the sampler had already recorded for it
        (its KV is rebuilt by a prefill of that longer prompt), for the remaining number of tokens. The
        ``AsyncResult`` objects handed out before stay valid and receive the complete token list. Returns the ids of
        the re-admitted requests. The reference has no recovery path (errors are fatal there)."""
        assert self._init_args is not None, "init_engine has not run"
        with self._lock:
            unfinished = [rid for rid, r in self.results.items() if not r.event.is_set()]
        for rid in unfinished:
            self._prefix[rid] = self._prefix.get(rid, []) + list(self.sampler.get_output_tokens(rid))
        self.stop_workers()
        self.workers.clear()
        self.suspect_workers.clear()
        self._progress.clear()
        with self._lock:
            self._req_rank.clear()
        self.port_shift = (self.port_shift + 16 * 4 * 11) % 6000        # the old sockets may linger in TIME_WAIT
        self.init_engine(*self._init_args)
        self.start_engine()
        again = []
        for rid in unfinished:
            prompt, max_out = self._req_info[rid]
            done = self._prefix[rid]
            remaining = max_out - len(done)
            res = self.results[rid]
            if remaining <= 0:
                res.tokens = list(done)
                res.event.set()
                continue
            self._submit(rid, prompt + done, remaining)
            again.append(rid)
        self._logger.info(f"recovered: {len(again)} request(s) re-admitted")
        return again

    # ---- stats / control ------------------------------------------------------------------------------------
    def fetch_step_stats(self):
        return self._all("fetch_step_stats")

    def fetch_logits(self) -> Dict[Tuple[int, int], object]:
        out = {}
        for d, w in self.workers.items():
            if self.placement.has_attn(d):
                out.update(w.call("fetch_logits"))
        return out

    def fetch_sampler_step_infos(self):
        return self.sampler.fetch_sampler_step_infos()

    def worker_errors(self) -> Dict[int, Optional[str]]:
        return self._all("check_error")

    def graph_attention_steps(self) -> Dict[int, int]:
        """Per worker: attention steps that replayed a CUDA graph (0 unless ``enable_cuda_graph_attn`` is set)."""
        return self._all("graph_attention_steps")

    def set_schedule_policy(self, policy: str) -> None:
        self._all("set_schedule_policy", policy)

    def set_schedule_block(self, step: int) -> None:
        self._all("set_schedule_block", step)

    def start_profile(self, profile_dir: Optional[str] = None) -> None:
        self._all("start_profile", profile_dir)

    def stop_profile(self) -> None:
        self._all("stop_profile")

    def reset(self) -> None:
        self._all("reset")
        self.sampler.reset()
        with self._lock:
            self.results.clear()

    def stop_workers(self) -> None:
        self._end = True
        if self._poll_thread is not None:
            self._poll_thread.join(timeout=5)
        if self.tokenizer is not None:
            self.tokenizer.terminate()
        if self.sampler is not None:
            self.sampler.terminate()
        for w in self.workers.values():
            try:
                if w.alive():
                    w.call("terminate", timeout=20)
            except Exception:
                pass
            w.stop()


def init_controller(n_node: int, n_gpu_per_node: int, device: str = "cuda", in_process: bool = False,
                    **kwargs) -> Controller:
    return Controller(n_node, n_gpu_per_node, device=device, in_process=in_process, **kwargs)
