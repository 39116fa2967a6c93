"""HTTP front end for interactive experiments (reference: benchmark/server.py:21-91, Flask there, FastAPI here).

    python -m benchmark.server --device cpu --model tiny -g 2 --ep-size 1 --step-attn 1 --port 6699

POST /run_once     {"rate": 10, "time": 10, "distribution": "poisson"}  runs one open-loop workload, returns its metrics
POST /generate     {"prompt_ids": [...], "max_new_tokens": 16}          one request; returns the generated token ids
POST /set_schedule {"policy": "mbflfs", "step": 8}                     switches the layer-scheduling policy / block size
                                                                       of every worker at run time
GET  /health       worker liveness
"""
from __future__ import annotations

import copy
import os
import sys
from dataclasses import asdict

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmark.benchmark_serving import analyze_results, launch, make_workload, run_benchmark_controller
from benchmark.utils import get_parser_base

POLICIES = ("mbfs", "flfs", "mbflfs", "mbtfs", "bin")


def create_app(args):
    from contextlib import asynccontextmanager
    from fastapi import FastAPI, HTTPException
    state = {"master": None, "cfg": None, "args": args}

    @asynccontextmanager
    async def lifespan(_app):
        state["master"], state["cfg"] = launch(args)      # workers come up with the server ...
        yield
        if state["master"] is not None:                   # ... and go down with it
            state["master"].stop_workers()

    app = FastAPI(title="disagmoe_b200 benchmark server", lifespan=lifespan)

    @app.post("/run_once")
    def run_once(body: dict):
        try:
            rate, secs = float(body.get("rate", 10)), float(body.get("time", 10))
            dist_name = str(body.get("distribution", "poisson"))
        except (TypeError, ValueError):
            raise HTTPException(400, "rate and time must be numbers")
        a = copy.copy(state["args"])
        a.rate, a.num_requests, a.generator_type, a.duration = rate, int(rate * secs), dist_name, 0
        wl = make_workload(a)
        stats, arrivals, dur = run_benchmark_controller(state["master"], state["cfg"], wl, a)
        return asdict(analyze_results(stats, arrivals, dur))

    @app.post("/set_schedule")
    def set_schedule(body: dict):
        policy, step = body.get("policy"), body.get("step")
        if policy is None and step is None:
            raise HTTPException(400, "missing parameter: policy or step")
        if policy is not None:
            if policy not in POLICIES:
                raise HTTPException(400, f"invalid policy {policy!r}; one of {POLICIES}")
            state["master"].set_schedule_policy(policy)
            state["args"].layer_scheduler_type = policy
        if step is not None:
            state["master"].set_schedule_block(int(step))
            state["args"].layer_scheduler_step = int(step)
        return {"ok": True}

    @app.post("/generate")
    def generate(body: dict):
        """One request through the serving system: {"prompt_ids": [...], "max_new_tokens": n} -> generated token ids
        and the request's timestamps (seconds)."""
        prompt, n_new = body.get("prompt_ids"), body.get("max_new_tokens", 16)
        if not isinstance(prompt, list) or not prompt or not all(isinstance(t, int) for t in prompt):
            raise HTTPException(400, "prompt_ids must be a non-empty list of token ids")
        cfg = state["cfg"]
        if not all(0 <= t < cfg.vocab_size for t in prompt) or not isinstance(n_new, int) or n_new < 1:
            raise HTTPException(400, "token ids must be inside the vocabulary and max_new_tokens >= 1")
        try:
            res = state["master"].put_single_request(prompt, output_len=n_new)
            slo = res.get(timeout=600)
        except ValueError as e:
            raise HTTPException(400, str(e))
        return {"req_id": res.req_id, "tokens": res.tokens, "t_tokens": slo.t_tokens}

    @app.get("/health")
    def health():
        m = state["master"]
        return {"suspect_workers": m.check_workers() if m else [], "workers": len(m.workers) if m else 0}

    return app


def main():
    p = get_parser_base()
    p.add_argument("--port", type=int, default=6699)
    args = p.parse_args()
    import uvicorn
    uvicorn.run(create_app(args), host="127.0.0.1", port=args.port, log_level="warning")


if __name__ == "__main__":
    main()
