"""Environment variables forwarded to every worker process (reference: disagmoe/env.py:3-21)."""
import os

_defaults = {
    "DMOE_PROFILE_DIR": "",
    "CUDA_LAUNCH_BLOCKING": "0",
    "NCCL_DEBUG": "",
    "NCCL_LAUNCH_MODE": "",
    "NCCL_NVLS_ENABLE": "",
    "CUDA_DEVICE_MAX_CONNECTIONS": "",
    "MASTER_ADDR": "127.0.0.1",
    "MASTER_PORT": "26500",
    "TORCH_NCCL_BLOCKING_WAIT": "0",
    "LD_LIBRARY_PATH": "",
    "ENABLE_NVTX": "0",                 # enables the native range recorder
    "DMOE_WEIGHTED_ROUTER_FILE": "",    # per-layer expert popularity used for trace-weighted routing
    "DMOE_WEIGHTED_ROUTER_CATEGORY": "",  # which trace category of that file to use (default closed_qa)
}

ENV_VARS = {k: os.environ.get(k, v) for k, v in _defaults.items()}


def worker_env() -> dict:
    """Environment handed to a spawned worker: the whitelist above plus the current values."""
    env = dict(os.environ)
    for k, v in ENV_VARS.items():
        if v != "":
            env.setdefault(k, v)
    return env
