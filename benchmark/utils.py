"""Command-line flags of the serving benchmark (flag names of the reference's benchmark/utils.py:4-48)."""
from argparse import ArgumentParser

from disagmoe_b200.utils.constants import BLOCK_SIZE


def get_parser_base() -> ArgumentParser:
    p = ArgumentParser()
    # benchmark
    p.add_argument("-r", "--rate", type=float, default=0, help="request arrival rate (requests per second); 0 = all at once")
    p.add_argument("--min-input-len", type=int, default=100)
    p.add_argument("-i", "--max-input-len", type=int, default=300)
    p.add_argument("--min-output-len", type=int, default=100)
    p.add_argument("-o", "--max-output-len", type=int, default=500)
    p.add_argument("-n", "--num-requests", type=int, default=1000)
    p.add_argument("-p", "--profile-dir", type=str, default=None, help="directory for torch profiler output")
    p.add_argument("--serial-gemm", action="store_true", default=False, help="one dense GEMM per expert instead of the grouped GEMM")
    p.add_argument("--nsys", action="store_true", help="kept for command-line compatibility; nsys is not on this image")
    p.add_argument("-f", "--file", type=str, default="reports/benchmark.csv")
    p.add_argument("--trace", action="store_true", default=False, help="write a Chrome trace of the engine steps")
    p.add_argument("--enable-trace-detail", action="store_true", default=False)
    p.add_argument("--generator-type", type=str, default="poisson",
                   help="poisson | uniform | offline | incremental_poisson")
    p.add_argument("--analyze-throughput", action="store_true", default=False)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--duration", type=float, default=0, help="generate requests for this many seconds instead of -n")
    # model
    p.add_argument("--model", type=str, default="mixtral", help="preset: mixtral | qwen-moe | deepseek-v2-lite | tiny")
    p.add_argument("-ca", "--cuda-graph-attn", action="store_true", default=False)
    p.add_argument("-N", "--num-nodes", type=int, default=1)
    p.add_argument("-g", "--num-gpus", type=int, default=4)
    p.add_argument("-u", "--gpu-usage", type=float, default=0.65)
    p.add_argument("--tp-size", type=int, default=1)
    p.add_argument("--ep-size", type=int, default=2)
    p.add_argument("--dp-size", type=int, default=1)
    p.add_argument("-L", "--num-layers", type=int, default=32)
    p.add_argument("-E", "--num-experts", type=int, default=8)
    p.add_argument("-K", "--topk", type=int, default=1)
    p.add_argument("--num-blocks", type=int, default=None)
    p.add_argument("--block-size", type=int, default=BLOCK_SIZE)
    p.add_argument("--graph-stride", type=int, default=8)
    p.add_argument("--max-batch-size-attn", type=int, default=160)
    p.add_argument("--max-batch-size-expert", type=int, default=512)
    p.add_argument("--layer-scheduler-type", type=str, default="mbfs", help="mbfs | flfs | mbflfs | mbtfs | bin")
    p.add_argument("--layer-scheduler-step", type=int, default=1)
    # placement
    p.add_argument("--placement", type=str, default="pipeline", help="pipeline | colocate | interleave | single")
    p.add_argument("--zigzag-attn", action="store_true", default=False)
    p.add_argument("--step-attn", type=int, default=2)
    p.add_argument("--step-expert", type=int, default=1)
    # this implementation
    p.add_argument("--backend", type=str, default="controller",
                   help="controller (one process per device, host-scheduled) | colocated (one GPU, fused executor) | "
                        "fused (one process per GPU on the peer-memory path: tp-size x dp-size attention GPUs, the rest experts)")
    p.add_argument("--device", type=str, default="cuda", help="cuda | cpu")
    p.add_argument("--prefill-budget", type=int, default=0,
                   help="colocated backend: prompt rows per step next to the decode tokens (chunked prefill); "
                        "0 = alternate whole-prompt prefill steps and decode steps")
    p.add_argument("--worker-addresses", type=str, default="",
                   help="multi-node: 'device=host:port,...' of the node agents (python -m disagmoe_b200.frontend.node_agent) "
                        "that host those devices' workers; devices not listed run on this machine")
    return p
