"""torchrun worker: the attention GPUs of the job as ONE pipeline over the layers (layer striping) plus expert GPUs, on
real GPUs; the last stage compares its logits with the colocated executor. Prints one JSON line on rank 0.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 ... tests/workers/striping_worker.py [stages]"""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from disagmoe_b200.parallel.disagg import selfcheck_against_colocated


def main():
    rank, lr, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(lr)
    dist.init_process_group("nccl", device_id=torch.device("cuda", lr))
    stages = int(sys.argv[1]) if len(sys.argv) > 1 else 2
    res = selfcheck_against_colocated(world, rank, lr, stages, 1, n_mb=2, batch=8, stripes=stages)
    if rank == 0:
        print(json.dumps(dict(res, stages=stages, expert_gpus=world - stages)))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
