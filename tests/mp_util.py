"""Run a function as N gloo CPU ranks (child processes) and collect their return values."""
import os
import sys
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, fn, port, ret, args):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    torch.set_num_threads(1)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        torch.save(out, os.path.join(ret, f"r{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        traceback.print_exc()
        os._exit(1)


def run_ranks(fn, world, *args, port=None):
    import random
    port = port or random.randint(20000, 40000)
    with tempfile.TemporaryDirectory() as ret:
        mp.spawn(_worker, args=(world, fn, port, ret, args), nprocs=world, join=True)
        return [torch.load(os.path.join(ret, f"r{r}.pt"), weights_only=False) for r in range(world)]
