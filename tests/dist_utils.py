"""Run a function on N CPU ranks (gloo) in child processes and collect results."""
import os
import socket
import tempfile
import traceback

import torch
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    import torch.distributed as dist
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        res = fn(rank, world, *args)
        torch.save(res, os.path.join(out_dir, f"{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        traceback.print_exc()
        raise


def run_ranks(fn, world, *args):
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_entry, args=(world, port, fn, args, d), nprocs=world, join=True)
        return [torch.load(os.path.join(d, f"{r}.pt"), weights_only=False) for r in range(world)]
