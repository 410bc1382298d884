"""Job bootstrap: rank discovery (torchrun / SLURM / single process), default
process group, and the SLURM pre-emption signal handlers (reference:
megalodon/distributed/setup.py:17-159).

Differences from the reference, on purpose: the backend is NCCL when a GPU is
present and gloo otherwise, so the whole framework also runs on CPU ranks; the
return value is a named tuple, which satisfies both the reference's annotated
`(is_slurm, global_rank, world_size)` unpacking and the README's attribute
access (`.global_rank`).
"""
from __future__ import annotations

import datetime
import logging
import os
import random
import signal
import socket
import subprocess
import sys
from functools import lru_cache
from typing import NamedTuple

import torch
import torch.distributed as dist

logger = logging.getLogger()


class DistInfo(NamedTuple):
    is_slurm: bool
    global_rank: int
    world_size: int


def _on_sigusr1(signum, frame):
    logger.warning(f"Signal handler called with signal {signum}")
    proc = int(os.environ.get("SLURM_PROCID", "0"))
    logger.warning(f"Host: {socket.gethostname()} - Global rank: {proc}")
    if proc == 0 and "SLURM_JOB_ID" in os.environ:
        logger.warning("Requeuing job " + os.environ["SLURM_JOB_ID"])
        subprocess.run(["scontrol", "requeue", os.environ["SLURM_JOB_ID"]], check=False)
        sys.exit(-1)
    logger.warning("Not the master process, no need to requeue.")


def _on_sigterm(signum, frame):
    logger.warning(f"Signal handler called with signal {signum}")
    logger.warning("Bypassing SIGTERM.")


def init_signal_handler() -> None:
    """SIGUSR1 (SLURM time limit / pre-emption) requeues from rank 0; SIGTERM is
    logged and ignored so a checkpoint in progress can finish."""
    signal.signal(signal.SIGUSR1, _on_sigusr1)
    signal.signal(signal.SIGTERM, _on_sigterm)
    logger.warning("Signal handler installed.")


def is_torch_run() -> bool:
    return os.environ.get("LOCAL_RANK") is not None


def is_slurm_job() -> bool:
    return "SLURM_JOB_ID" in os.environ and not is_torch_run()


def _from_env(torchrun_key: str, slurm_key: str, default: int) -> int:
    if is_torch_run():
        return int(os.environ[torchrun_key])
    if is_slurm_job():
        return int(os.environ[slurm_key])
    return default


def get_global_rank() -> int:
    return _from_env("RANK", "SLURM_PROCID", 0)


def get_local_rank() -> int:
    return _from_env("LOCAL_RANK", "SLURM_LOCALID", 0)


def get_world_size() -> int:
    return _from_env("WORLD_SIZE", "SLURM_NTASKS", 1)


def is_master() -> bool:
    return get_global_rank() == 0


def get_master_port(job_id: int) -> int:
    if "MASTER_PORT" in os.environ:
        return int(os.environ["MASTER_PORT"])
    return random.Random(job_id).randint(20000, 60000)


@lru_cache()
def get_master_addr() -> str:
    if "MASTER_ADDR" in os.environ:
        return os.environ["MASTER_ADDR"]
    if is_slurm_job():
        out = subprocess.check_output(["scontrol", "show", "hostnames", os.environ["SLURM_JOB_NODELIST"]])
        return out.split()[0].decode()
    return "127.0.0.1"


def default_backend() -> str:
    return "nccl" if torch.cuda.is_available() else "gloo"


_PG_TIMEOUT_S = [None]


def process_group_timeout():
    """Seconds given to `init_torch_distributed` (None before it ran): the timeout that
    `initialize_model_parallel` passes on to the groups it creates."""
    return _PG_TIMEOUT_S[0]


def init_distributed_process_group(timeout: int, backend: str | None = None) -> None:
    kwargs = {}
    _PG_TIMEOUT_S[0] = int(timeout)
    backend = backend or default_backend()
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(init_method="env://", backend=backend,
                            timeout=datetime.timedelta(seconds=int(timeout)), **kwargs)


def init_torch_distributed(timeout: int = 1800, backend: str | None = None) -> DistInfo:
    info = DistInfo(is_slurm_job(), get_global_rank(), get_world_size())
    local_rank = get_local_rank()
    os.environ["RANK"] = str(info.global_rank)
    os.environ["WORLD_SIZE"] = str(info.world_size)
    os.environ["MASTER_ADDR"] = get_master_addr()
    os.environ["MASTER_PORT"] = str(get_master_port(int(os.environ.get("SLURM_JOB_ID", -1))))
    how = "torchrun" if is_torch_run() else ("slurm" if info.is_slurm else "single process")
    logger.info(f"Run launched with {how}, local rank: {local_rank}")
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        init_distributed_process_group(timeout, backend)
    assert info.global_rank == dist.get_rank() and info.world_size == dist.get_world_size()
    return info
