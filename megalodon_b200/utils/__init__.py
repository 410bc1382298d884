"""General helpers with the names and behaviour of the reference's
megalodon/utils.py:26-211, made device-agnostic (CPU + gloo works)."""
from __future__ import annotations

import contextlib
import logging
import math
import os
import random
import socket
from functools import partial
from typing import Callable, List, Optional, Tuple, Union

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn

Scalar = Union[int, float]
logger = logging.getLogger()


def parse_bool_flag(arg) -> bool:
    if isinstance(arg, bool):
        return arg
    low = str(arg).lower()
    if low == "true":
        return True
    if low == "false":
        return False
    raise ValueError("Invalid value for a boolean flag!")


def get_parallel_ranks(global_rank: int, model_parallel_size: Optional[int] = None,
                       chunk_parallel_size: Optional[int] = None) -> Tuple[int, int, int]:
    """global rank -> (data, chunk, model) parallel ranks for the layout
    rank = (dp * CP + cp) * MP + mp."""
    from ..parallel.initialize import get_chunk_parallel_world_size, get_model_parallel_world_size
    if model_parallel_size is None and chunk_parallel_size is None:
        model_parallel_size = get_model_parallel_world_size()
        chunk_parallel_size = get_chunk_parallel_world_size()
    mp = model_parallel_size or 1
    cp = chunk_parallel_size or 1
    return global_rank // (mp * cp), (global_rank // mp) % cp, global_rank % mp


def get_torch_dtype(dtype: str) -> torch.dtype:
    return {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[dtype]


def get_default_half() -> str:
    return "bf16"


def get_init_fn(mode: str, dim: Optional[int] = None) -> Callable[[torch.Tensor], torch.Tensor]:
    if mode == "none":
        return lambda x: x
    if mode == "bert":
        return partial(nn.init.normal_, mean=0.0, std=0.02)
    if mode == "he":
        return partial(nn.init.kaiming_normal_, a=math.sqrt(5.0))
    if mode == "gaussian":
        std = 1.0 if dim is None else 1.0 / math.sqrt(dim)
        return partial(nn.init.trunc_normal_, mean=0.0, std=std, a=-3 * std, b=3 * std)
    if mode == "xavier":
        return nn.init.xavier_uniform_
    raise ValueError(f"Unknown init mode: {mode}")


def set_random_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)


def default_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


@contextlib.contextmanager
def create_on_gpu():
    """Allocate new tensors on the accelerator (on the CPU when there is none)."""
    with torch.device(default_device()):
        yield


@torch.no_grad()
def check_same_in_process_group(x: torch.Tensor, name: str, group_name: str,
                                group: Optional[dist.ProcessGroup] = None) -> None:
    assert isinstance(x, torch.Tensor) and x.dtype in (torch.int64, torch.int32, torch.bool)
    if not (dist.is_available() and dist.is_initialized()):
        return
    from ..parallel.utils import comm_device
    ref = x.to(comm_device(group)).to(torch.int64)
    top = ref.clone()
    dist.all_reduce(top, op=dist.ReduceOp.MAX, group=group)
    if not torch.equal(top, ref):
        raise RuntimeError(
            f"ISSUE: different tensor {name} detected in the same {group_name} parallel group !!! - ")


@torch.no_grad()
def clip_grad_norm_(fsdp_module, max_norm: Union[float, int], norm_type: Union[float, int] = 2.0):
    """Global-norm clipping across the data- and model-parallel groups."""
    return fsdp_module.clip_grad_norm_(max_norm, norm_type)


def pad(tokens: List[int], max_length: int, value: int, padding: str = "post",
        truncating: str = "post") -> List[int]:
    short = max_length - len(tokens)
    if short > 0:
        fill = [value] * short
        tokens = tokens + fill if padding == "post" else (fill + tokens if padding == "pre" else tokens)
    if truncating == "post":
        tokens = tokens[:max_length]
    elif truncating == "pre" and len(tokens) > max_length:
        tokens = tokens[len(tokens) - max_length:]
    return tokens


def setup_env() -> None:
    env = {
        "NCCL_DEBUG": "INFO",
        "OMP_NUM_THREADS": "1",
        "MKL_NUM_THREADS": "1",
        "TORCH_NCCL_ASYNC_ERROR_HANDLING": "1",
        "NCCL_IB_TIMEOUT": "22",
    }
    if "LOCAL_RANK" in os.environ:      # launched by torchrun
        env.pop("NCCL_DEBUG")
    for name, value in env.items():
        if os.environ.get(name) != value:
            os.environ[name] = value
            logger.warning(f"WARNING: Setting {name} to {value}")


def log_host() -> None:
    logger.warning(f"Host: {socket.gethostname()}")
    logger.warning(f"Job hosts: {os.environ.get('SLURM_JOB_NODELIST', '')}")
    logger.warning(f"Slurm job id: {int(os.environ.get('SLURM_JOB_ID', -1))}")


def init_cache(bsz: int, model, compute_dtype: torch.dtype, truncate: bool = False, device=None):
    """Empty inference cache: per layer ((k, v, count) | None, (count, mean, var), hx)
    and (count, mean, var) for the output norm.  `truncate=True` builds the
    cache used to re-derive normalisation statistics only (no KV, no CEMA state)."""
    if device is None:
        device = next(model.parameters()).device
    layers = []
    for _ in range(model.num_layers):
        kv = None if truncate else (
            torch.empty((bsz, 0, model.local_heads, model.z_head_dim), dtype=compute_dtype, device=device),
            torch.empty((bsz, 0, model.local_heads, getattr(model, "local_v_head_dim", model.v_head_dim)),
                        dtype=compute_dtype, device=device),
            0,
        )
        layers.append((kv, (None, None, None), None))
    return layers, (None, None, None)


def reshard_cache(cache, mp_rank: int, mp_size: int):
    """Slice a cache produced without tensor parallelism (e.g. by a chunk-parallel prefill) down to
    what model-parallel rank `mp_rank` of `mp_size` holds: its heads of the key/value tail, its
    TimestepNorm groups, its features of the CEMA state.  Counts are shared."""
    if mp_size == 1:
        return cache

    def part(t, dim):
        n = t.size(dim) // mp_size
        return t.narrow(dim, mp_rank * n, n).contiguous()

    def kv_part(k, v):
        """k [B, len, H, dk], v [B, len, H, dv].  Up to one rank per head the heads are split; beyond
        that each head's value columns are split over mp_size / H ranks and its keys are replicated."""
        heads = k.size(2)
        if mp_size <= heads:
            return part(k, 2), part(v, 2)
        split = mp_size // heads
        h, s = mp_rank // split, mp_rank % split
        dv = v.size(3) // split
        return k.narrow(2, h, 1).contiguous(), v.narrow(2, h, 1).narrow(3, s * dv, dv).contiguous()

    layers, out_norm = cache
    new_layers = []
    for kv, (count, mean, var), hx in layers:
        if kv is not None:
            kv = kv_part(kv[0], kv[1]) + (kv[2],)
        new_layers.append((kv, (count, part(mean, 1), part(var, 1)), None if hx is None else part(hx, 1)))
    count, mean, var = out_norm
    return new_layers, (count, part(mean, 1), part(var, 1))


def expand_cache(cache, batch: int):
    """Repeat a batch-1 cache `batch` times (the same prompt decoded in `batch` streams)."""
    def rep(t):
        return t if t is None or not torch.is_tensor(t) or t.size(0) == batch else \
            t.expand(batch, *t.shape[1:]).contiguous()

    layers, out_norm = cache
    new_layers = []
    for kv, norm, hx in layers:
        kv = None if kv is None else (rep(kv[0]), rep(kv[1]), kv[2])
        new_layers.append((kv, tuple(rep(t) for t in norm), rep(hx)))
    return new_layers, tuple(rep(t) for t in out_norm)


def truncate_cache(cache, truncated_cache):
    """Keep KV and CEMA state of `cache` but take the normalisation statistics
    from `truncated_cache` (statistics re-derived over a recent window)."""
    layers, _ = cache
    t_layers, t_out = truncated_cache
    for i, (kv, _, hx) in enumerate(layers):
        layers[i] = (kv, t_layers[i][1], hx)
    return layers, t_out
