"""Process-group topology: data x chunk x model parallel.

Global ranks are laid out as `rank = (dp * CP + cp) * MP + mp`, i.e. model
parallel ranks are adjacent, then chunk-parallel ranks, then data-parallel
ranks (reference: megalodon/distributed/initialize.py:64-111).  The chunk
group is a line, not a ring: the first rank has no predecessor and the last
no successor.

On an NVSwitch box every peer is equally far, so adjacency does not matter for
bandwidth; the layout is kept because checkpoints and `get_parallel_ranks`
depend on it.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist

from .utils import ensure_divisibility

logger = logging.getLogger()


@dataclass
class _Topology:
    mp_group: Optional[dist.ProcessGroup] = None
    dp_group: Optional[dist.ProcessGroup] = None
    cp_group: Optional[dist.ProcessGroup] = None
    shard_group: Optional[dist.ProcessGroup] = None
    shard_ranks: List[int] = field(default_factory=list)
    mp_ranks: List[int] = field(default_factory=list)
    dp_ranks: List[int] = field(default_factory=list)
    cp_ranks: List[int] = field(default_factory=list)
    mp_rank: int = 0
    dp_rank: int = 0
    cp_rank: int = 0
    prev_chunk_rank: Optional[int] = None
    next_chunk_rank: Optional[int] = None
    ready: bool = False


_TOPO = _Topology()


def initialize_model_parallel(
    model_parallel_size: int,
    chunk_parallel_size: int = 1,
    *,
    model_parallel_backend: Optional[str] = None,
    chunk_parallel_backend: Optional[str] = None,
    ddp_backend: Optional[str] = None,
    timeout: Optional[float] = None,
) -> None:
    """`timeout` (seconds) applies to every group created here; by default the groups inherit the
    timeout `init_torch_distributed` was given (a group created without one gets the backend's own
    default - 10 minutes for NCCL - whatever the default group was told)."""
    global _TOPO
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed must be initialised first")
    if _TOPO.ready:
        raise RuntimeError("parallel groups are already initialised")
    world = dist.get_world_size()
    rank = dist.get_rank()
    mp, cp = int(model_parallel_size), int(chunk_parallel_size)
    ensure_divisibility(world, mp)
    ensure_divisibility(world, mp * cp)
    dp = world // (mp * cp)
    if rank == 0:
        logger.info(f"> initializing data  parallel with size {dp}")
        logger.info(f"> initializing chunk parallel with size {cp}")
        logger.info(f"> initializing model parallel with size {mp}")

    import datetime
    from .setup import process_group_timeout
    seconds = timeout if timeout is not None else process_group_timeout()
    tkw = {} if seconds is None else {"timeout": datetime.timedelta(seconds=float(seconds))}

    grid = torch.arange(world).reshape(dp, cp, mp)
    my_dp, my_cp, my_mp = (int(v[0]) for v in torch.where(grid == rank))
    topo = _Topology(mp_rank=my_mp, dp_rank=my_dp, cp_rank=my_cp)

    # Every rank must take part in every new_group call, in the same order.
    for j in range(cp):
        for k in range(mp):
            ranks = grid[:, j, k].tolist()
            g = dist.new_group(ranks, backend=ddp_backend, **tkw)
            if (j, k) == (my_cp, my_mp):
                topo.dp_group, topo.dp_ranks = g, ranks
    for i in range(dp):
        for j in range(cp):
            ranks = grid[i, j, :].tolist()
            g = dist.new_group(ranks, backend=model_parallel_backend, **tkw)
            if (i, j) == (my_dp, my_cp):
                topo.mp_group, topo.mp_ranks = g, ranks
    for i in range(dp):
        for k in range(mp):
            ranks = grid[i, :, k].tolist()
            g = dist.new_group(ranks, backend=chunk_parallel_backend, **tkw)
            if (i, k) == (my_dp, my_mp):
                topo.cp_group, topo.cp_ranks = g, ranks
                topo.prev_chunk_rank = ranks[my_cp - 1] if my_cp > 0 else None
                topo.next_chunk_rank = ranks[my_cp + 1] if my_cp + 1 < cp else None
    # data x chunk ranks sharing one model-parallel rank: the group an FSDP that
    # also shards over the chunk group uses (not present in the reference)
    if cp > 1 and dp > 1:
        for k in range(mp):
            ranks = grid[:, :, k].reshape(-1).tolist()
            g = dist.new_group(ranks, backend=ddp_backend, **tkw)
            if k == my_mp:
                topo.shard_group, topo.shard_ranks = g, ranks
    elif cp > 1:
        # The same ranks as the chunk group, but a communicator of its own.  The chunk group carries the
        # rank-to-rank hand-off of the CEMA / TimestepNorm state, which the ranks of a line issue at
        # different points of their programs (one sends where its neighbour receives); parameter gathers
        # and gradient reduce-scatters issued into the SAME communicator are ordered against those
        # transfers in issue order, and two neighbours that interleave them differently wait for each
        # other for ever (rank r: reduce-scatter, then send; rank r-1: receive, then reduce-scatter).
        for i in range(dp):
            for k in range(mp):
                ranks = grid[i, :, k].tolist()
                g = dist.new_group(ranks, backend=ddp_backend, **tkw)
                if (i, k) == (my_dp, my_mp):
                    topo.shard_group, topo.shard_ranks = g, ranks
    else:
        topo.shard_group, topo.shard_ranks = topo.dp_group, topo.dp_ranks
    topo.ready = True
    _TOPO = topo


def model_parallel_is_initialized() -> bool:
    return _TOPO.ready


def _need(group, what):
    if group is None:
        raise AssertionError(f"{what} parallel group is not initialized")
    return group


def get_model_parallel_group() -> dist.ProcessGroup:
    return _need(_TOPO.mp_group, "model")


def get_data_parallel_group() -> dist.ProcessGroup:
    return _need(_TOPO.dp_group, "data")


def get_chunk_parallel_group() -> dist.ProcessGroup:
    return _need(_TOPO.cp_group, "chunk")


def get_shard_parallel_group() -> dist.ProcessGroup:
    """Group of all ranks holding the same model-parallel slice (data x chunk)."""
    return _need(_TOPO.shard_group, "shard")


def get_model_parallel_world_size() -> int:
    return len(_TOPO.mp_ranks) if _TOPO.ready else 1


def get_data_parallel_world_size() -> int:
    return len(_TOPO.dp_ranks) if _TOPO.ready else 1


def get_chunk_parallel_world_size() -> int:
    return len(_TOPO.cp_ranks) if _TOPO.ready else 1


def get_model_parallel_rank() -> int:
    return _TOPO.mp_rank


def get_data_parallel_rank() -> int:
    return _TOPO.dp_rank


def get_chunk_parallel_rank() -> int:
    return _TOPO.cp_rank


def get_model_parallel_ranks() -> List[int]:
    return list(_TOPO.mp_ranks)


def get_data_parallel_ranks() -> List[int]:
    return list(_TOPO.dp_ranks)


def get_chunk_parallel_ranks() -> List[int]:
    _need(_TOPO.cp_group, "chunk")
    return list(_TOPO.cp_ranks)


def get_model_parallel_src_rank() -> int:
    """Global rank of model-parallel rank 0 in the caller's group."""
    if _TOPO.ready:
        return _TOPO.mp_ranks[0]
    return 0


def get_chunk_parallel_prev_rank() -> Optional[int]:
    return _TOPO.prev_chunk_rank


def get_chunk_parallel_next_rank() -> Optional[int]:
    return _TOPO.next_chunk_rank


def destroy_model_parallel() -> None:
    """Forget the groups (they are destroyed with the default group)."""
    global _TOPO
    _TOPO = _Topology()
