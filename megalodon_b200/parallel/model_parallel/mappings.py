"""Autograd-aware tensor-parallel region boundaries.

Six mappings with the same names and forward/backward pairing as the reference
(megalodon/modules/model_parallel/mappings.py:93-198):

    copy_to          identity            / all-reduce
    reduce_from      all-reduce          / identity
    scatter_to       keep own slice      / all-gather
    gather_from      all-gather          / keep own slice
    gather_copy      all-gather          / reduce-scatter
    reduce_scatter   reduce-scatter      / all-gather

The collectives use the tensor forms (`all_gather_into_tensor`,
`reduce_scatter_tensor`) on a leading-dim layout and move the requested dim to
the front only when it is not already there, instead of building Python lists
of per-rank tensors.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..utils import all_gather_flat, reduce_scatter_flat
from ..initialize import (
    get_model_parallel_group,
    get_model_parallel_rank,
    get_model_parallel_world_size,
)


def _dim(x: torch.Tensor, dim: Optional[int]) -> int:
    return x.dim() - 1 if dim is None else dim % x.dim()


# Set by a decode session on tensor-parallel ranks (`use_small_collective`): small inference-time
# activations then go through one peer-memory kernel per collective, which a CUDA graph can hold.
_SMALL = [None]


def use_small_collective(obj) -> None:
    """`obj`: a `parallel.symm.SmallCollective` over the model-parallel group, or None to go back to NCCL."""
    _SMALL[0] = obj


_STRICT = [False]


def small_collective_strict(on: bool) -> None:
    """While on (a decode step being captured in a CUDA graph), a collective that the small-collective
    kernel cannot take raises instead of falling back to NCCL, which must not run inside the capture."""
    _STRICT[0] = bool(on)


def _small_for(x: torch.Tensor):
    sc = _SMALL[0]
    ok = sc is not None and not torch.is_grad_enabled() and sc.fits(x)
    if _STRICT[0] and not ok:
        raise RuntimeError(f"collective on a {tuple(x.shape)} {x.dtype} tensor cannot go through the "
                           "graph-capturable kernel")
    return sc if ok else None


def _all_reduce(x: torch.Tensor) -> torch.Tensor:
    if get_model_parallel_world_size() == 1:
        return x
    x = x.contiguous()
    sc = _small_for(x)
    if sc is not None:
        return sc.all_reduce(x)
    dist.all_reduce(x, group=get_model_parallel_group())
    return x


def _split(x: torch.Tensor, dim: Optional[int]) -> torch.Tensor:
    world = get_model_parallel_world_size()
    if world == 1:
        return x
    d = _dim(x, dim)
    width = x.shape[d] // world
    assert width * world == x.shape[d]
    r = get_model_parallel_rank()
    return x.narrow(d, r * width, width).contiguous()


def _gather(x: torch.Tensor, dim: Optional[int]) -> torch.Tensor:
    world = get_model_parallel_world_size()
    if world == 1:
        return x
    d = _dim(x, dim)
    x = x.contiguous()
    if d == x.dim() - 1:
        sc = _small_for(x)
        if sc is not None:
            return sc.all_gather_last_dim(x)
    out = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    all_gather_flat(out, x, get_model_parallel_group())
    # [W, ..., n_d, ...] -> [..., W * n_d, ...]
    out = out.movedim(0, d)
    shape = list(x.shape)
    shape[d] *= world
    return out.reshape(shape)


def _reduce_scatter(x: torch.Tensor, dim: Optional[int]) -> torch.Tensor:
    world = get_model_parallel_world_size()
    if world == 1:
        return x
    d = _dim(x, dim)
    width = x.shape[d] // world
    assert width * world == x.shape[d]
    shape = list(x.shape)
    shape[d] = width
    # [..., W * n_d, ...] -> [W, ..., n_d, ...] contiguous
    parts = x.reshape(shape[:d] + [world, width] + shape[d + 1:]).movedim(d, 0).contiguous()
    out = torch.empty(shape, dtype=x.dtype, device=x.device)
    reduce_scatter_flat(out, parts, get_model_parallel_group())
    return out


class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g)


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _all_reduce(x.clone() if get_model_parallel_world_size() > 1 else x)

    @staticmethod
    def backward(ctx, g):
        return g


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        return _split(x, dim)

    @staticmethod
    def backward(ctx, g):
        return _gather(g, ctx.dim), None


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        return _gather(x, dim)

    @staticmethod
    def backward(ctx, g):
        return _split(g, ctx.dim), None


class _GatherCopy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        return _gather(x, dim)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter(g, ctx.dim), None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        return _reduce_scatter(x, dim)

    @staticmethod
    def backward(ctx, g):
        return _gather(g, ctx.dim), None


def copy_to_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    return _Copy.apply(input_)


def reduce_from_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    return _Reduce.apply(input_)


def scatter_to_model_parallel_region(input_: torch.Tensor, dim: Optional[int] = None) -> torch.Tensor:
    return _Scatter.apply(input_, dim)


def gather_from_model_parallel_region(input_: torch.Tensor, dim: Optional[int] = None) -> torch.Tensor:
    return _Gather.apply(input_, dim)


def gather_copy_model_parallel_region(input_: torch.Tensor, dim: Optional[int] = None) -> torch.Tensor:
    return _GatherCopy.apply(input_, dim)


def reduce_scatter_model_parallel_region(input_: torch.Tensor, dim: Optional[int] = None) -> torch.Tensor:
    return _ReduceScatter.apply(input_, dim)
