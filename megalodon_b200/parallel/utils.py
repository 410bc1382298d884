"""Small helpers shared by the parallel layers (API of the reference's
megalodon/distributed/utils.py:10-56).  `reduce_scalar` is device-agnostic:
it reduces on the GPU under NCCL and on the host under gloo."""
from __future__ import annotations

from typing import List, Optional, Union

import torch
import torch.distributed as dist

Scalar = Union[int, float]

ReduceOpMap = {
    "sum": dist.ReduceOp.SUM,
    "max": dist.ReduceOp.MAX,
    "min": dist.ReduceOp.MIN,
    "mean": dist.ReduceOp.AVG,
    "avg": dist.ReduceOp.AVG,
}


def ensure_divisibility(numerator: int, denominator: int) -> None:
    if numerator % denominator != 0:
        raise AssertionError(f"{numerator} is not divisible by {denominator}")


def divide_and_check_no_remainder(numerator: int, denominator: int) -> int:
    ensure_divisibility(numerator, denominator)
    return numerator // denominator


def split_tensor_along_specific_dim(tensor: torch.Tensor, num_partitions: int, split_dim: int,
                                    contiguous_split_chunks: bool = False) -> List[torch.Tensor]:
    width = divide_and_check_no_remainder(tensor.shape[split_dim], num_partitions)
    parts = torch.split(tensor, width, dim=split_dim)
    if contiguous_split_chunks:
        return [p.contiguous() for p in parts]
    return list(parts)


def comm_device(group: Optional[dist.ProcessGroup] = None) -> torch.device:
    """Device on which tensors handed to collectives of `group` must live."""
    if dist.is_available() and dist.is_initialized():
        backend = dist.get_backend(group)
        if "nccl" in str(backend):
            return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def reduce_scalar(x: Scalar, op: str, group: Optional[dist.ProcessGroup] = None) -> Scalar:
    if not (dist.is_available() and dist.is_initialized()):
        return x
    dev = comm_device(group)
    op = op.lower()
    is_float = isinstance(x, float) or op in ("mean", "avg")
    t = torch.tensor(float(x) if is_float else x, device=dev,
                     dtype=torch.float64 if is_float else torch.int64)
    if op in ("mean", "avg") and dev.type == "cpu":
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        t /= dist.get_world_size(group)
    else:
        dist.all_reduce(t, op=ReduceOpMap[op], group=group)
    return t.item()


def _is_gloo(group: Optional[dist.ProcessGroup]) -> bool:
    return "gloo" in str(dist.get_backend(group))


def all_gather_flat(out: torch.Tensor, inp: torch.Tensor, group: Optional[dist.ProcessGroup]) -> None:
    """out[W * n] <- concatenation over ranks of inp[n] (contiguous, same dtype)."""
    dist.all_gather_into_tensor(out.view(-1), inp.reshape(-1), group=group)


def reduce_scatter_flat(out: torch.Tensor, inp: torch.Tensor, group: Optional[dist.ProcessGroup]) -> None:
    """out[n] <- this rank's slice of the element-wise sum over ranks of inp[W * n].
    gloo has no reduce-scatter; there the sum is an all-reduce followed by a slice."""
    if _is_gloo(group):
        tmp = inp.clone()
        dist.all_reduce(tmp, group=group)
        r = dist.get_rank(group)
        out.copy_(tmp.view(-1)[r * out.numel():(r + 1) * out.numel()].view_as(out))
    else:
        dist.reduce_scatter_tensor(out.view(-1), inp.reshape(-1), group=group)
