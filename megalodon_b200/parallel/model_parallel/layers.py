"""Tensor-parallel building blocks: embedding split along the embedding dim,
column-parallel and row-parallel linear layers (interfaces of the reference's
megalodon/modules/model_parallel/layers.py:65-349).

Weight initialisation under model parallelism draws the full ("master") matrix
from the caller's RNG on every rank and keeps this rank's slice, so a model
built with mp>1 from a given seed holds exactly the slices of the model built
with mp=1 from the same seed.

The matrix products go through `ops.linear`, which on a GPU runs the tcgen05
GEMM with the bias/activation epilogue fused in.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn.functional as F
import torch.nn.init as init
from torch.nn.parameter import Parameter

from ... import ops
from ..initialize import get_model_parallel_rank, get_model_parallel_world_size
from ..utils import divide_and_check_no_remainder
from .mappings import (
    copy_to_model_parallel_region,
    gather_copy_model_parallel_region,
    gather_from_model_parallel_region,
    reduce_from_model_parallel_region,
    reduce_scatter_model_parallel_region,
    scatter_to_model_parallel_region,
)

InitFn = Callable[[torch.Tensor], torch.Tensor]


def _initialize_affine_weight(weight: torch.Tensor, out_features: int, in_features: int,
                              per_partition_size: int, partition_dim: int, init_method: InitFn,
                              stride: int = 1, return_master_weight: bool = False,
                              partition: Optional[tuple] = None) -> Optional[torch.Tensor]:
    """`partition = (index, count)`: slice number `index` of `count` instead of (rank, world) - several
    ranks may then hold the same slice."""
    world = get_model_parallel_world_size()
    index = get_model_parallel_rank()
    if partition is not None:
        index, world = partition
    if world == 1 and partition is None:
        init_method(weight)
        return weight if return_master_weight else None
    master = torch.empty(out_features, in_features, dtype=weight.dtype, device="cpu")
    init_method(master)
    block = divide_and_check_no_remainder(per_partition_size, stride)
    pieces = torch.split(master, block, dim=partition_dim)
    mine = pieces[index::world]
    with torch.no_grad():
        weight.copy_(torch.cat(mine, dim=partition_dim))
    return master if return_master_weight else None


class ParallelEmbedding(torch.nn.Module):
    """Embedding table whose *columns* (embedding features) are split over the
    model-parallel group; with `gather_output=False` the residual stream stays
    feature-sharded between blocks."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None,
                 max_norm: Optional[float] = None, norm_type: float = 2.0,
                 scale_grad_by_freq: bool = False, sparse: bool = False, gather_output: bool = True,
                 init_method: InitFn = init.normal_) -> None:
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.padding_idx = padding_idx
        self.max_norm = max_norm
        self.norm_type = norm_type
        self.scale_grad_by_freq = scale_grad_by_freq
        self.sparse = sparse
        self.gather_output = gather_output
        world = get_model_parallel_world_size()
        self.embedding_dim_per_partition = divide_and_check_no_remainder(embedding_dim, world)
        self.weight = Parameter(torch.empty(num_embeddings, self.embedding_dim_per_partition))
        _initialize_affine_weight(self.weight, num_embeddings, embedding_dim,
                                  self.embedding_dim_per_partition, 1, init_method)

    def forward(self, input_: torch.Tensor) -> torch.Tensor:
        out = F.embedding(input_, self.weight, self.padding_idx, self.max_norm, self.norm_type,
                          self.scale_grad_by_freq, self.sparse)
        return gather_from_model_parallel_region(out) if self.gather_output else out

    def extra_repr(self) -> str:
        return (f"{self.num_embeddings}, {self.embedding_dim} ({self.embedding_dim_per_partition}), "
                f"gather_output={self.gather_output}")


class ColumnParallelLinear(torch.nn.Module):
    """Y = X A^T + b with the output features of A split over the group.

    `input_is_parallel=True` means X arrives feature-sharded and is
    all-gathered in forward (reduce-scattered in backward); otherwise X is
    replicated and its gradient is all-reduced in backward.
    `activation="silu"` fuses the activation into the GEMM epilogue."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 input_is_parallel: bool = False, gather_output: bool = False,
                 init_method: InitFn = init.xavier_normal_, stride: int = 1,
                 keep_master_weight_for_test: bool = False, activation: Optional[str] = None,
                 partition: Optional[tuple] = None) -> None:
        """`partition = (index, count)`: this rank holds output slice `index` of `count` (count smaller
        than the group: consecutive ranks hold the same slice and compute the same output).  Used
        where a projection must be replicated over part of the group - the shared q/k projection when
        one attention head is split over several ranks.  Forward only: in training the gradient of a
        replicated slice would have to be summed over its replicas, which this layer does not do."""
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.input_is_parallel = input_is_parallel
        self.gather_output = gather_output
        self.activation = activation
        self.partition = partition
        world = get_model_parallel_world_size() if partition is None else partition[1]
        assert partition is None or not gather_output, "a replicated partition cannot be gathered"
        self.output_size_per_partition = divide_and_check_no_remainder(out_features, world)
        self.weight = Parameter(torch.empty(self.output_size_per_partition, in_features))
        self.has_bias = bias
        if bias:
            self.bias = Parameter(torch.zeros(self.output_size_per_partition))
        else:
            self.register_parameter("bias", None)
        self.master_weight = _initialize_affine_weight(
            self.weight, out_features, in_features, self.output_size_per_partition, 0,
            init_method, stride=stride, return_master_weight=keep_master_weight_for_test, partition=partition)

    def get_master_weight(self) -> torch.Tensor:
        return gather_from_model_parallel_region(self.weight.data.t()).t()

    def forward(self, input_: torch.Tensor) -> torch.Tensor:
        from .. import tp_comm
        if self.input_is_parallel and not self.gather_output and tp_comm.usable(input_):
            # all-gather of the feature-sharded input fused into the GEMM (peer-memory TMA loads)
            return tp_comm.AGLinear.apply(input_, self.weight, self.bias, self.activation)
        if self.input_is_parallel:
            x = gather_copy_model_parallel_region(input_)
        else:
            x = copy_to_model_parallel_region(input_)
        y = ops.linear(x, self.weight, self.bias, self.activation)
        return gather_from_model_parallel_region(y) if self.gather_output else y

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features} "
                f"({self.output_size_per_partition}), bias={self.has_bias}, "
                f"parallel_input={self.input_is_parallel}, gather_output={self.gather_output}")


class RowParallelLinear(torch.nn.Module):
    """Y = X A^T + b with the input features of A split over the group; the
    partial products are reduce-scattered (`parallel_output=True`) or
    all-reduced."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 input_is_parallel: bool = False, parallel_output: bool = False,
                 init_method: InitFn = init.xavier_normal_, stride: int = 1,
                 keep_master_weight_for_test: bool = False):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.input_is_parallel = input_is_parallel
        self.parallel_output = parallel_output
        world = get_model_parallel_world_size()
        self.input_size_per_partition = divide_and_check_no_remainder(in_features, world)
        self.output_size_per_partition = (
            divide_and_check_no_remainder(out_features, world) if parallel_output else out_features)
        self.weight = Parameter(torch.empty(out_features, self.input_size_per_partition))
        self.has_bias = bias
        if bias:
            self.bias = Parameter(torch.zeros(self.output_size_per_partition))
        else:
            self.register_parameter("bias", None)
        self.master_weight = _initialize_affine_weight(
            self.weight, out_features, in_features, self.input_size_per_partition, 1,
            init_method, stride=stride, return_master_weight=keep_master_weight_for_test)

    def get_master_weight(self) -> torch.Tensor:
        return gather_from_model_parallel_region(self.weight.data)

    def forward(self, input_: torch.Tensor) -> torch.Tensor:
        from .. import tp_comm
        x = input_ if self.input_is_parallel else scatter_to_model_parallel_region(input_)
        if self.parallel_output and tp_comm.usable(x):
            # reduce-scatter fused into the GEMM epilogue (partials pushed into the owners' memory)
            y = tp_comm.LinearRS.apply(x, self.weight)
            return y if self.bias is None else y + self.bias
        y = ops.linear(x, self.weight, None, None)
        if self.parallel_output:
            y = reduce_scatter_model_parallel_region(y)
        else:
            y = reduce_from_model_parallel_region(y)
        return y if self.bias is None else y + self.bias

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features} ({self.input_size_per_partition}), "
                f"out_features={self.out_features} ({self.output_size_per_partition}), "
                f"bias={self.has_bias}, parallel_input={self.input_is_parallel}, "
                f"parallel_output={self.parallel_output}")
