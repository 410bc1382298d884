"""TimestepNorm: group normalisation whose statistics are cumulative over
time, so that position t is normalised with the mean/variance of positions
<= t (plus a carried prefix).  Module interface and parameterisation follow
the reference (megalodon/modules/timestep_norm.py:67-131): `weight` and `bias`
are zero-initialised and applied as `weight + 1`; the starting statistics come
from `prior_count / prior_mean / exp(prior_logv)` unless the caller passes the
running values of the previous chunk (or previous chunk-parallel rank).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn
from torch.nn.parameter import Parameter

from .. import ops
from ..parallel.initialize import get_model_parallel_world_size
from ..parallel.utils import divide_and_check_no_remainder


def timestep_norm(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask=None,
                  num_groups=None, eps=1e-5):
    return ops.timestep_norm(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask,
                             num_groups, eps)


class TimestepNorm(nn.Module):
    def __init__(self, num_features: int, num_groups: Optional[int] = None, prior_count: int = 0,
                 eps: float = 1e-5) -> None:
        super().__init__()
        self.num_features = num_features
        self.num_groups = num_groups
        self._prior_count = prior_count
        if num_groups is None or num_groups == num_features:
            # one feature per group has zero within-step variance: a prior is needed
            num_groups = num_features
            assert prior_count > 1, "ungrouped TimestepNorm needs prior_count > 1"
        else:
            assert num_features % num_groups == 0
        world = get_model_parallel_world_size()
        self.features_per_partition = divide_and_check_no_remainder(num_features, world)
        self.groups_per_partition = divide_and_check_no_remainder(num_groups, world)

        self.register_buffer("prior_count", torch.tensor(prior_count, dtype=torch.int64))
        if prior_count > 0:
            self.prior_mean = Parameter(torch.zeros(self.groups_per_partition))
            self.prior_logv = Parameter(torch.zeros(self.groups_per_partition))
        else:
            self.register_buffer("prior_mean", torch.zeros(self.groups_per_partition))
            self.register_buffer("prior_logv", torch.zeros(self.groups_per_partition))
        self.weight = Parameter(torch.zeros(self.features_per_partition))
        self.bias = Parameter(torch.zeros(self.features_per_partition))
        self.eps = eps

    def initial_stats(self, batch_size: int, dtype: torch.dtype):
        count = self.prior_count.expand(batch_size).contiguous()
        mean = self.prior_mean.to(dtype).expand(batch_size, -1).contiguous()
        var = self.prior_logv.to(dtype).exp().expand(batch_size, -1).contiguous()
        return count, mean, var

    def forward(
        self,
        x: torch.Tensor,
        prev_count: Optional[torch.Tensor] = None,
        prev_mean: Optional[torch.Tensor] = None,
        prev_var: Optional[torch.Tensor] = None,
        padding_mask: Optional[torch.Tensor] = None,
    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        c0, m0, v0 = self.initial_stats(x.size(0), x.dtype)
        prev_count = c0 if prev_count is None else prev_count
        prev_mean = m0 if prev_mean is None else prev_mean
        prev_var = v0 if prev_var is None else prev_var
        return ops.timestep_norm(x, prev_count, prev_mean, prev_var, self.weight, self.bias,
                                 padding_mask, self.groups_per_partition, self.eps, gamma_offset=1.0)

    def extra_repr(self) -> str:
        return (f"num_features={self.num_features} ({self.features_per_partition}), "
                f"num_groups={self.num_groups} ({self.groups_per_partition}), "
                f"prior_count={self._prior_count}, eps={self.eps}")
