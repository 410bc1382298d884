"""Multi-dimensional complex exponential moving average (CEMA).

Per feature d and state index n:  h_t = q h_{t-1} + p x_t,
y_t = Re(sum_n gamma_n h_t,n) + omega x_t, with

    p = sigmoid(alpha),  q = (1 - sigmoid(alpha) sigmoid(delta)) e^{i theta_n},
    theta_n = sigmoid(theta) * (2 pi / N) * n   (n = 1..N),
    gamma = (gamma_re + i gamma_im) / sqrt(N).

Parameter shapes, initialisation and the eval-mode coefficient cache follow the
reference (megalodon/modules/complex_exponential_moving_average.py:18-150).
The feature permutation used by the theta initialisation is drawn on the host
and, when a process group exists, broadcast from rank 0 through whichever
backend is active (the reference hard-codes a CUDA broadcast).

`forward` keeps the reference's [B, D, L] interface; `forward_channels_last`
takes [B, L, D] directly, which is what the fused CUDA scan kernel consumes
(consecutive threads own consecutive features, so loads are coalesced without
a transpose).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from .. import ops
from ..parallel.initialize import get_model_parallel_rank, get_model_parallel_world_size
from ..parallel.utils import comm_device, divide_and_check_no_remainder

_r2c = torch.view_as_complex


def _global_permutation(n: int) -> torch.Tensor:
    idx = torch.randperm(n)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dev = comm_device(None)
        wire = idx.to(dev)
        dist.broadcast(wire, src=0)
        idx = wire.cpu()
    return idx


def _reset_parameters(alpha, delta, theta, gamma, omega, embed_dim: int) -> None:
    with torch.no_grad():
        nn.init.normal_(alpha, mean=0.0, std=0.2)
        nn.init.normal_(delta, mean=0.0, std=0.2)
        idx = _global_permutation(embed_dim)
        rate = math.log(embed_dim) / embed_dim
        freqs = torch.exp(torch.arange(1, embed_dim + 1, dtype=torch.float32) * -rate)[idx]
        theta.copy_(torch.log(freqs / (1.0 - freqs)).view(embed_dim, 1, 1))
        nn.init.normal_(gamma, mean=0.0, std=1.0)
        gamma[:, :, 1] = 0.0
        nn.init.trunc_normal_(omega, mean=0.0, std=0.25, a=-1.0, b=1.0)


class MultiHeadComplexEMA(nn.Module):
    def __init__(self, embed_dim: int, ndim: int = 16):
        super().__init__()
        self.embed_dim = embed_dim
        self.ndim = ndim
        self.scale = math.sqrt(1.0 / ndim)
        world = get_model_parallel_world_size()
        d = self.dim_per_partition = divide_and_check_no_remainder(embed_dim, world)
        self.alpha = nn.Parameter(torch.empty(d, ndim, 1))
        self.delta = nn.Parameter(torch.empty(d, ndim, 1))
        self.theta = nn.Parameter(torch.empty(d, 1, 1))
        self.gamma = nn.Parameter(torch.empty(d, ndim, 2))
        self.omega = nn.Parameter(torch.empty(d, 1))
        self._coeffs = None
        self._init_parameters()

    def _init_parameters(self) -> None:
        world = get_model_parallel_world_size()
        if world == 1:
            _reset_parameters(self.alpha, self.delta, self.theta, self.gamma, self.omega, self.embed_dim)
            return
        E, N = self.embed_dim, self.ndim
        master = [torch.empty(E, N, 1), torch.empty(E, N, 1), torch.empty(E, 1, 1),
                  torch.empty(E, N, 2), torch.empty(E, 1)]
        _reset_parameters(*master, E)
        lo = get_model_parallel_rank() * self.dim_per_partition
        with torch.no_grad():
            for dst, src in zip((self.alpha, self.delta, self.theta, self.gamma, self.omega), master):
                dst.copy_(src[lo:lo + self.dim_per_partition])

    def _calc_coeffs(self):
        theta = torch.sigmoid(self.theta.float()) * (2.0 * math.pi / self.ndim)
        n = torch.arange(1, self.ndim + 1, dtype=theta.dtype, device=theta.device).view(1, self.ndim, 1)
        theta = n * theta                                     # D x N x 1
        alpha = torch.sigmoid(self.alpha.float())
        delta = torch.sigmoid(self.delta.float())
        p = alpha
        q = torch.polar(1.0 - alpha * delta, theta)
        gamma = _r2c(self.gamma.float()) * self.scale         # D x N
        return p, q, gamma

    def coeffs(self):
        if self.training:
            self._coeffs = None
            return self._calc_coeffs()
        if self._coeffs is None:
            self._coeffs = self._calc_coeffs()
        return self._coeffs

    def train(self, mode: bool = True):
        self._coeffs = None
        return super().train(mode)

    def forward_channels_last(self, x: torch.Tensor, hx: Optional[torch.Tensor],
                              compute_last_state: bool) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """x [B, L, D] -> (y [B, L, D], last state [B, D, N] complex or None)."""
        p, q, gamma = self.coeffs()
        return ops.cema(x, p, q, gamma, self.omega, hx, compute_last_state)

    def forward(self, x: torch.Tensor, hx: Optional[torch.Tensor],
                compute_last_state: bool) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """x [B, D, L] (the reference layout)."""
        y, h = self.forward_channels_last(x.transpose(1, 2), hx, compute_last_state)
        return y.transpose(1, 2), h

    def extra_repr(self) -> str:
        return f"edim={self.embed_dim} ({self.dim_per_partition}), ndim={self.ndim}"
