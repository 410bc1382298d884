"""LayerNorm / RMSNorm modules with the `weight + 1` parameterisation, plus the
raw forward/backward helpers the reference exposes over apex
(megalodon/modules/layer_norm.py:14-129).  Here they sit on this framework's
own kernels (`ops.rms_norm`, `ops.layer_norm`); no apex."""
from __future__ import annotations

import numbers
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops


def _shape(normalized_shape):
    if isinstance(normalized_shape, numbers.Integral):
        normalized_shape = (int(normalized_shape),)
    shape = torch.Size(normalized_shape)
    assert len(shape) == 1, "only last-dim normalisation is supported"
    return shape


class FusedLayerNorm(nn.Module):
    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True):
        super().__init__()
        self.normalized_shape = _shape(normalized_shape)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if elementwise_affine:
            self.weight = nn.Parameter(torch.zeros(*self.normalized_shape))
            self.bias = nn.Parameter(torch.zeros(*self.normalized_shape))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    def forward(self, input_: torch.Tensor) -> torch.Tensor:
        return ops.layer_norm(input_, self.weight, self.bias, self.eps, weight_offset=1.0)

    def extra_repr(self):
        return f"{tuple(self.normalized_shape)}, eps={self.eps}, elementwise_affine={self.elementwise_affine}"


class FusedRMSNorm(nn.Module):
    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True):
        super().__init__()
        self.normalized_shape = _shape(normalized_shape)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if elementwise_affine:
            self.weight = nn.Parameter(torch.zeros(*self.normalized_shape))
        else:
            self.register_parameter("weight", None)

    def forward(self, input_: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(input_, self.weight, self.eps, weight_offset=1.0)

    def extra_repr(self):
        return f"{tuple(self.normalized_shape)}, eps={self.eps}, elementwise_affine={self.elementwise_affine}"


# Raw helpers: explicit forward returning the saved statistics, explicit backward.
def layernorm_fwd(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                  dim: int, eps: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    xf = x.float()
    mean = xf.mean(-1)
    invvar = torch.rsqrt(xf.var(-1, unbiased=False) + eps)
    return ops.layer_norm(x, weight, bias, eps, weight_offset=1.0), mean, invvar


def layernorm_bwd(y_grad, x, mean, invvar, weight, bias, dim: int, eps: float):
    xf, g = x.float(), y_grad.float()
    xhat = (xf - mean.unsqueeze(-1)) * invvar.unsqueeze(-1)
    w = None if weight is None else (weight + 1.0).float()
    gw = g if w is None else g * w
    dx = invvar.unsqueeze(-1) * (gw - gw.mean(-1, keepdim=True) - xhat * (gw * xhat).mean(-1, keepdim=True))
    if weight is None:
        return dx.to(x.dtype), None, None
    red = tuple(range(x.dim() - 1))
    return dx.to(x.dtype), (g * xhat).sum(red).to(weight.dtype), g.sum(red).to(weight.dtype)


def rmsnorm_fwd(x: torch.Tensor, weight: Optional[torch.Tensor], dim: int, eps: float):
    invvar = torch.rsqrt(x.float().pow(2).mean(-1) + eps)
    return ops.rms_norm(x, weight, eps, weight_offset=1.0), invvar


def rmsnorm_bwd(y_grad, x, invvar, weight, dim: int, eps: float):
    xf, g = x.float(), y_grad.float()
    xhat = xf * invvar.unsqueeze(-1)
    w = None if weight is None else (weight + 1.0).float()
    gw = g if w is None else g * w
    dx = invvar.unsqueeze(-1) * (gw - xhat * (gw * xhat).mean(-1, keepdim=True))
    if weight is None:
        return dx.to(x.dtype), None
    red = tuple(range(x.dim() - 1))
    return dx.to(x.dtype), (g * xhat).sum(red).to(weight.dtype)
