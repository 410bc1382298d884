"""Dropout that stores no mask: the backward pass regenerates the Bernoulli
mask from the RNG state captured in the forward pass (same contract as the
reference's fused_ops/memory_efficient_dropout.py:37-96, but device-agnostic:
it snapshots the generator of whichever device holds the tensor)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def _get_state(device: torch.device) -> torch.Tensor:
    if device.type == "cuda":
        return torch.cuda.get_rng_state(device)
    return torch.get_rng_state()


def _set_state(device: torch.device, state: torch.Tensor) -> None:
    if device.type == "cuda":
        torch.cuda.set_rng_state(state, device)
    else:
        torch.set_rng_state(state)


def _mask_like(x: torch.Tensor, p: float) -> torch.Tensor:
    return torch.empty_like(x).bernoulli_(1.0 - p).div_(1.0 - p)


def memory_efficient_dropout_fwd(x: torch.Tensor, p: float, training: bool,
                                 rng_state: Optional[torch.Tensor] = None
                                 ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    if not 0.0 <= p <= 1.0:
        raise ValueError(f"dropout probability has to be between 0 and 1, but got {p}")
    if not training or p == 0.0:
        return x, None
    if rng_state is None:
        state = _get_state(x.device)
        return x * _mask_like(x, p), state
    saved = _get_state(x.device)
    _set_state(x.device, rng_state)
    noise = _mask_like(x, p)
    _set_state(x.device, saved)
    return x * noise, noise


def memory_efficient_dropout_bwd(y_grad: torch.Tensor, p: float, rng_state: Optional[torch.Tensor],
                                 noise: Optional[torch.Tensor] = None) -> torch.Tensor:
    if p == 0.0 or rng_state is None and noise is None:
        return y_grad
    if noise is None:
        saved = _get_state(y_grad.device)
        _set_state(y_grad.device, rng_state)
        noise = _mask_like(y_grad, p)
        _set_state(y_grad.device, saved)
    return y_grad * noise


class _Dropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, training):
        y, state = memory_efficient_dropout_fwd(x, p, training)
        ctx.p = p if state is not None else 0.0
        ctx.state = state
        return y

    @staticmethod
    def backward(ctx, g):
        return memory_efficient_dropout_bwd(g, ctx.p, ctx.state), None, None


def memory_efficient_dropout(x: torch.Tensor, p: float = 0.0, training: bool = True) -> torch.Tensor:
    if not training or p == 0.0:
        return x
    if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16, torch.float16):
        from ._ext import native_for
        if native_for(x):
            from . import cuda_ops
            return cuda_ops.dropout(x, p)      # Philox mask generated in the kernel
    return _Dropout.apply(x, p, training)
