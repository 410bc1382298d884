"""The operator names of the reference's `megalodon.modules.fused_ops`
(fused_ops/__init__.py:1-14), served by `megalodon_b200.ops`.  The raw forward / backward pairs the
reference exports for attention and fftconv are provided as thin functions over the same kernels."""
from ...ops import (  # noqa: F401
    attention_softmax,
    ema_hidden,
    ema_parameters,
    fftconv,
    memory_efficient_dropout,
    memory_efficient_dropout_bwd,
    memory_efficient_dropout_fwd,
    swift_efficient_attention,
)
from ... import ops as _ops

import torch


def swift_efficient_attention_fwd(q, k, v, scale: float = 1.0, dropout: float = 0.0, use_causal_mask: bool = True):
    """Forward only (no autograd graph): y [B, L1, H, dv]."""
    with torch.no_grad():
        return _ops.attention(q, k, v, scale, dropout, use_causal_mask, training=dropout > 0.0)


def swift_efficient_attention_bwd(y_grad, q, k, v, scale: float = 1.0, use_causal_mask: bool = True):
    """Gradients (dq, dk, dv) of the attention output w.r.t. its inputs for a given output gradient;
    the probabilities are recomputed instead of being passed in."""
    q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
    with torch.enable_grad():
        y = _ops.attention(q, k, v, scale, 0.0, use_causal_mask, training=False)
    return torch.autograd.grad(y, (q, k, v), y_grad)


def fused_fftconv_fwd(x, k):
    """Forward only: causal long convolution of x [B, D, L] with k [D, L]."""
    with torch.no_grad():
        return _ops.fftconv(x, k)


def fused_fftconv_bwd(y_grad, x, k):
    """(dx, dk) for a given output gradient."""
    x, k = x.detach().requires_grad_(True), k.detach().requires_grad_(True)
    with torch.enable_grad():
        y = _ops.fftconv(x, k)
    return torch.autograd.grad(y, (x, k), y_grad)
