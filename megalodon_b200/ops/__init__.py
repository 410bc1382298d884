"""Operator layer: one functional entry point per operator.

Each function runs the hand-written sm_100a kernel (`ops/cuda_ops.py` over the
`_C` extension) for CUDA tensors and the plain-PyTorch statement in
`ops/reference.py` for CPU tensors.  The names follow the reference's
`megalodon.modules.fused_ops` (fused_ops/__init__.py:1-14) plus the operators
the reference takes from apex / ATen (norms, linear, cross-entropy, AdamW).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import reference
from ._ext import have_ext, native_for, require as require_ext
from .dropout import (
    memory_efficient_dropout,
    memory_efficient_dropout_fwd,
    memory_efficient_dropout_bwd,
)

Tensor = torch.Tensor


def _cuda():
    from . import cuda_ops
    return cuda_ops


def _cpu_native_ok(x: Tensor, *others) -> bool:
    """The C++ host implementations (csrc/cpu_ops.cpp) cover fp32 forward passes without autograd."""
    if x.is_cuda or x.dtype != torch.float32 or not have_ext():
        return False
    if torch.is_grad_enabled() and any(t is not None and torch.is_tensor(t) and t.requires_grad for t in (x,) + others):
        return False
    return True


def _cpu_native_autograd_ok(x: Tensor, *others) -> bool:
    """fp32 host tensors that take part in autograd: forward and backward both run in C++
    (`ops/cpu_native.py`).  MEGALODON_B200_CPU_NATIVE_AUTOGRAD=0 keeps the PyTorch statements."""
    import os
    if x.is_cuda or x.dtype != torch.float32 or not have_ext():
        return False
    if os.environ.get("MEGALODON_B200_CPU_NATIVE_AUTOGRAD", "1") != "1":
        return False
    for t in others:
        if t is not None and torch.is_tensor(t) and (t.is_cuda or t.dtype not in (torch.float32, torch.complex64)):
            return False
    return torch.is_grad_enabled() and any(t is not None and torch.is_tensor(t) and t.requires_grad
                                           for t in (x,) + others)


# ------------------------------------------------------------------ GEMM-shaped
def linear(x: Tensor, w: Tensor, b: Optional[Tensor] = None, act: Optional[str] = None) -> Tensor:
    """y = act(x @ w^T + b); `act` is None or "silu"."""
    if native_for(x):
        return _cuda().linear(x, w, b, act)
    return reference.linear(x, w, b, act)


def linear_add(x: Tensor, w: Tensor, b: Optional[Tensor], addend: Tensor) -> Tensor:
    """x @ w^T + b + addend (on the GPU the addition rides in the GEMM epilogue)."""
    if native_for(x):
        return _cuda().linear_add(x, w, b, addend)
    return reference.linear(x, w, b, None) + addend


def qk_rotary(z: Tensor, gamma: Tensor, beta: Tensor, freqs_cis: Tensor, head_dim: int):
    """Shared q / k of the MEGA attention: (z (gamma + 1) / sqrt(head_dim) + beta) for the two rows of
    gamma / beta [2, S], then the rotary rotation; z [B, L, S], position of (b, l) = (b L + l) % len(freqs_cis)."""
    if native_for(z) and z.dtype in (torch.bfloat16, torch.float16) and z.shape[-1] % 8 == 0 and z.shape[-1] <= 8192:
        return _cuda().qk_rotary(z, gamma, beta, freqs_cis, head_dim)
    import math
    B, L, S = z.shape
    scale = (gamma + 1.0) / math.sqrt(head_dim)
    qk = z.unsqueeze(2) * scale.to(z.dtype) + beta.to(z.dtype)
    q, k = torch.unbind(qk, dim=2)
    P = freqs_cis.shape[0]
    shape = (B * L // P, P, S // head_dim, head_dim)
    q = rotary(q.reshape(shape), freqs_cis).reshape(B, L, S)
    k = rotary(k.reshape(shape), freqs_cis).reshape(B, L, S)
    return q, k


def decode_attention_native(q: Tensor, k_buf: Tensor) -> bool:
    return (native_for(q) and q.dtype in (torch.bfloat16, torch.float16) and k_buf.dtype == q.dtype
            and q.shape[-1] % 8 == 0 and k_buf.is_contiguous() and k_buf.shape[2] * 4 <= 200 * 1024)


def decode_attention(q: Tensor, k_buf: Tensor, v_buf: Tensor, pos: Tensor, scale: float) -> Tensor:
    """One decode step against fixed buffers: q [B, H, dk], k_buf [B, H, C, dk], v_buf [B, H, C, dv], `pos` a
    device index tensor [1]; keys 0 .. pos take part.  Returns [B, H, dv]."""
    if decode_attention_native(q, k_buf):
        return _cuda().decode_attention(q, k_buf, v_buf, pos, scale)
    scores = torch.einsum("bhd,bhcd->bhc", q.float(), k_buf.float()) * scale
    hidden = torch.arange(k_buf.size(2), device=pos.device) > pos
    probs = torch.softmax(scores.masked_fill(hidden, float("-inf")), dim=-1)
    return torch.einsum("bhc,bhcd->bhd", probs, v_buf.float()).to(q.dtype)


def swiglu(a: Tensor, b: Tensor) -> Tensor:
    if native_for(a):
        return _cuda().swiglu(a, b)
    return reference.swiglu(a, b)


# ------------------------------------------------------------------ norms
def rms_norm(x: Tensor, weight: Optional[Tensor], eps: float, weight_offset: float = 0.0) -> Tensor:
    """The scale applied is `weight + weight_offset`, formed in fp32."""
    if native_for(x):
        return _cuda().rms_norm(x, weight, eps, weight_offset)
    return reference.rms_norm(x, weight, eps, weight_offset)


def layer_norm(x: Tensor, weight: Optional[Tensor], bias: Optional[Tensor], eps: float,
               weight_offset: float = 0.0) -> Tensor:
    if native_for(x):
        return _cuda().layer_norm(x, weight, bias, eps, weight_offset)
    return reference.layer_norm(x, weight, bias, eps, weight_offset)


def timestep_norm(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask=None,
                  num_groups=None, eps: float = 1e-5, gamma_offset: float = 0.0):
    """Returns (y, count, mean, var); see `reference.timestep_norm`."""
    if native_for(x):
        return _cuda().timestep_norm(x, prev_count, prev_mean, prev_var, gamma, beta,
                                     padding_mask, num_groups, eps, gamma_offset)
    if _cpu_native_ok(x, prev_mean, prev_var, gamma, beta) and prev_count is not None:
        G = x.shape[-1] if num_groups is None else num_groups
        return require_ext().cpu_timestep_norm_fwd(x, prev_count, prev_mean, prev_var, gamma, float(gamma_offset),
                                                   beta, padding_mask, G, float(eps))
    if _cpu_native_autograd_ok(x, prev_mean, prev_var, gamma, beta) and prev_count is not None:
        from . import cpu_native
        return cpu_native.timestep_norm(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask,
                                        x.shape[-1] if num_groups is None else num_groups, eps, gamma_offset)
    return reference.timestep_norm(x, prev_count, prev_mean, prev_var, gamma, beta,
                                   padding_mask, num_groups, eps, gamma_offset)


def sequence_norm(x, gamma, beta, padding_mask=None, num_groups=None, eps: float = 1e-5,
                  length_last: bool = False):
    if native_for(x):
        return _cuda().sequence_norm(x, gamma, beta, padding_mask, num_groups, eps, length_last)
    if _cpu_native_ok(x, gamma, beta):
        return require_ext().cpu_sequence_norm_fwd(x, gamma, beta, padding_mask, int(num_groups or 0), float(eps),
                                                   bool(length_last))
    if _cpu_native_autograd_ok(x, gamma, beta):
        from . import cpu_native
        return cpu_native.sequence_norm(x, gamma, beta, padding_mask, int(num_groups or 0), eps, length_last)
    return reference.sequence_norm(x, gamma, beta, padding_mask, num_groups, eps, length_last)


# ------------------------------------------------------------------ CEMA
def ema_parameters(p, q, gamma, hx, length: int):
    if native_for(p):
        return _cuda().ema_parameters(p, q, gamma, hx, length)
    if (not p.is_cuda and have_ext() and not (torch.is_grad_enabled() and any(
            t is not None and t.requires_grad for t in (p, q, gamma, hx)))):
        k, b = require_ext().cpu_ema_parameters_fwd(p, q, gamma, hx, int(length))
        return k, b
    if _cpu_native_autograd_ok(p, q, gamma, hx):
        from . import cpu_native
        return cpu_native.ema_parameters(p, q, gamma, hx, length)
    return reference.ema_parameters(p, q, gamma, hx, length)


def ema_hidden(x, p, q, hx):
    if native_for(x):
        return _cuda().ema_hidden(x, p, q, hx)
    if _cpu_native_ok(x, p, q, hx):
        return require_ext().cpu_ema_hidden_fwd(x, p, q, hx)
    if _cpu_native_autograd_ok(x, p, q, hx):
        from . import cpu_native
        return cpu_native.ema_hidden(x, p, q, hx)
    return reference.ema_hidden(x, p, q, hx)


def fftconv(x, k):
    if native_for(x):
        return _cuda().fftconv(x, k)
    return reference.fftconv(x, k)


def rfft(x, flip: bool = False):
    if native_for(x):
        return _cuda().rfft(x, flip)
    return reference.rfft(x, flip)


def cema(x, p, q, gamma, omega, hx, compute_last_state: bool):
    """Fused complex-EMA layer on channels-last x [B, L, D] -> (y, h_last)."""
    if native_for(x):
        return _cuda().cema(x, p, q, gamma, omega, hx, compute_last_state)
    if _cpu_native_ok(x, p, q, gamma, omega, hx):
        y, h = require_ext().cpu_cema_fwd(x, p, q, gamma, omega, hx)
        return y, (h if compute_last_state else None)
    if _cpu_native_autograd_ok(x, p, q, gamma, omega, hx):
        from . import cpu_native
        return cpu_native.cema(x, p, q, gamma, omega, hx, compute_last_state)
    return reference.cema(x, p, q, gamma, omega, hx, compute_last_state)


# ------------------------------------------------------------------ attention
def attention(q, k, v, scale: float = 1.0, dropout: float = 0.0, use_causal_mask: bool = True,
              training: bool = True):
    if native_for(q):
        return _cuda().attention(q, k, v, scale, dropout, use_causal_mask, training)
    return reference.attention(q, k, v, scale, dropout, use_causal_mask, training)


swift_efficient_attention = attention


def attention_softmax(x, dropout: float = 0.0, use_causal_mask: bool = True, training: bool = True):
    if native_for(x):
        return _cuda().attention_softmax(x, dropout, use_causal_mask, training)
    return reference.attention_softmax(x, dropout, use_causal_mask, training)


def rotary(x, freqs_cis, conj: bool = False):
    if native_for(x):
        return _cuda().rotary(x, freqs_cis, conj)
    return reference.rotary(x, freqs_cis, conj)


# ------------------------------------------------------------------ loss / optimiser
def sum_squares(g: Tensor, out: Tensor) -> None:
    """out (fp64 scalar tensor) += sum(g^2)."""
    if native_for(g):
        return _cuda().sum_squares(g, out)
    out.add_(g.double().pow(2).sum())


def cross_entropy(logits, target, weight=None, ignore_index: int = -100, label_smoothing: float = 0.0):
    """Per-token negative log-likelihood [N]; logits [N, V] in any float dtype."""
    if native_for(logits) and weight is None and label_smoothing == 0.0:
        return _cuda().cross_entropy(logits, target, ignore_index)
    return reference.cross_entropy(logits, target, weight, ignore_index, label_smoothing)


def adamw_step(param, grad, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
               low=None, scale_ptr=None):
    """`scale_ptr`: optional device scalar multiplied into the gradient (deferred clipping)."""
    if native_for(param):
        return _cuda().adamw_step(param, grad, m, v, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                                  weight_decay=weight_decay, step=step, grad_scale=grad_scale, low=low,
                                  scale_ptr=scale_ptr)
    if scale_ptr is not None:
        grad_scale = grad_scale * float(scale_ptr)
    return reference.adamw_step(param, grad, m, v, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                                weight_decay=weight_decay, step=step, grad_scale=grad_scale, low=low)
