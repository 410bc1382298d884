"""Autograd wrappers around the sm_100a kernels in `megalodon_b200._C`.

One `torch.autograd.Function` per operator: forward and backward each call a
hand-written kernel.  The reference keeps the same split between Python
autograd wrappers and native fwd/bwd entry points
(megalodon/modules/fused_ops/*.py, megalodon/modules/timestep_norm.py:13-64).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import reference
from ._ext import require

Tensor = torch.Tensor
_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def _C():
    return require()


# ----------------------------------------------------------------------------- GEMM / linear
_GEMM_ERR = {}
_GEMM_BACKEND = [os.environ.get("MEGALODON_B200_GEMM", "tcgen05")]
_launches = [0]          # kernels launched by this framework (bench bookkeeping)


def count_launches() -> int:
    return _launches[0]


def _bump(n: int = 1) -> None:
    _launches[0] += n


def set_gemm_backend(name: str) -> None:
    """"tcgen05": this framework's kernel; "cublas": torch.matmul (baseline only)."""
    assert name in ("tcgen05", "cublas")
    _GEMM_BACKEND[0] = name


def gemm_backend() -> str:
    return _GEMM_BACKEND[0]


def _err_flag(device: torch.device) -> Tensor:
    key = (device.type, device.index)
    if key not in _GEMM_ERR:
        _GEMM_ERR[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _GEMM_ERR[key]


def check_kernel_errors(device: Optional[torch.device] = None) -> None:
    """Raise if a kernel gave up on one of its bounded waits (synchronises)."""
    for key, flag in _GEMM_ERR.items():
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            raise RuntimeError(f"tcgen05 kernel wait timed out on {key} (role code {code})")


def gemm(a: Tensor, b: Tensor, bias: Optional[Tensor] = None, act: Optional[str] = None, *,
         a_mn: bool = False, b_mn: bool = False, want_preact: bool = False,
         out_dtype: Optional[torch.dtype] = None):
    """C = act(A B^T + bias).  `a_mn` / `b_mn`: operand is stored [K, rows].  Returns (C, preact | None)."""
    out_dtype = out_dtype or a.dtype
    # TMA needs 16-byte row strides: the contiguous dim of each operand and N must be multiples of 8
    aligned = a.shape[-1] % 8 == 0 and b.shape[-1] % 8 == 0 and (b.shape[1] if b_mn else b.shape[0]) % 8 == 0
    if _GEMM_BACKEND[0] == "cublas" or a.dtype == torch.float32 or not aligned:
        A = a.t() if a_mn else a
        Bm = b if b_mn else b.t()
        pre = torch.matmul(A, Bm)
        if bias is not None:
            pre = pre + bias.to(pre.dtype)
        out = F.silu(pre) if act == "silu" else pre
        return out.to(out_dtype), (pre.to(out_dtype) if want_preact else None)
    _bump()
    out, pre, rc = _C().gemm(a.contiguous(), b.contiguous(), bias, 1 if act == "silu" else 0, a_mn, b_mn,
                             want_preact, _DT[out_dtype], _err_flag(a.device))
    if rc != 0:
        raise RuntimeError(f"tcgen05 GEMM launch failed with code {rc}")
    return out, pre


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, act):
        x2 = x.reshape(-1, x.shape[-1])
        need_pre = act is not None and any(ctx.needs_input_grad[:3])
        y, pre = gemm(x2, w, b, act, want_preact=need_pre)
        ctx.save_for_backward(x2, w, pre if pre is not None else torch.empty(0, device=x.device))
        ctx.has_bias = b is not None
        ctx.act = act
        ctx.x_shape = x.shape
        ctx.bias_dtype = b.dtype if b is not None else None
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, pre = ctx.saved_tensors
        g = dy.reshape(-1, dy.shape[-1]).contiguous()
        if ctx.act == "silu":
            g = silu_bwd(g, pre)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx, _ = gemm(g, w, None, None, b_mn=True)          # [M, N] x [N, K] -> [M, K]
            dx = dx.view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dw, _ = gemm(g, x2, None, None, a_mn=True, b_mn=True)   # [M, N]^T x [M, K] -> [N, K]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = g.sum(0, dtype=torch.float32).to(ctx.bias_dtype)
        return dx, dw, db, None


def linear(x: Tensor, w: Tensor, b: Optional[Tensor] = None, act: Optional[str] = None) -> Tensor:
    if x.dtype == torch.float32:
        return reference.linear(x, w, b, act)
    return _Linear.apply(x, w, b, act)


def silu_bwd(g: Tensor, pre: Tensor) -> Tensor:
    """g * silu'(pre) through the SwiGLU-backward kernel (b = 1 gives da = g silu'(a))."""
    _bump()
    ones = _ones_like_cache(pre)
    da, _ = _C().swiglu_bwd(g.contiguous(), pre.contiguous(), ones)
    return da


_ONES = {}


def _ones_like_cache(t: Tensor) -> Tensor:
    key = (t.device, t.dtype, t.numel())
    if key not in _ONES:
        _ONES.clear()
        _ONES[key] = torch.ones(t.numel(), dtype=t.dtype, device=t.device)
    return _ONES[key].view(t.shape)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        a, b = a.contiguous(), b.contiguous()
        ctx.save_for_backward(a, b)
        _bump()
        return _C().swiglu_fwd(a, b)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        _bump()
        da, db = _C().swiglu_bwd(g.contiguous(), a, b)
        return da, db


def swiglu(a: Tensor, b: Tensor) -> Tensor:
    return _SwiGLU.apply(a, b)


# ----------------------------------------------------------------------------- norms
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, offset):
        xc = x.contiguous()
        w = None if weight is None else weight.contiguous()
        _bump()
        y, rstd = _C().rms_norm_fwd(xc, w, offset, eps)
        ctx.save_for_backward(xc, rstd, w if w is not None else torch.empty(0, device=x.device))
        ctx.has_w = w is not None
        ctx.offset = offset
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, rstd, w = ctx.saved_tensors
        _bump()
        dx, dw = _C().rms_norm_bwd(dy.contiguous(), xc, w if ctx.has_w else None, ctx.offset, rstd)
        if dw is not None:
            dw = dw.to(w.dtype)
        return dx, dw, None, None


def rms_norm(x, weight, eps, weight_offset: float = 0.0):
    return _RMSNorm.apply(x, weight, eps, weight_offset)


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, offset):
        xc = x.contiguous()
        w = None if weight is None else weight.contiguous()
        b = None if bias is None else bias.contiguous()
        _bump()
        y, mean, rstd = _C().layer_norm_fwd(xc, w, b, offset, eps)
        ctx.save_for_backward(xc, mean, rstd, w if w is not None else torch.empty(0, device=x.device))
        ctx.has_w = w is not None
        ctx.has_b = b is not None
        ctx.offset = offset
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, mean, rstd, w = ctx.saved_tensors
        _bump()
        dx, dw, db = _C().layer_norm_bwd(dy.contiguous(), xc, w if ctx.has_w else None, ctx.offset, mean, rstd)
        if dw is not None:
            dw = dw.to(w.dtype)
        db = db.to(w.dtype) if (db is not None and ctx.has_b) else None
        return dx, dw, db, None, None


def layer_norm(x, weight, bias, eps, weight_offset: float = 0.0):
    return _LayerNorm.apply(x, weight, bias, eps, weight_offset)


class _TimestepNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, prev_count, prev_mean, prev_var, gamma, beta, mask, groups, eps, offset):
        xc = x.contiguous()
        G = x.shape[-1] if groups is None else groups
        pm = prev_mean.to(x.dtype).contiguous()
        pv = prev_var.to(x.dtype).contiguous()
        gm, bt = gamma.contiguous(), beta.contiguous()
        mk = None if mask is None else mask.contiguous()
        _bump(3)
        y, count, mean, var, cummean, cumrstd = _C().timestep_norm_fwd(
            xc, prev_count.contiguous(), pm, pv, gm, offset, bt, mk, G, eps)
        ctx.save_for_backward(xc, pm, count, cummean, cumrstd, gm,
                              mk if mk is not None else torch.empty(0, device=x.device))
        ctx.has_mask = mk is not None
        ctx.G = G
        ctx.offset = offset
        ctx.stat_dtypes = (prev_mean.dtype, prev_var.dtype)
        ctx.mark_non_differentiable(count)
        return y, count, mean, var

    @staticmethod
    def backward(ctx, dy, _dcount, dmean, dvar):
        xc, pm, count, cummean, cumrstd, gm, mk = ctx.saved_tensors
        dmean = torch.zeros_like(pm) if dmean is None else dmean.to(pm.dtype).contiguous()
        dvar = torch.zeros_like(pm) if dvar is None else dvar.to(pm.dtype).contiguous()
        _bump(3)
        dx, dpm, dpv, dgamma, dbeta = _C().timestep_norm_bwd(
            dy.contiguous(), dmean, dvar, xc, pm, count, cummean, cumrstd, gm, ctx.offset,
            mk if ctx.has_mask else None, ctx.G)
        return (dx, None, dpm.to(ctx.stat_dtypes[0]), dpv.to(ctx.stat_dtypes[1]), dgamma.to(gm.dtype),
                dbeta.to(gm.dtype), None, None, None, None)


def timestep_norm(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask, num_groups, eps,
                  gamma_offset: float = 0.0):
    return _TimestepNorm.apply(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask, num_groups,
                               eps, gamma_offset)


def sequence_norm(x, gamma, beta, padding_mask, num_groups, eps, length_last):
    return reference.sequence_norm(x, gamma, beta, padding_mask, num_groups, eps, length_last)


# ----------------------------------------------------------------------------- CEMA
def _c2r(t: Tensor) -> Tensor:
    return torch.view_as_real(t.to(torch.complex64).contiguous())


class _CEMA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, q, gamma, omega, hx, want_last):
        D = x.shape[-1]
        xc = x.contiguous()
        p2 = p.reshape(D, -1).float().contiguous()
        N = p2.shape[1]
        q2 = _c2r(q.reshape(D, N))
        g2 = _c2r(gamma.reshape(D, N))
        om = omega.reshape(D).float().contiguous()
        h2 = None if hx is None else _c2r(hx)
        S = -(-x.shape[1] // 128)
        _bump(3 if S > 1 else 1)
        y, h_last = _C().cema_fwd(xc, p2, q2, g2, om, h2, bool(want_last))
        ctx.save_for_backward(xc, p2, q2, g2, om, h2 if h2 is not None else torch.empty(0, device=x.device))
        ctx.has_h = h2 is not None
        ctx.shapes = (p.shape, q.shape, gamma.shape, omega.shape)
        ctx.dtypes = (p.dtype, omega.dtype)
        ctx.S = S
        if h_last is None:
            return y, None
        return y, torch.view_as_complex(h_last)

    @staticmethod
    def backward(ctx, dy, dh_last):
        xc, p2, q2, g2, om, h2 = ctx.saved_tensors
        dh = None if dh_last is None else _c2r(dh_last)
        _bump(6 if ctx.S > 1 else 2)
        dx, dp, dq, dg, dom, dhx = _C().cema_bwd(dy.contiguous(), xc, p2, q2, g2, om,
                                                 h2 if ctx.has_h else None, dh)
        ps, qs, gs, os_ = ctx.shapes
        return (dx, dp.view(ps).to(ctx.dtypes[0]), torch.view_as_complex(dq).view(qs),
                torch.view_as_complex(dg).view(gs), dom.view(os_).to(ctx.dtypes[1]),
                torch.view_as_complex(dhx) if ctx.has_h else None, None)


def cema(x, p, q, gamma, omega, hx, compute_last_state: bool):
    N = p.reshape(x.shape[-1], -1).shape[1]
    if N not in (1, 2, 4, 8, 16, 32):
        return reference.cema(x, p, q, gamma, omega, hx, compute_last_state)
    return _CEMA.apply(x, p, q, gamma, omega, hx, compute_last_state)


def ema_parameters(p, q, gamma, hx, length):
    return reference.ema_parameters(p, q, gamma, hx, length)


def ema_hidden(x, p, q, hx):
    return reference.ema_hidden(x, p, q, hx)


def fftconv(x, k):
    return reference.fftconv(x, k)


def rfft(x, flip=False):
    return reference.rfft(x, flip)


# ----------------------------------------------------------------------------- attention
def attention(q, k, v, scale, dropout, use_causal_mask, training):
    return reference.attention(q, k, v, scale, dropout, use_causal_mask, training)


def attention_softmax(x, dropout, use_causal_mask, training):
    return reference.attention_softmax(x, dropout, use_causal_mask, training)


class _Rotary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, freqs, conj):
        ctx.save_for_backward(freqs)
        ctx.conj = conj
        _bump()
        return _C().rotary(x.contiguous(), freqs, conj)

    @staticmethod
    def backward(ctx, g):
        (freqs,) = ctx.saved_tensors
        _bump()
        return _C().rotary(g.contiguous(), freqs, not ctx.conj), None, None


def rotary(x, freqs_cis, conj=False):
    freqs = torch.view_as_real(freqs_cis.to(torch.complex64).contiguous())
    return _Rotary.apply(x, freqs, conj)


# ----------------------------------------------------------------------------- loss / optimiser
class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, ignore_index):
        lc = logits.contiguous()
        tc = target.contiguous()
        _bump()
        loss, lse = _C().cross_entropy_fwd(lc, tc, ignore_index)
        ctx.save_for_backward(lc, tc, lse)
        ctx.ignore_index = ignore_index
        return loss

    @staticmethod
    def backward(ctx, dloss):
        lc, tc, lse = ctx.saved_tensors
        _bump()
        return _C().cross_entropy_bwd(lc, tc, lse, dloss.contiguous(), ctx.ignore_index), None, None


def cross_entropy(logits, target, ignore_index=-100):
    return _CrossEntropy.apply(logits, target, ignore_index)


def adamw_step(param, grad, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, low=None,
               scale_ptr=None):
    _bump()
    _C().adamw_step(param, grad.contiguous(), m, v, low, lr, beta1, beta2, eps, weight_decay, step,
                    grad_scale, scale_ptr)


def sum_squares(g: Tensor, out: Tensor) -> None:
    _bump()
    _C().sum_squares(g, out)


def clip_coef(sumsq: Tensor, max_norm: float):
    _bump()
    return _C().clip_coef(sumsq, max_norm)


def scale_by_ptr(g: Tensor, scale: Tensor) -> None:
    _bump()
    _C().scale_by_ptr(g, scale)
