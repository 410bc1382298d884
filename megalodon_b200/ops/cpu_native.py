"""Autograd over the C++ host implementations (csrc/cpu_ops.cpp forward, csrc/cpu_ops_bwd.cpp backward).

fp32 CPU tensors that take part in autograd go through these functions, so that training and the
gradient checks on a machine without a GPU run the same native recurrences as the reference's CPU code
(megalodon/csrc/ops/timestep_norm.cc:218-450, sequence_norm.cc, ema_parameters.cc:17-188,
ema_hidden.cc:15-159) instead of the element-by-element PyTorch statements of `ops/reference.py`, which
stay the oracle the kernels are tested against.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ._ext import require as _require


def _c(t: Optional[Tensor]) -> Optional[Tensor]:
    return None if t is None else t.contiguous()


class _TimestepNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, prev_count, prev_mean, prev_var, gamma, beta, mask, groups, eps, gamma_offset):
        x, prev_mean, prev_var, gamma, beta = (_c(t) for t in (x, prev_mean, prev_var, gamma, beta))
        y, count, mean, var = _require().cpu_timestep_norm_fwd(x, prev_count, prev_mean, prev_var, gamma,
                                                              float(gamma_offset), beta, mask, int(groups), float(eps))
        ctx.save_for_backward(x, prev_count, prev_mean, prev_var, gamma)
        ctx.mask, ctx.meta = mask, (int(groups), float(eps), float(gamma_offset))
        ctx.mark_non_differentiable(count)
        return y, count, mean, var

    @staticmethod
    def backward(ctx, gy, _gcount, gmean, gvar):
        x, prev_count, prev_mean, prev_var, gamma = ctx.saved_tensors
        groups, eps, gamma_offset = ctx.meta
        gy = torch.zeros_like(x) if gy is None else gy.contiguous()
        gmean = torch.zeros_like(prev_mean) if gmean is None else gmean.contiguous()
        gvar = torch.zeros_like(prev_var) if gvar is None else gvar.contiguous()
        dx, dpm, dpv, dgamma, dbeta = _require().cpu_timestep_norm_bwd(gy, gmean, gvar, x, prev_count, prev_mean,
                                                                      prev_var, gamma, gamma_offset, ctx.mask, groups, eps)
        return dx, None, dpm, dpv, dgamma, dbeta, None, None, None, None


class _SequenceNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, mask, groups, eps, length_last):
        x, gamma, beta = _c(x), _c(gamma), _c(beta)
        y = _require().cpu_sequence_norm_fwd(x, gamma, beta, mask, int(groups), float(eps), bool(length_last))
        ctx.save_for_backward(x, gamma)
        ctx.mask, ctx.meta = mask, (int(groups), float(eps), bool(length_last))
        return y

    @staticmethod
    def backward(ctx, gy):
        x, gamma = ctx.saved_tensors
        groups, eps, length_last = ctx.meta
        dx, dgamma, dbeta = _require().cpu_sequence_norm_bwd(gy.contiguous(), x, gamma, ctx.mask, groups, eps, length_last)
        return dx, dgamma, dbeta, None, None, None, None


class _EmaParameters(torch.autograd.Function):
    @staticmethod
    def forward(ctx, p, q, gamma, hx, length):
        p, q, gamma, hx = _c(p), _c(q), _c(gamma), _c(hx)
        k, b = _require().cpu_ema_parameters_fwd(p, q, gamma, hx, int(length))
        ctx.save_for_backward(p, q, gamma, *(() if hx is None else (hx,)))
        ctx.has_h = hx is not None
        if b is None:
            return k, None
        return k, b

    @staticmethod
    def backward(ctx, dk, db):
        saved = ctx.saved_tensors
        p, q, gamma = saved[:3]
        hx = saved[3] if ctx.has_h else None
        dk = torch.zeros(p.shape[0], 0) if dk is None else dk.contiguous()
        if ctx.has_h and db is not None:
            db = db.contiguous()
        else:
            db = None
        dp, dq, dgamma, dh = _require().cpu_ema_parameters_bwd(dk, db, p, q, gamma, hx if db is not None else None)
        if ctx.has_h and dh is None:
            dh = torch.zeros_like(hx)
        return dp, dq, dgamma, (dh if ctx.has_h else None), None


class _EmaHidden(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, q, hx):
        x, p, q, hx = _c(x), _c(p), _c(q), _c(hx)
        h = _require().cpu_ema_hidden_fwd(x, p, q, hx)
        ctx.save_for_backward(x, p, q, *(() if hx is None else (hx,)))
        ctx.has_h = hx is not None
        return h

    @staticmethod
    def backward(ctx, g):
        saved = ctx.saved_tensors
        x, p, q = saved[:3]
        hx = saved[3] if ctx.has_h else None
        dx, dp, dq, dh = _require().cpu_ema_hidden_bwd(g.contiguous(), x, p, q, hx)
        return dx, dp, dq, (dh if ctx.has_h else None)


class _Cema(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, q, gamma, omega, hx):
        x, p, q, gamma, omega, hx = (_c(t) for t in (x, p, q, gamma, omega, hx))
        y, h = _require().cpu_cema_fwd(x, p, q, gamma, omega, hx)
        ctx.save_for_backward(x, p, q, gamma, omega, *(() if hx is None else (hx,)))
        ctx.has_h = hx is not None
        ctx.shapes = (p.shape, q.shape, gamma.shape, omega.shape)
        return y, h

    @staticmethod
    def backward(ctx, dy, dh):
        saved = ctx.saved_tensors
        x, p, q, gamma, omega = saved[:5]
        hx = saved[5] if ctx.has_h else None
        dy = torch.zeros_like(x) if dy is None else dy.contiguous()
        dx, dp, dq, dg, dom, dhx = _require().cpu_cema_bwd(dy, None if dh is None else dh.contiguous(), x, p, q,
                                                          gamma, omega, hx)
        ps, qs, gs, os_ = ctx.shapes
        return dx, dp.reshape(ps), dq.reshape(qs), dg.reshape(gs), dom.reshape(os_), (dhx if ctx.has_h else None)


def cema(x, p, q, gamma, omega, hx, compute_last_state: bool):
    y, h = _Cema.apply(x, p, q, gamma, omega, hx)
    return y, (h if compute_last_state else None)


def timestep_norm(x, prev_count, prev_mean, prev_var, gamma, beta, mask, groups, eps, gamma_offset):
    return _TimestepNorm.apply(x, prev_count, prev_mean, prev_var, gamma, beta, mask, groups, eps, gamma_offset)


def sequence_norm(x, gamma, beta, mask, groups, eps, length_last):
    return _SequenceNorm.apply(x, gamma, beta, mask, groups, eps, length_last)


def ema_parameters(p, q, gamma, hx, length):
    return _EmaParameters.apply(p, q, gamma, hx, length)


def ema_hidden(x, p, q, hx):
    return _EmaHidden.apply(x, p, q, hx)
