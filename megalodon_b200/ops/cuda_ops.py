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
_GEMV_MAX_ROWS = 4          # up to this many rows a product runs on the weight-streaming CUDA-core kernel
_launches = [0]          # kernels launched by this framework (bench bookkeeping)


def count_launches() -> int:
    return _launches[0]


def _bump(n: int = 1) -> None:
    _launches[0] += n


def set_gemm_backend(name: str) -> None:
    """"tcgen05": this framework's kernel (CTA pairs, 256 x 256 tiles, for more than 128 rows);
    "tcgen05_1cta": the same kernel family restricted to single-CTA 128 x 256 tiles;
    "cublas": torch.matmul (baseline only)."""
    assert name in ("tcgen05", "tcgen05_1cta", "cublas")
    if name.startswith("tcgen05"):
        require().gemm_set_cta_pairs(name == "tcgen05")
        name = "tcgen05"
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


def _tma_ok(t: Tensor) -> bool:
    return (t.stride(-1) == 1 and t.stride(-2) % 8 == 0 and t.data_ptr() % 16 == 0
            and (t.dim() == 2 or t.stride(0) % 8 == 0))


def gemm(a: Tensor, b: Tensor, bias: Optional[Tensor] = None, act: Optional[str] = None, *,
         a_mn: bool = False, b_mn: bool = False, want_preact: bool = False,
         out_dtype: Optional[torch.dtype] = None, out: Optional[Tensor] = None, mode: int = 0,
         alpha: float = 1.0, a_part_ptrs=None, a_first: int = 0, c_part_ptrs=None, accumulate: bool = False,
         b_gather=None, softmax=None):
    """C = act(alpha * A B^T + bias), or with `accumulate` (needs `out`) C += alpha * A B^T + bias.
    `a_mn` / `b_mn`: operand is stored [K, rows].  `b_gather = (addresses of every rank's row block of
    B, this rank)`: B (a contiguous [N, K] matrix) is filled from those blocks by the kernel itself
    while it computes (FSDP all-gather fused into the consuming GEMM).  `softmax = dict(epi_kind=..,
    row_in=.., row_in2=.., row_out=.., aux=.., causal_off=..)`: one of the fused-softmax epilogues of the
    attention products (csrc/kernels.h, GemmSoftmaxSpec); native path only.
    Operands may be 2-D or 3-D (batched) strided views with a contiguous last
    dim.  `mode` 1..3 exploits causal structure (see gemm_sm100.cu).  Returns
    (C, preact | None)."""
    out_dtype = out_dtype or (out.dtype if out is not None else a.dtype)
    native = (_GEMM_BACKEND[0] == "tcgen05" and a.dtype in (torch.bfloat16, torch.float16)
              and _tma_ok(a) and _tma_ok(b) and (out is None or _tma_ok(out))
              and (b.shape[-1] if b_mn else b.shape[-2]) % 8 == 0)
    if a_part_ptrs or c_part_ptrs or b_gather:
        if not native:
            raise RuntimeError("peer-memory GEMM needs the tcgen05 backend and TMA-compatible operands")
        _bump()
        res, pre, rc = _C().gemm(a, b, out, bias, 1 if act == "silu" else 0, a_mn, b_mn, want_preact,
                                 _DT[out_dtype], mode, alpha, _err_flag(a.device),
                                 a_part_ptrs=list(a_part_ptrs or []), a_first=a_first,
                                 c_part_ptrs=list(c_part_ptrs or []),
                                 b_gather_ptrs=list(b_gather[0]) if b_gather else [],
                                 b_gather_rank=int(b_gather[1]) if b_gather else 0, **(softmax or {}))
        if rc != 0:
            raise RuntimeError(f"tcgen05 GEMM launch failed with code {rc}")
        return res, pre
    if softmax and not native:
        raise RuntimeError("fused-softmax epilogues need the tcgen05 backend and TMA-compatible operands")
    if not native:
        A = a.transpose(-1, -2) if a_mn else a
        Bm = b if b_mn else b.transpose(-1, -2)
        pre = torch.matmul(A, Bm)
        if alpha != 1.0:
            pre = pre * alpha
        if bias is not None:
            pre = pre + bias.to(pre.dtype)
        res = F.silu(pre) if act == "silu" else pre
        if mode == 1:       # the kernel leaves tiles above the diagonal unwritten; nothing reads them
            pass
        if out is not None:
            if accumulate:
                out.add_(res.to(out.dtype))
            else:
                out.copy_(res)
            res = out
        return res.to(out_dtype), (pre.to(out_dtype) if want_preact else None)
    if (a.dim() == 2 and a.shape[0] <= _GEMV_MAX_ROWS and not a_mn and not b_mn and mode == 0 and out is None
            and not want_preact and not accumulate and not softmax):
        # a few rows (decoding): one pass over the weights on the CUDA cores beats a 128-row MMA tile; its
        # time grows with the rows (7B decode: 6.3 / 12.7 / 42 ms per token at 1 / 4 / 16 rows), the MMA
        # tile's does not, and from about five rows the tile wins
        _bump()
        res = _C().gemv_small_m(a, b, bias, 1 if act == "silu" else 0, _DT[out_dtype], alpha)
        if res is not None:
            return res, None
    _bump()
    res, pre, rc = _C().gemm(a, b, out, bias, 1 if act == "silu" else 0, a_mn, b_mn, want_preact,
                             _DT[out_dtype], mode, alpha, _err_flag(a.device),
                             accumulate=bool(accumulate and out is not None), **(softmax or {}))
    if rc != 0:
        raise RuntimeError(f"tcgen05 GEMM launch failed with code {rc}")
    return res, pre


def _gemm_gathering(x2: Tensor, w: Tensor, b, act, **kw):
    """`gemm(x2, w, ...)` for a linear layer's forward.  A sharded weight seen for the first time since the
    last optimiser step (`_gather_spec` pending) is gathered by this GEMM itself where the kernel can,
    by a stand-alone pull otherwise."""
    spec = getattr(w, "_gather_spec", None)
    if spec is not None and spec.pending:
        if (_GEMM_BACKEND[0] == "tcgen05" and w.is_contiguous() and _tma_ok(x2)
                and _C().gemm_gather_supported(x2.shape[0], w.shape[0], w.shape[1], len(spec.sources()[0]))):
            out = gemm(x2, w, b, act, b_gather=spec.sources(), **kw)
            spec.done()
            return out
        spec.pull_now()
    return gemm(x2, w, b, act, **kw)


class _LinearAdd(torch.autograd.Function):
    """y = x w^T + b + addend, the addition done in the GEMM epilogue (residual adds and the sum of two
    projections cost no kernel of their own).  Gradients as for `_Linear`; the addend's is dy itself."""

    @staticmethod
    def forward(ctx, x, w, b, addend):
        x2 = x.reshape(-1, x.shape[-1])
        a2 = addend.reshape(-1, addend.shape[-1])
        if not a2.is_contiguous():
            a2 = a2.contiguous()
        y, _ = _gemm_gathering(x2, w, b, None, softmax=dict(aux=a2), out=torch.empty_like(a2))
        ctx.save_for_backward(x2, w)
        ctx.wgrad_sink = getattr(w, "_wgrad_sink", None)
        ctx.has_bias = b is not None
        ctx.x_shape = x.shape
        ctx.bias_dtype = b.dtype if b is not None else None
        return y.view(addend.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        g = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx, _ = gemm(g, w, None, None, b_mn=True)
            dx = dx.view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            sink = ctx.wgrad_sink
            if sink is not None and w.dtype == g.dtype:
                target, add = sink()
                gemm(g, x2, None, None, a_mn=True, b_mn=True, out=target, accumulate=add)
            else:
                dw, _ = gemm(g, x2, None, None, a_mn=True, b_mn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _bias_grad(g).to(ctx.bias_dtype)
        return dx, dw, db, (dy if ctx.needs_input_grad[3] else None)


def _bias_grad(g: Tensor) -> Tensor:
    """fp32 column sums of the output gradient [rows, features]."""
    if g.is_cuda and g.dtype in (torch.bfloat16, torch.float16) and g.dim() == 2 and g.is_contiguous():
        _bump()
        return _C().colsum(g)
    return g.sum(0, dtype=torch.float32)


def linear_add(x: Tensor, w: Tensor, b: Optional[Tensor], addend: Tensor) -> Tensor:
    """x w^T + b + addend; `addend` has the shape of the result."""
    rows = x.numel() // x.shape[-1]
    if (x.dtype == torch.float32 or _GEMM_BACKEND[0] != "tcgen05" or addend.dtype != x.dtype
            or w.shape[0] % 8 != 0 or rows <= _GEMV_MAX_ROWS or not _tma_ok(x.reshape(-1, x.shape[-1]))):
        # (a few rows - decoding - stay on the weight-streaming kernel behind `linear`)
        return linear(x, w, b) + addend
    return _LinearAdd.apply(x, w, b, addend)


def ensure_gathered(w: Tensor) -> Tensor:
    """A weight whose all-gather was left to its first consuming GEMM (`_gather_spec`) but is about to
    be read by something else: gather it now."""
    spec = getattr(w, "_gather_spec", None)
    if spec is not None and spec.pending:
        spec.pull_now()
    return w


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, act):
        x2 = x.reshape(-1, x.shape[-1])
        need_pre = act is not None and any(ctx.needs_input_grad[:3])
        y, pre = _gemm_gathering(x2, w, b, act, want_preact=need_pre)
        ctx.save_for_backward(x2, w, pre if pre is not None else torch.empty(0, device=x.device))
        ctx.wgrad_sink = getattr(w, "_wgrad_sink", None)
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
            # A weight that is a view into an FSDP unit's flat buffer carries the matching view of the
            # unit's flat gradient: the weight gradient is accumulated there by the GEMM epilogue and
            # nothing is handed to autograd (no per-parameter tensor, no concatenation, no add).
            sink = ctx.wgrad_sink
            if sink is not None and w.dtype == g.dtype:
                target, add = sink()        # first product of the iteration writes, later ones accumulate
                gemm(g, x2, None, None, a_mn=True, b_mn=True, out=target, accumulate=add)
            else:
                dw, _ = gemm(g, x2, None, None, a_mn=True, b_mn=True)   # [M, N]^T x [M, K] -> [N, K]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _bias_grad(g).to(ctx.bias_dtype)
        return dx, dw, db, None


def linear(x: Tensor, w: Tensor, b: Optional[Tensor] = None, act: Optional[str] = None) -> Tensor:
    if x.dtype == torch.float32:
        return reference.linear(x, w, b, act)
    return _Linear.apply(x, w, b, act)


def silu_bwd(g: Tensor, pre: Tensor) -> Tensor:
    """g * silu'(pre): two reads and one write."""
    _bump()
    return _C().silu_bwd(g.contiguous(), pre.contiguous())


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


class _SequenceNorm(torch.autograd.Function):
    """Two bandwidth-bound kernels per direction (time sums, affine apply); the [B, H]-sized
    statistics in between are combined here with a handful of tiny tensor ops."""

    @staticmethod
    def forward(ctx, x, gamma, beta, mask, groups, eps, length_last):
        xc = x.contiguous()
        B = xc.shape[0]
        L = xc.shape[2] if length_last else xc.shape[1]
        H = xc.shape[1] if length_last else xc.shape[2]
        mk = None if mask is None else mask.contiguous()
        _bump(2)
        s1, s2 = _C().time_sums(xc, None, mk, length_last)
        count = torch.full((B, 1), float(L), device=x.device) if mk is None else \
            (~mk).sum(1, keepdim=True).float().clamp_min(1.0)
        g32, b32 = gamma.float(), beta.float()
        if groups is None:
            n = count
            mean = s1 / n
            var = (s2 / n - mean * mean).clamp_min(0.0)
        else:
            D = H // groups
            n = count * D
            mean = (s1.view(B, groups, D).sum(-1) / n)
            var = (s2.view(B, groups, D).sum(-1) / n - mean * mean).clamp_min(0.0)
            mean = mean.repeat_interleave(D, dim=1)
            var = var.repeat_interleave(D, dim=1)
        rstd = torch.rsqrt(var + eps)
        A = (rstd * g32).contiguous()
        y = _C().affine_apply(xc, None, A, None, (b32 - mean * A).contiguous(), mk, length_last)
        ctx.save_for_backward(xc, mean, rstd, g32, mk if mk is not None else torch.empty(0, device=x.device), n)
        ctx.meta = (groups, length_last, mk is not None, gamma.dtype, beta.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, mean, rstd, g32, mk, n = ctx.saved_tensors
        groups, length_last, has_mask, gdt, bdt = ctx.meta
        mk = mk if has_mask else None
        dyc = dy.contiguous()
        B, H = mean.shape
        _bump(2)
        db, ds = _C().time_sums(dyc, xc, mk, length_last)          # sum dy, sum dy * x   [B, H]
        c = 1.0 / n
        if groups is None:
            dv = 0.5 * rstd ** 3 * g32 * (mean * db - ds)
            du = -rstd * g32 * db
        else:
            D = H // groups
            dsg = (ds * g32).view(B, groups, D).sum(-1).repeat_interleave(D, dim=1)
            dbg = (db * g32).view(B, groups, D).sum(-1).repeat_interleave(D, dim=1)
            dv = 0.5 * rstd ** 3 * (mean * dbg - dsg)
            du = -rstd * dbg
        A = (rstd * g32).contiguous()
        Bc = (2.0 * c * dv).contiguous()
        Cc = (c * du - Bc * mean).contiguous()
        dx = _C().affine_apply(dyc, xc, A, Bc, Cc, mk, length_last)
        dgamma = (rstd * (ds - mean * db)).sum(0).to(gdt)
        dbeta = db.sum(0).to(bdt)
        return dx, dgamma, dbeta, None, None, None, None


def sequence_norm(x, gamma, beta, padding_mask, num_groups, eps, length_last):
    return _SequenceNorm.apply(x, gamma, beta, padding_mask, num_groups, eps, length_last)


class _Dropout(torch.autograd.Function):
    """Philox mask regenerated in backward from (seed, offset); nothing is stored."""

    @staticmethod
    def forward(ctx, x, p):
        # the offset comes from the CPU generator, whose state activation checkpointing restores,
        # so a recomputed forward draws the same mask
        ctx.key = (torch.initial_seed() & ((1 << 62) - 1), int(torch.randint(0, 2 ** 62, (1,)).item()))
        ctx.p = p
        _bump()
        return _C().dropout(x.contiguous(), p, *ctx.key)

    @staticmethod
    def backward(ctx, g):
        _bump()
        return _C().dropout(g.contiguous(), ctx.p, *ctx.key), None


def dropout(x, p):
    return _Dropout.apply(x, float(p))


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


class _EMAParameters(torch.autograd.Function):
    @staticmethod
    def forward(ctx, p, q, gamma, hx, length):
        D = p.shape[0]
        p2 = p.reshape(D, -1).float().contiguous()
        N = p2.shape[1]
        logq = _c2r(q.reshape(D, N).log())
        g2 = _c2r(gamma.reshape(D, N))
        h2 = None if hx is None else _c2r(hx)
        _bump(1 if hx is None else 2)
        k, b = _C().ema_parameters_fwd(p2, logq, g2, h2, length)
        ctx.save_for_backward(p2, logq, g2, h2 if h2 is not None else torch.empty(0, device=p.device))
        ctx.meta = (p.shape, q.shape, gamma.shape, hx is not None, length, p.dtype)
        return k, b

    @staticmethod
    def backward(ctx, dk, db):
        p2, logq, g2, h2 = ctx.saved_tensors
        ps, qs, gs, has_h, length, pdt = ctx.meta
        _bump()
        dp, dq, dg, dh = _C().ema_parameters_bwd(None if dk is None else dk.float().contiguous(),
                                                 None if db is None else db.float().contiguous(), p2, logq, g2,
                                                 h2 if has_h else None, length)
        return (dp.view(ps).to(pdt), torch.view_as_complex(dq).view(qs), torch.view_as_complex(dg).view(gs),
                torch.view_as_complex(dh) if has_h else None, None)


def ema_parameters(p, q, gamma, hx, length):
    return _EMAParameters.apply(p, q, gamma, hx, length)


def ema_hidden(x, p, q, hx):
    """Last CEMA state of x [B, D, L]: the fused scan run with gamma = omega = 0."""
    D = x.shape[1]
    N = p.reshape(D, -1).shape[1]
    if N not in (1, 2, 4, 8, 16, 32):
        return reference.ema_hidden(x, p, q, hx)
    zg = torch.zeros(D, N, dtype=torch.complex64, device=x.device)
    zo = torch.zeros(D, device=x.device)
    _, h = _CEMA.apply(x.transpose(1, 2), p, q, zg, zo, hx, True)
    return h


class _FFTConv(torch.autograd.Function):
    """Causal long convolution x [B, D, L] * k [D, L] through the shared-memory FFT kernels.  The
    input spectrum is not kept: the backward pass recomputes it inside the kernels that need it."""

    @staticmethod
    def forward(ctx, x, k):
        xc = x.contiguous()
        kf = _C().rfft_rows(k.float().contiguous(), False)          # [D, bins, 2]
        _bump(2)
        y = _C().fftconv_apply(xc, kf, False)
        ctx.save_for_backward(xc, kf)
        ctx.k_dtype = k.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, kf = ctx.saved_tensors
        dyc = dy.contiguous()
        dx = dk = None
        if ctx.needs_input_grad[0]:
            _bump()
            dx = _C().fftconv_apply(dyc, kf, True)
        if ctx.needs_input_grad[1]:
            L = xc.shape[-1]
            if L <= 8192:
                _bump(2)
                dk = _C().fftconv_dk(dyc, xc).to(ctx.k_dtype)
            else:
                # rows too long for one full-size transform in shared memory: two packed transforms per
                # row, the product summed over the batch, one packed inverse per feature
                _bump(3)
                gy = torch.view_as_complex(_C().rfft_rows(dyc, False))
                xs = torch.view_as_complex(_C().rfft_rows(xc, False))
                acc = torch.view_as_real((gy * xs.conj()).sum(0)).contiguous()
                dk = _C().irfft_rows(acc, L).to(ctx.k_dtype)
        return dx, dk


def _fft_native_ok(x, L) -> bool:
    return x.is_cuda and x.dtype in (torch.float32, torch.bfloat16, torch.float16) and 1 <= L <= 16384


def fftconv(x, k):
    """x [B, D, L] (or [D, L]), k [D, L] -> causal convolution along L."""
    if not _fft_native_ok(x, x.shape[-1]) or x.dim() not in (2, 3) or k.dim() != 2:
        return reference.fftconv(x, k)
    x3 = x if x.dim() == 3 else x.unsqueeze(0)
    y = _FFTConv.apply(x3, k)
    return y if x.dim() == 3 else y.squeeze(0)


def rfft(x, flip=False):
    """Real FFT of the zero-padded rows (length 2 * max(32, next_pow2(L))) as a complex tensor."""
    if not _fft_native_ok(x, x.shape[-1]) or x.requires_grad:
        return reference.rfft(x, flip)
    _bump()
    return torch.view_as_complex(_C().rfft_rows(x.contiguous(), bool(flip)))


# ----------------------------------------------------------------------------- attention
# Chunk-local attention as five tensor-core products around an in-place softmax:
#   S = scale Q K^T -> P = softmax_causal(S) -> O = P V
#   dV = P^T dO,  dP = dO V^T,  dS = P (dP - rowsum(P dP)),  dQ = scale dS K,  dK = scale dS^T Q
# All products run on the tcgen05 GEMM, batched over heads through strided 3-D
# views of the [B, L, H, d] tensors (no per-head copies) and, for square causal
# blocks, restricted to the tiles on or below the diagonal.
def _heads_view(t: Tensor, b: int) -> Tensor:
    """[B, L, H, d] -> view [H, L, d] of batch element b (strides d, H*d, 1)."""
    return t[b].permute(1, 0, 2)


def _attention_native_ok(q, k, v) -> bool:
    return (q.dtype in (torch.bfloat16, torch.float16) and q.shape[-1] % 8 == 0 and v.shape[-1] % 8 == 0
            and k.shape[1] <= 8192 and _GEMM_BACKEND[0] == "tcgen05")


class _Attention(torch.autograd.Function):
    """Chunk-local attention as matrix products on the tcgen05 GEMM (batched over heads).

    Without DropKey and with square causal (or unmasked) scores the softmax lives in the GEMM
    epilogues: Q K^T runs twice - the first pass keeps only the row maxima, the second writes
    exp(s - max) in the activation dtype and accumulates the row sums - so the logits are never
    rounded to 16 bits or written out in fp32, and P V divides by the row sum in its epilogue.
    Backward: dV = P^T dO', dS comes out of the epilogue of dO V^T, then dQ and dK.  What is kept for
    backward is the un-normalised P (16-bit), the row sums and the output.  With DropKey (or a key
    cache longer than the query block) the scores go through the stand-alone softmax kernels."""

    @staticmethod
    def forward(ctx, q, k, v, scale, drop_p, causal):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        B, L1, H, dk = q.shape
        L2, dv = k.shape[1], v.shape[-1]
        square = causal and L1 == L2
        # (key counts that are not a multiple of 8 leave the tensor-core path, see `gemm`)
        fused = drop_p == 0.0 and (square or not causal) and _FUSED_SOFTMAX[0] and L2 % 8 == 0
        ld = -(-L2 // 128) * 128                     # padded row length of the score buffer
        P = torch.empty(B, H, L1, ld, dtype=q.dtype, device=q.device)
        out = torch.empty(B, L1, H, dv, dtype=q.dtype, device=q.device)
        mode_s, mode_o = (1, 2) if square else (0, 0)
        if fused:
            rmax = torch.full((B, H, L1), float("-inf"), dtype=torch.float32, device=q.device)
            rsum = torch.zeros((B, H, L1), dtype=torch.float32, device=q.device)
            for b in range(B):
                Pb, qb, kb = P[b][:, :, :L2], _heads_view(q, b), _heads_view(k, b)
                gemm(qb, kb, out=Pb, mode=mode_s, alpha=scale, softmax=dict(epi_kind=1, row_out=rmax[b]))
                gemm(qb, kb, out=Pb, mode=mode_s, alpha=scale,
                     softmax=dict(epi_kind=2, row_in=rmax[b], row_out=rsum[b]))
                gemm(Pb, _heads_view(v, b), b_mn=True, out=_heads_view(out, b), mode=mode_o,
                     softmax=dict(epi_kind=3, row_in=rsum[b]))
            if _RECOMPUTE_SCORES[0]:
                # keep the row maxima (16 KB per head) instead of the 32 MB of P~ per head: backward runs
                # the second score pass again
                ctx.save_for_backward(q, k, v, rmax, rsum, out)
                ctx.scores_kept = False
            else:
                ctx.save_for_backward(q, k, v, P, rsum, out)
                ctx.scores_kept = True
        else:
            seed = offset = 0
            if drop_p > 0.0:
                seed = int(torch.randint(0, 2 ** 62, (1,)).item())
            for b in range(B):
                Pb = P[b][:, :, :L2]
                gemm(_heads_view(q, b), _heads_view(k, b), out=Pb, mode=mode_s, alpha=scale)
                _bump()
                _C().attn_softmax_fwd(Pb, L1, L2, causal, drop_p, seed, offset + b)
                gemm(Pb, _heads_view(v, b), b_mn=True, out=_heads_view(out, b), mode=mode_o)
            ctx.save_for_backward(q, k, v, P)
        ctx.meta = (scale, causal, square, L2, fused)
        return out

    @staticmethod
    def backward(ctx, dout):
        scale, causal, square, L2, fused = ctx.meta
        if fused:
            q, k, v, P, rsum, out = ctx.saved_tensors
            if not ctx.scores_kept:
                rmax, (Bq, Lq, Hq, _) = P, q.shape
                ld = -(-L2 // 128) * 128
                P = torch.empty(Bq, Hq, Lq, ld, dtype=q.dtype, device=q.device)
                scratch = torch.empty_like(rsum)
                for b in range(Bq):
                    gemm(_heads_view(q, b), _heads_view(k, b), out=P[b][:, :, :L2], mode=1 if square else 0,
                         alpha=scale, softmax=dict(epi_kind=2, row_in=rmax[b], row_out=scratch[b]))
        else:
            q, k, v, P = ctx.saved_tensors
        dout = dout.contiguous()
        B, L1, H, dk = q.shape
        dq, dk_, dv_ = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        m1, m2, m3 = (1, 2, 3) if square else (0, 0, 0)
        if fused:
            # delta_i = dO_i . O_i (what sum_j P_ij dP_ij equals) and dO' = dO / rowsum, in one pass
            _bump()
            dos, delta = _C().attn_bwd_prep(dout, out, rsum)                                      # delta [B, H, L1]
        else:
            dP = torch.empty_like(P[0])
        for b in range(B):
            Pb = P[b][:, :, :L2]
            if fused:
                # dV = P~^T (dO / l); dS = P~ / l * (dO V^T - delta) written over P~; dQ, dK from dS
                gemm(Pb, _heads_view(dos, b), a_mn=True, b_mn=True, out=_heads_view(dv_, b), mode=m3)
                gemm(_heads_view(dout, b), _heads_view(v, b), out=Pb, mode=m1,
                     softmax=dict(epi_kind=4, row_in=rsum[b], row_in2=delta[b], aux=Pb))
                dSb = Pb
            else:
                dPb = dP[:, :, :L2]
                dOb = _heads_view(dout, b)
                # dV = P^T dO   (A = P stored [q, key] = [K, M]; B = dO stored [q, dv] = [K, N])
                gemm(Pb, dOb, a_mn=True, b_mn=True, out=_heads_view(dv_, b), mode=m3)
                # dP = dO V^T
                gemm(dOb, _heads_view(v, b), out=dPb, mode=m1)
                _bump()
                _C().attn_softmax_bwd(Pb, dPb, L1, L2, causal)      # dP <- dS in place
                dSb = dPb
            # dQ = scale dS K ; dK = scale dS^T Q
            gemm(dSb, _heads_view(k, b), b_mn=True, out=_heads_view(dq, b), mode=m2, alpha=scale)
            gemm(dSb, _heads_view(q, b), a_mn=True, b_mn=True, out=_heads_view(dk_, b), mode=m3, alpha=scale)
        return dq, dk_, dv_, None, None, None


def decode_attention(q, k_buf, v_buf, pos, scale):
    _bump()
    return _C().decode_attention(q.contiguous(), k_buf, v_buf.contiguous(), pos, float(scale))


_FUSED_SOFTMAX = [True]
_RECOMPUTE_SCORES = [False]


def set_attention_recompute_scores(on: bool) -> None:
    """Fused-softmax attention keeps the un-normalised probabilities for backward (default) or only the
    row maxima and recomputes the probabilities there (one more pass of the Q K^T product per backward;
    128 MB less kept per layer and 4096-token chunk of the 7B model)."""
    _RECOMPUTE_SCORES[0] = bool(on)


def set_fused_attention_softmax(on: bool) -> None:
    """Softmax inside the epilogues of the attention products (default) or the stand-alone kernels."""
    _FUSED_SOFTMAX[0] = bool(on)


def attention(q, k, v, scale, dropout, use_causal_mask, training):
    if not _attention_native_ok(q, k, v):
        return reference.attention(q, k, v, scale, dropout, use_causal_mask, training)
    return _Attention.apply(q, k, v, float(scale), float(dropout) if training else 0.0, bool(use_causal_mask))


class _AttentionSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, drop_p, causal):
        L1, L2 = x.shape[-2:]
        y = x.contiguous().clone()
        seed = int(torch.randint(0, 2 ** 62, (1,)).item()) if drop_p > 0.0 else 0
        _bump()
        _C().attn_softmax_fwd(y, L1, L2, causal, drop_p, seed, 0)
        ctx.save_for_backward(y)
        ctx.causal = causal
        return y

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        L1, L2 = y.shape[-2:]
        dx = g.contiguous().clone()
        _bump()
        _C().attn_softmax_bwd(y, dx, L1, L2, ctx.causal)
        if ctx.causal:       # columns the kernel does not visit carry the incoming gradient: clear them
            r = torch.arange(L1, device=y.device).unsqueeze(-1)
            c = torch.arange(L2, device=y.device).unsqueeze(0)
            dx = dx.masked_fill(c > r + (L2 - L1), 0)
        return dx, None, None


def attention_softmax(x, dropout, use_causal_mask, training):
    if x.shape[-1] > 8192:
        return reference.attention_softmax(x, dropout, use_causal_mask, training)
    return _AttentionSoftmax.apply(x, float(dropout) if training else 0.0, bool(use_causal_mask))


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


class _QKRotary(torch.autograd.Function):
    """q, k = rotary(z (gamma + 1) / sqrt(d) + beta) for the two rows of gamma / beta, one kernel each way
    (replaces two broadcast multiply-adds, two strided copies and two rotary launches, and in backward
    their gradients and four column reductions)."""

    @staticmethod
    def forward(ctx, z, gamma, beta, freqs, head_dim):
        zc = z.contiguous()
        gc, bc = gamma.contiguous(), beta.contiguous()
        _bump()
        q, k = _C().qk_rotary_fwd(zc, gc, bc, freqs, head_dim)
        ctx.save_for_backward(zc, gc, freqs)
        ctx.meta = (head_dim, gamma.dtype, beta.dtype)
        return q, k

    @staticmethod
    def backward(ctx, dq, dk):
        zc, gc, freqs = ctx.saved_tensors
        head_dim, gdt, bdt = ctx.meta
        _bump(2)
        dz, dgamma, dbeta = _C().qk_rotary_bwd(dq.contiguous(), dk.contiguous(), zc, gc, freqs, head_dim)
        return dz, dgamma.to(gdt), dbeta.to(bdt), None, None


def qk_rotary(z, gamma, beta, freqs_cis, head_dim: int):
    """z [B, L, S] normalised per head; gamma, beta [2, S]; freqs_cis [P, head_dim / 2] complex with the
    position of (b, l) being (b L + l) % P.  Returns rotated q, k [B, L, S]."""
    freqs = torch.view_as_real(freqs_cis.to(torch.complex64).contiguous())
    return _QKRotary.apply(z, gamma, beta, freqs, int(head_dim))


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
