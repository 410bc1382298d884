"""Plain-PyTorch statements of every operator in the framework.

These are (a) the CPU execution path, (b) the numerics oracle that the CUDA
kernels are tested against, and (c) differentiable by autograd, which gives an
independent check of the hand-derived backward passes.  Accumulation happens
in float64 where the reference's CPU code uses its "opmath" type, so the
oracle is at least as accurate as the reference's own
(csrc/ops/timestep_norm.cc:218-450, sequence_norm.cc:259-529,
ema_parameters.cc:17-117, ema_hidden.cc:15-159, fused_ops/fftconv.py:30-76).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

Tensor = torch.Tensor


# --------------------------------------------------------------------------- norms
def rms_norm(x: Tensor, weight: Optional[Tensor], eps: float, weight_offset: float = 0.0) -> Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * (weight + weight_offset) over the last
    dim; the scale is formed in fp32 (modules keep zero-centred weights and
    pass offset 1)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * (weight.float() + weight_offset)
    return y.to(x.dtype)


def layer_norm(x: Tensor, weight: Optional[Tensor], bias: Optional[Tensor], eps: float,
               weight_offset: float = 0.0) -> Tensor:
    y = F.layer_norm(x.float(), (x.shape[-1],),
                     None if weight is None else weight.float() + weight_offset,
                     None if bias is None else bias.float(), eps)
    return y.to(x.dtype)


def timestep_norm(
    x: Tensor, prev_count: Tensor, prev_mean: Tensor, prev_var: Tensor,
    gamma: Tensor, beta: Tensor, padding_mask: Optional[Tensor],
    num_groups: Optional[int], eps: float, gamma_offset: float = 0.0,
) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    """Cumulative (prefix) group normalisation over time.

    x [B, L, H]; statistics are kept per (batch, group).  At step t the group's
    H/G features give one sample (mean_t, var_t) of weight one, merged into the
    running population (count, mean, var).  The merge is associative, so the
    running values are written here in closed form with prefix sums of the
    first and second moments instead of a loop.  Padded steps output zero and
    leave the statistics untouched.  Returns (y, count, mean, var).
    """
    B, L, H = x.shape
    G = H if num_groups is None else num_groups
    D = H // G
    xd = x.double().view(B, L, G, D)
    gu = xd.mean(-1)
    gv = xd.var(-1, unbiased=False) if D > 1 else torch.zeros_like(gu)
    if padding_mask is None:
        valid = torch.ones(B, L, 1, dtype=torch.float64, device=x.device)
    else:
        valid = (~padding_mask).double().unsqueeze(-1)
    n0 = prev_count.double().view(B, 1, 1)
    u0 = prev_mean.double().view(B, 1, G)
    v0 = prev_var.double().view(B, 1, G)
    n = n0 + torch.cumsum(valid, dim=1)
    n_safe = n.clamp_min(1.0)
    s1 = n0 * u0 + torch.cumsum(gu * valid, dim=1)
    s2 = n0 * (v0 + u0 * u0) + torch.cumsum((gv + gu * gu) * valid, dim=1)
    mean = s1 / n_safe
    var = (s2 / n_safe - mean * mean).clamp_min(0.0)
    # with no history at all (count 0) the carried values are the state
    empty = n < 0.5
    mean = torch.where(empty, u0.expand_as(mean), mean)
    var = torch.where(empty, v0.expand_as(var), var)
    rstd = torch.rsqrt(var + eps)
    y = (xd - mean.unsqueeze(-1)) * rstd.unsqueeze(-1)
    y = y.view(B, L, H) * (gamma.double() + gamma_offset) + beta.double()
    y = y * valid
    count = prev_count + (valid.squeeze(-1).sum(1)).to(prev_count.dtype)
    return y.to(x.dtype), count, mean[:, -1].to(prev_mean.dtype), var[:, -1].to(prev_var.dtype)


def sequence_norm(
    x: Tensor, gamma: Tensor, beta: Tensor, padding_mask: Optional[Tensor],
    num_groups: Optional[int], eps: float, length_last: bool,
) -> Tensor:
    """Normalisation over the whole time axis (non-causal).  `x` is [B, L, H]
    (or [B, H, L] when `length_last`).  Ungrouped: statistics per (batch,
    feature) over the non-padded steps.  Grouped: per (batch, group) over the
    group's features times the non-padded steps."""
    if length_last:
        x = x.transpose(1, 2)
    B, L, H = x.shape
    xd = x.double()
    if padding_mask is None:
        valid = torch.ones(B, L, 1, dtype=torch.float64, device=x.device)
    else:
        valid = (~padding_mask).double().unsqueeze(-1)
    cnt = valid.sum(1, keepdim=True).clamp_min(1.0)           # B,1,1
    if num_groups is None:
        mean = (xd * valid).sum(1, keepdim=True) / cnt
        var = (((xd - mean) ** 2) * valid).sum(1, keepdim=True) / cnt
    else:
        G = num_groups
        D = H // G
        xg = xd.view(B, L, G, D)
        vg = valid.unsqueeze(-1)
        mean = (xg * vg).sum((1, 3), keepdim=True) / (cnt.unsqueeze(-1) * D)
        var = (((xg - mean) ** 2) * vg).sum((1, 3), keepdim=True) / (cnt.unsqueeze(-1) * D)
        mean = mean.expand(B, 1, G, D).reshape(B, 1, H)
        var = var.expand(B, 1, G, D).reshape(B, 1, H)
    y = (xd - mean) * torch.rsqrt(var + eps) * gamma.double() + beta.double()
    y = (y * valid).to(x.dtype)
    if length_last:
        y = y.transpose(1, 2)
    return y


# --------------------------------------------------------------------------- CEMA
def _powers(q: Tensor, start: int, length: int) -> Tensor:
    """q [D, N] complex -> q^(start + j) for j < length, shape [D, N, length]."""
    j = torch.arange(start, start + length, device=q.device, dtype=torch.float64)
    logq = torch.log(q.to(torch.complex128))
    return torch.exp(logq.unsqueeze(-1) * j)


def ema_parameters(p: Tensor, q: Tensor, gamma: Tensor, hx: Optional[Tensor], length: int):
    """CEMA convolution kernel k [D, L] and carried-state bias b [B, D, L].

    k[d, j] = Re sum_n p*gamma*q^j ;  b[b, d, j] = Re sum_n gamma*q^(j+1)*h.
    p [D, N] or [D, N, 1] real; q, gamma complex of the same shape."""
    p2 = p.reshape(p.shape[0], -1).double()
    q2 = q.reshape(p2.shape)
    g2 = gamma.reshape(p2.shape).to(torch.complex128)
    qp = _powers(q2, 0, length + 1)                                # D,N,L+1
    k = ((p2 * g2).unsqueeze(-1) * qp[..., :length]).sum(1).real   # D,L
    b = None
    if hx is not None:
        gh = g2.unsqueeze(0) * hx.to(torch.complex128)             # B,D,N
        b = torch.einsum("bdn,dnl->bdl", gh, qp[..., 1:]).real
        b = b.float()
    return k.float(), b


def ema_hidden(x: Tensor, p: Tensor, q: Tensor, hx: Optional[Tensor]) -> Tensor:
    """Last CEMA state: h' = p * sum_j q^(L-1-j) x_j + q^L h.  x [B, D, L]."""
    B, D, L = x.shape
    p2 = p.reshape(D, -1).double()
    q2 = q.reshape(p2.shape)
    qp = _powers(q2, 0, L + 1)                                     # D,N,L+1
    w = torch.flip(qp[..., :L], dims=(-1,)) * p2.unsqueeze(-1)     # q^(L-1-j) p
    h = torch.einsum("bdl,dnl->bdn", x.to(torch.complex128), w)
    if hx is not None:
        h = h + qp[..., L].unsqueeze(0) * hx.to(torch.complex128)
    return h.to(torch.complex64)


def fftconv(x: Tensor, k: Tensor) -> Tensor:
    """Causal long convolution along the last dim: y[t] = sum_{j<=t} k[j] x[t-j]."""
    L = x.shape[-1]
    n = 1 << max(L - 1, 1).bit_length() if L & (L - 1) else max(L, 1)
    xf = torch.fft.rfft(x.float(), n=2 * n)
    kf = torch.fft.rfft(k.float(), n=2 * n)
    y = torch.fft.irfft(xf * kf, n=2 * n)[..., :L]
    return y.to(x.dtype)


def rfft(x: Tensor, flip: bool = False) -> Tensor:
    """Real FFT of length 2N, N = max(32, next_pow2(L)) - the spectrum layout
    the reference's `rfft` op returns (csrc/ops/fftconv_kernel.cu:166-214)."""
    L = x.shape[-1]
    n = max(32, 1 << (L - 1).bit_length())
    xf = x.float()
    if flip:
        xf = torch.flip(xf, dims=(-1,))
    return torch.fft.rfft(xf, n=2 * n)


def cema(x: Tensor, p: Tensor, q: Tensor, gamma: Tensor, omega: Tensor,
         hx: Optional[Tensor], compute_last_state: bool):
    """Whole complex-EMA layer on channels-last input x [B, L, D]:
    y = conv(x, k) + b(h) + omega * x ; optionally the last state [B, D, N]."""
    xt = x.transpose(1, 2)
    L = xt.shape[-1]
    k, b = ema_parameters(p, q, gamma, hx, L)
    y = fftconv(xt, k)
    if b is not None:
        y = y + b.to(y.dtype)
    y = y + xt * omega.reshape(1, -1, 1).to(xt.dtype)
    h = ema_hidden(xt, p, q, hx) if compute_last_state else None
    return y.transpose(1, 2), h


def cema_scan(x: Tensor, p: Tensor, q: Tensor, gamma: Tensor, omega: Tensor,
              hx: Optional[Tensor]):
    """The same layer as an explicit recurrence (slow; used to cross-check the
    convolution form and the CUDA scan kernels): h_t = q h_{t-1} + p x_t,
    y_t = Re(sum_n gamma_n h_t,n) + omega x_t."""
    B, L, D = x.shape
    p2 = p.reshape(D, -1).double()
    q2 = q.reshape(p2.shape).to(torch.complex128)
    g2 = gamma.reshape(p2.shape).to(torch.complex128)
    h = torch.zeros(B, D, p2.shape[1], dtype=torch.complex128, device=x.device) if hx is None \
        else hx.to(torch.complex128)
    ys = []
    xd = x.double()
    for t in range(L):
        h = q2 * h + p2 * xd[:, t].unsqueeze(-1)
        ys.append((g2 * h).sum(-1).real)
    y = torch.stack(ys, 1) + xd * omega.reshape(1, 1, -1).double()
    return y.to(x.dtype), h.to(torch.complex64)


# --------------------------------------------------------------------------- attention
def attention_softmax(x: Tensor, dropout: float, use_causal_mask: bool, training: bool = True) -> Tensor:
    """Row softmax over the last dim of [..., L1, L2]; with a causal mask row r
    sees columns 0 .. L2-L1+r.  DropKey: keys are dropped *before* softmax."""
    L1, L2 = x.shape[-2:]
    s = x.float()
    if use_causal_mask:
        r = torch.arange(L1, device=x.device).unsqueeze(-1)
        c = torch.arange(L2, device=x.device).unsqueeze(0)
        s = s.masked_fill(c > r + (L2 - L1), float("-inf"))
    if training and dropout > 0:
        drop = torch.rand_like(s) < dropout
        s = s.masked_fill(drop, float("-inf"))
    w = torch.softmax(s, dim=-1)
    w = torch.nan_to_num(w, nan=0.0)        # fully masked rows give zeros
    return w.to(x.dtype)


def attention(q: Tensor, k: Tensor, v: Tensor, scale: float, dropout: float,
              use_causal_mask: bool, training: bool = True) -> Tensor:
    """q [B, L1, H, Dk], k [B, L2, H, Dk], v [B, L2, H, Dv] -> [B, L1, H, Dv]."""
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) * scale
    w = attention_softmax(s, dropout, use_causal_mask, training)
    return torch.einsum("bhqk,bkhd->bqhd", w.to(v.dtype), v)


def rotary(x: Tensor, freqs_cis: Tensor, conj: bool = False) -> Tensor:
    """Interleaved-pair RoPE in fp32.  x [B, L, H, D], freqs_cis [L, D/2] complex."""
    f = freqs_cis.conj() if conj else freqs_cis
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    out = torch.view_as_real(xc * f.unsqueeze(1)).flatten(-2)
    return out.to(x.dtype)


# --------------------------------------------------------------------------- misc
def linear(x: Tensor, w: Tensor, b: Optional[Tensor] = None, act: Optional[str] = None) -> Tensor:
    y = F.linear(x, w, b)
    if act == "silu":
        y = F.silu(y)
    elif act is not None:
        raise ValueError(act)
    return y


def swiglu(a: Tensor, b: Tensor) -> Tensor:
    return F.silu(a) * b


def cross_entropy(logits: Tensor, target: Tensor, weight=None, ignore_index: int = -100,
                  label_smoothing: float = 0.0) -> Tensor:
    return F.cross_entropy(logits.float(), target, reduction="none", weight=weight,
                           ignore_index=ignore_index, label_smoothing=label_smoothing)


def adamw_step(param: Tensor, grad: Tensor, m: Tensor, v: Tensor, *, lr: float, beta1: float,
               beta2: float, eps: float, weight_decay: float, step: int, grad_scale: float = 1.0,
               low: Optional[Tensor] = None) -> None:
    """Decoupled-weight-decay Adam on flat fp32 state; optionally refreshes the
    low-precision copy `low` used by the forward pass."""
    g = grad.float() * grad_scale
    param.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    param.addcdiv_(m, denom, value=-lr / bc1)
    if low is not None:
        low.copy_(param)
