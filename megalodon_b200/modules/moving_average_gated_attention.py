"""The MEGA layer: TimestepNorm -> CEMA -> RMSNorm -> gated chunk-local
attention with normalised shared q/k, plus the inner attention with its
chunk-tail KV cache (reference: megalodon/modules/moving_average_gated_attention.py).

    out_tsn = TimestepNorm(x)            v = SiLU(Wv out_tsn)     (v uses out_tsn)
    mx      = RMSNorm(CEMA(out_tsn))     r = SiLU(Wr mx)
    z       = RMSNorm_per_head(Wz mx);   q, k = z (gamma+1)/sqrt(d) + beta
    attn    = softmax_causal_per_chunk(rope(q) rope(k)^T) v       (scale 1)
    out     = Wh1 mx + Wh2 (attn * r) + x

Everything stays channels-last ([B, L, D]); the reference transposes to
[B, D, L] around the CEMA.  Under chunk parallelism the carried state
(TimestepNorm mean/var and the CEMA hidden state) is received from the
previous rank before TimestepNorm and sent to the next rank right after the
CEMA, packed as one fp32 row per sequence: [mean(G) | var(G) | Re/Im h (2 D N)].
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import Tensor, nn
from torch.nn import Parameter

from .. import ops
from ..parallel.initialize import get_chunk_parallel_rank, get_model_parallel_world_size
from ..parallel.utils import divide_and_check_no_remainder
from ..parallel.model_parallel import (
    ColumnParallelLinear,
    RowParallelLinear,
    gather_from_model_parallel_region,
)
from ..parallel.chunk_parallel import (
    attach_to_graph,
    recv_from_prev_chunk_parallel_region,
    send_to_next_chunk_parallel_region,
    should_recv_from_prev,
    should_send_to_next,
)
from ..utils import get_init_fn
from .complex_exponential_moving_average import MultiHeadComplexEMA
from .layer_norm import FusedRMSNorm
from .rotary_positional_embedding import apply_rotary_emb
from .timestep_norm import TimestepNorm

_c2r = torch.view_as_real
_r2c = torch.view_as_complex


class _InnerAttention(nn.Module):
    """Causal attention restricted to fixed-size chunks.  Sequences longer than
    a chunk are folded to [(B * n_chunks), chunk, H, d]; the KV cache only ever
    holds the tail of the current chunk and empties at a chunk boundary."""

    def __init__(self, z_head_dim: int, v_head_dim: int, n_heads: int, chunk_size: int,
                 dropout: float, efficient_attn: Optional[str]):
        super().__init__()
        self.z_head_dim = z_head_dim
        self.v_head_dim = v_head_dim
        self.n_heads = n_heads
        self.chunk_size = chunk_size
        self.dropout = dropout
        self.efficient_attn = efficient_attn

    def forward(self, xq: Tensor, xk: Tensor, xv: Tensor, mask: Optional[Tensor],
                freqs_cis: Optional[Tensor], cache: Optional[Tuple[Tensor, Tensor, int]] = None):
        bs, slen, _ = xq.shape
        c = self.chunk_size
        xq = xq.view(bs, slen, self.n_heads, self.z_head_dim)
        xk = xk.view(bs, slen, self.n_heads, self.z_head_dim)
        xv = xv.view(bs, slen, self.n_heads, self.v_head_dim)
        # freqs_cis None: the caller already rotated q and k (fused with their affine map)
        if slen <= c and freqs_cis is not None:
            xq, xk = apply_rotary_emb(xq, xk, freqs_cis, backward=False)

        if cache is not None and isinstance(cache[2], torch.Tensor):
            return self._static_step(xq, xk, xv, cache)

        new_cache = None
        clen = slen
        if cache is not None:
            cache_k, cache_v, count = cache
            if cache_k is not None and cache_k.size(1) > 0:
                xk = torch.cat([cache_k, xk], dim=1)
                xv = torch.cat([cache_v, xv], dim=1)
            clen = count + slen
            tail = clen % c
            new_cache = (xk.detach()[:, clen - tail:], xv.detach()[:, clen - tail:], tail)

        if c < slen:
            xq = xq.reshape(bs * (slen // c), c, self.n_heads, self.z_head_dim)
        if c < clen:
            xk = xk.reshape(bs * (clen // c), c, self.n_heads, self.z_head_dim)
            xv = xv.reshape(bs * (clen // c), c, self.n_heads, self.v_head_dim)
        if slen > c and freqs_cis is not None:
            xq, xk = apply_rotary_emb(xq, xk, freqs_cis, backward=False)

        if self.efficient_attn is None:
            # unfused path: post-softmax dropout, explicit additive mask
            assert mask is not None
            q, k, v = xq.transpose(1, 2), xk.transpose(1, 2), xv.transpose(1, 2)
            scores = torch.matmul(q, k.transpose(2, 3)) + mask
            scores = torch.softmax(scores.float(), dim=-1).to(q.dtype)
            scores = ops.memory_efficient_dropout(scores, self.dropout, self.training)
            out = torch.matmul(scores, v).transpose(1, 2).contiguous()
        else:
            causal = not (slen == 1 and cache is not None)
            out = ops.attention(xq, xk, xv, 1.0, self.dropout, causal, self.training)
        return out.reshape(bs, slen, -1), new_cache

    def _static_step(self, xq: Tensor, xk: Tensor, xv: Tensor, cache):
        """One decode step against fixed-size buffers: `cache = (k_buf, v_buf, pos)` with
        k_buf / v_buf [B, H, chunk, d] and `pos` a device index tensor [1] holding the position of
        this token inside its chunk.  Shapes never change and nothing is read back to the host, so
        the step can be captured in a CUDA graph; keys beyond `pos` (stale entries of the previous
        chunk) are masked, which is the same as the tail cache emptying at a chunk boundary.  The
        head-major layout makes both products plain batched matmuls over the buffers (no copies)."""
        k_buf, v_buf, pos = cache
        bs, slen = xq.shape[:2]
        assert slen == 1, "the static cache takes one token per step"
        k_buf.index_copy_(2, pos, xk.transpose(1, 2).to(k_buf.dtype))
        v_buf.index_copy_(2, pos, xv.transpose(1, 2).to(v_buf.dtype))
        if ops.decode_attention_native(xq, k_buf):
            # one kernel that attends over the filled slots only (keys 0 .. pos)
            out = ops.decode_attention(xq[:, 0], k_buf, v_buf, pos, 1.0)                 # [B, H, dv]
            return out.reshape(bs, 1, -1), cache
        scores = torch.matmul(xq.transpose(1, 2), k_buf.transpose(2, 3)).float()         # [B, H, 1, chunk]
        hidden = torch.arange(k_buf.size(2), device=pos.device) > pos
        probs = torch.softmax(scores.masked_fill(hidden, float("-inf")), dim=-1).to(xq.dtype)
        out = torch.matmul(probs, v_buf)                                                 # [B, H, 1, dv]
        return out.transpose(1, 2).reshape(bs, 1, -1), cache

    def extra_repr(self) -> str:
        return (f"heads={self.n_heads}, z_head_dim={self.z_head_dim}, "
                f"v_head_dim={self.v_head_dim}, chunk={self.chunk_size}")


class MovingAverageGatedAttention(nn.Module):
    def __init__(self, mdim: int, zdim: int, hdim: int, ndim: int, num_heads: int,
                 dropout: float = 0.0, attention_dropout: float = 0.0, hidden_dropout: float = 0.0,
                 chunk_size: int = 2048, efficient_attn: Optional[str] = None,
                 norm_num_groups: Optional[int] = None, norm_affine: bool = True,
                 norm_eps: float = 1e-5, init_mode: str = "he"):
        super().__init__()
        self.mdim, self.hdim, self.zdim, self.ndim = mdim, hdim, zdim, ndim
        self.num_heads = num_heads
        self.init_mode = init_mode
        assert zdim % num_heads == 0 and hdim % num_heads == 0
        self.z_head_dim = zdim // num_heads
        self.v_head_dim = hdim // num_heads
        world = get_model_parallel_world_size()
        # Heads are the unit of tensor parallelism (reference: moving_average_gated_attention.py:181).
        # With more ranks than heads (e.g. 8 ranks, 4 heads) one head is split over `head_split`
        # consecutive ranks along d_v: each of them projects that head's shared q/k (replicated
        # slice of wz, gamma, beta), its own slice of v and r, and attends with the full scores over
        # its d_v / head_split value columns; wh2 sums the partial outputs as usual.  The reference
        # cannot shard below one head per rank.  Inference only (see ColumnParallelLinear.partition).
        self.head_split = 1
        z_partition = None
        if world > num_heads:
            self.head_split = divide_and_check_no_remainder(world, num_heads)
            self.local_heads = 1
            from ..parallel.initialize import get_model_parallel_rank
            z_partition = (get_model_parallel_rank() // self.head_split, num_heads)
        else:
            self.local_heads = divide_and_check_no_remainder(num_heads, world)
        self.local_v_head_dim = divide_and_check_no_remainder(self.v_head_dim, self.head_split)
        self.local_mdim = divide_and_check_no_remainder(mdim, world)
        self.chunk_size = chunk_size
        self.efficient_attn = efficient_attn
        self.dropout = dropout
        self.attention_dropout = attention_dropout
        self.hidden_dropout = hidden_dropout

        self.timenorm = TimestepNorm(mdim, norm_num_groups, eps=norm_eps)
        self.cema = MultiHeadComplexEMA(mdim, ndim)
        self.rmsnorm = FusedRMSNorm(mdim, elementwise_affine=norm_affine, eps=norm_eps)
        self.znorm = FusedRMSNorm(self.z_head_dim, elementwise_affine=False, eps=norm_eps)

        init_fn = get_init_fn(init_mode)
        # v and r carry a SiLU that is fused into the GEMM epilogue
        self.wv = ColumnParallelLinear(mdim, hdim, bias=True, input_is_parallel=True,
                                       gather_output=False, init_method=init_fn, activation="silu")
        self.wz = ColumnParallelLinear(mdim, zdim, bias=True, input_is_parallel=False,
                                       gather_output=False, init_method=init_fn, partition=z_partition)
        self.wr = ColumnParallelLinear(mdim, hdim, bias=True, input_is_parallel=False,
                                       gather_output=False, init_method=init_fn, activation="silu")
        self.wh1 = ColumnParallelLinear(mdim, mdim, bias=True, input_is_parallel=False,
                                        gather_output=False, init_method=init_fn)
        self.wh2 = RowParallelLinear(hdim, mdim, bias=False, input_is_parallel=True,
                                     parallel_output=True, init_method=init_fn)
        self.inner_attention = _InnerAttention(self.z_head_dim, self.local_v_head_dim, self.local_heads,
                                               chunk_size, attention_dropout, efficient_attn)
        self.gamma = Parameter(torch.zeros(2, self.z_head_dim * self.local_heads))
        self.beta = Parameter(torch.zeros(2, self.z_head_dim * self.local_heads))

    # ---- chunk-parallel state packing: [mean(G) | var(G) | Re/Im h (2 D N)] fp32 ----
    def _empty_prev(self, x: Tensor, local_len: int):
        bsz = x.size(0)
        g = self.timenorm.groups_per_partition
        width = 2 * g + 2 * self.local_mdim * self.cema.ndim
        prev_count = torch.full((bsz,), local_len * get_chunk_parallel_rank(), dtype=torch.int64,
                                device=x.device)
        buf = torch.empty((bsz, width), dtype=torch.float32, device=x.device,
                          requires_grad=self.training and torch.is_grad_enabled())
        return prev_count, buf

    def _pack_prev_tensors(self, prev_mean: Tensor, prev_var: Tensor, hx: Tensor) -> Tensor:
        return torch.cat([prev_mean.float(), prev_var.float(), _c2r(hx).flatten(1)], dim=-1)

    def _unpack_prev_tensors(self, x: Tensor, packed: Tensor):
        g = self.timenorm.groups_per_partition
        d, n = self.local_mdim, self.cema.ndim
        mean, var, h = torch.split(packed, [g, g, 2 * d * n], dim=-1)
        return mean.to(x.dtype), var.to(x.dtype), _r2c(h.reshape(x.size(0), d, n, 2))

    def forward(self, x: Tensor, freqs_cis: Tensor, mask: Optional[Tensor] = None,
                cache: Optional[Tuple] = None, carry: Optional[Tuple] = None,
                piece: Optional[Tuple[int, int, int]] = None):
        """`cache`: inference state (detached).  `carry` / `piece`: sequence
        micro-batching in training - the local sequence is fed in `piece[1]`
        consecutive pieces (`piece = (index, count, local_len)`), and `carry =
        (count, mean, var, hx)` hands the differentiable running state from one
        piece to the next; only the first piece receives from the previous
        chunk-parallel rank and only the last one sends to the next."""
        bsz, seq_len, _ = x.shape
        residual = x
        streaming = piece is not None
        first_piece = piece is None or piece[0] == 0
        last_piece = piece is None or piece[0] == piece[1] - 1
        local_len = seq_len if piece is None else piece[2]
        # prefill: the last piece also returns the final (count, mean, var, h) of this rank
        emit = piece is not None and len(piece) > 3 and bool(piece[3])
        cache_attn = cache_norm = hx = None
        prev_count = prev_mean = prev_var = None
        if cache is not None:
            cache_attn, cache_norm, hx = cache
            prev_count, prev_mean, prev_var = cache_norm
        elif carry is not None:
            prev_count, prev_mean, prev_var, hx = carry
        elif first_piece and should_recv_from_prev():
            prev_count, buf = self._empty_prev(x, local_len)
            packed = recv_from_prev_chunk_parallel_region(buf)
            prev_mean, prev_var, hx = self._unpack_prev_tensors(x, packed)

        out_tsn, prev_count, prev_mean, prev_var = self.timenorm(x, prev_count, prev_mean, prev_var)
        send_now = cache is None and last_piece and should_send_to_next()
        need_state = cache_attn is not None or send_now or (streaming and not last_piece) or emit
        out_cema, hx = self.cema.forward_channels_last(out_tsn, hx, need_state)

        new_carry = None
        if cache is not None:
            cache_norm = (prev_count.detach(), prev_mean.detach(), prev_var.detach())
            hx = None if hx is None else hx.detach()
        elif send_now:
            packed = send_to_next_chunk_parallel_region(self._pack_prev_tensors(prev_mean, prev_var, hx))
            out_cema = attach_to_graph(out_cema, packed)
        elif streaming and not last_piece:
            new_carry = (prev_count, prev_mean, prev_var, hx)
        if emit and last_piece and cache is None:
            new_carry = (prev_count.detach(), prev_mean.detach(), prev_var.detach(), hx.detach())

        out_cema = gather_from_model_parallel_region(out_cema)
        mx = self.rmsnorm(out_cema)
        mx = ops.memory_efficient_dropout(mx, self.hidden_dropout, self.training)

        z = self.wz(mx).view(bsz, seq_len, self.local_heads, self.z_head_dim)
        z = self.znorm(z).view(bsz, seq_len, -1)
        # q, k = rotary(z (gamma + 1) / sqrt(d) + beta): one kernel; positions are those of the chunk
        q, k = ops.qk_rotary(z, self.gamma, self.beta, freqs_cis, self.z_head_dim)

        v = self.wv(out_tsn)          # SiLU fused
        r = self.wr(mx)               # SiLU fused

        attn, cache_attn = self.inner_attention(q, k, v, mask, None, cache_attn)
        attn = ops.memory_efficient_dropout(attn * r, self.hidden_dropout, self.training)

        if get_model_parallel_world_size() == 1 and not (self.training and self.dropout > 0.0):
            # both additions ride in the epilogues of the two projections
            h = ops.linear_add(mx, self.wh1.weight, self.wh1.bias, residual)
            out = ops.linear_add(attn, self.wh2.weight, None, h)
        else:
            h = self.wh1(mx) + self.wh2(attn)
            h = ops.memory_efficient_dropout(h, self.dropout, self.training)
            out = h + residual
        if cache is not None:
            return out, (cache_attn, cache_norm, hx)
        return out, new_carry

    def extra_repr(self) -> str:
        return (f"edim={self.mdim}, zdim={self.zdim}, hdim={self.hdim}, heads={self.num_heads}, "
                f"chunk={self.chunk_size}, eff_attn={self.efficient_attn}, init={self.init_mode}")
