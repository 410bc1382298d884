"""Tensor-parallel linears whose collective is fused into the GEMM.

* all-gather -> GEMM (`ag_linear`): the activation is sharded along its feature
  dim over the model-parallel group.  Every rank stages its shard in peer-mapped
  memory; the tcgen05 GEMM then walks K piece by piece, its TMA producer loading
  each piece straight from the owning GPU (starting with the local one), so the
  gather travels over NVLink while the tensor cores work on the previous tiles.
  Nothing is gathered into a full copy.
* GEMM -> reduce-scatter (`linear_rs`): each rank's partial product is stored by
  the GEMM epilogue directly into a slot in the memory of the rank that owns
  those output columns; after a flag barrier the owner sums its slots.

They replace the `gather_copy` + `F.linear` and `F.linear` + `reduce_scatter`
pairs of the Megatron-style layers (reference: modules/model_parallel/layers.py:224-232,
323-335 with mappings.py:145-170).  Weight gradients still gather the activation
with NCCL (the gathered operand is the MN-major one there).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .symm import AbortRecord, SymmetricRegion, _round_up

_WORKSPACE = [None]


def workspace():
    return _WORKSPACE[0]


class TensorParallelWorkspace:
    def __init__(self, group, device, max_tokens: int, part_features: int, dtype=torch.bfloat16,
                 timeout_s: float = 30.0):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.dtype = dtype
        esize = torch.empty(0, dtype=dtype).element_size()
        self.part_bytes = _round_up(max_tokens * part_features * esize, 256)
        self.max_elems = max_tokens * part_features
        # [2 stage buffers][2 x world slots][pads]
        self.stage_off = [0, self.part_bytes]
        self.slot_off = [2 * self.part_bytes, (2 + self.world) * self.part_bytes]
        self.pad_off = (2 + 2 * self.world) * self.part_bytes
        self.region = SymmetricRegion(self.pad_off + _round_up(4 * self.world, 256), group, device)
        self.timeout_ns = int(timeout_s * 1e9)
        self._abort = AbortRecord.get(device)
        self._pads = self.region.ptr_table_at(self.pad_off).contiguous()
        self.epoch = 0
        self._stage_toggle = 0
        self._slot_toggle = 0

    def _barrier(self) -> None:
        from ..ops._ext import require
        self.epoch += 1
        require().peer_barrier(self._pads, self.rank, self.epoch, self.timeout_ns, self._abort.dev, self.epoch)

    def check(self) -> None:
        self._abort.check()

    # y[M, N] = act([x_0 | x_1 | ...] w^T + bias), x_r = this rank's [M, K / world] shard
    def ag_gemm(self, x_part: torch.Tensor, w: torch.Tensor, bias=None, act=None, b_mn: bool = False,
                want_preact: bool = False):
        from ..ops import cuda_ops
        x_part = x_part.contiguous()
        assert x_part.numel() <= self.max_elems and x_part.dtype == self.dtype
        t = self._stage_toggle
        self._stage_toggle ^= 1
        stage = self.region.view(self.stage_off[t], x_part.numel() * x_part.element_size(), x_part.dtype)
        stage = stage.view(x_part.shape)
        stage.copy_(x_part)
        self._barrier()                                # every rank's shard is staged
        ptrs = [self.region.peer_ptr(r, self.stage_off[t]) for r in range(self.world)]
        return cuda_ops.gemm(stage, w, bias, act, b_mn=b_mn, want_preact=want_preact, a_part_ptrs=ptrs,
                             a_first=self.rank)

    # y_r[M, N / world] = sum over ranks of (x_p w_p^T)[:, r-th column block]
    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, b_mn: bool = False) -> torch.Tensor:
        from ..ops import cuda_ops
        from ..ops._ext import require
        x = x.contiguous()
        M = x.shape[0]
        N = w.shape[1] if b_mn else w.shape[0]
        cols = N // self.world
        assert M * cols <= self.max_elems and x.dtype == self.dtype
        t = self._slot_toggle
        self._slot_toggle ^= 1
        esize = x.element_size()
        # my partial for owner o goes to slot [my rank] in o's memory
        ptrs = [self.region.peer_ptr(o, self.slot_off[t] + self.rank * self.part_bytes) for o in range(self.world)]
        cuda_ops.gemm(x, w, b_mn=b_mn, c_part_ptrs=ptrs, out_dtype=x.dtype)
        self._barrier()                                # every rank has pushed its partials
        slots = self.region.view(self.slot_off[t], self.world * self.part_bytes, x.dtype)
        out = torch.empty(M, cols, dtype=x.dtype, device=x.device)
        if self.part_bytes == M * cols * esize:
            require().reduce_slots(slots, out, self.world)
        else:
            per = self.part_bytes // esize
            out.copy_(slots.view(self.world, per)[:, :M * cols].float().sum(0).view(M, cols))
        return out


def _all_gather_last(x: torch.Tensor, group) -> torch.Tensor:
    world = dist.get_world_size(group)
    parts = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(parts.view(-1), x.contiguous().view(-1), group=group)
    return parts.movedim(0, -2).reshape(*x.shape[:-1], world * x.shape[-1])


class AGLinear(torch.autograd.Function):
    """Column-parallel linear on a feature-sharded input: all-gather fused into the GEMM."""

    @staticmethod
    def forward(ctx, x_part, w, bias, act):
        from ..ops import cuda_ops
        ws = workspace()
        cuda_ops.ensure_gathered(w)
        x2 = x_part.reshape(-1, x_part.shape[-1])
        need_pre = act is not None and any(ctx.needs_input_grad[:3])
        y, pre = ws.ag_gemm(x2, w, bias, act, want_preact=need_pre)
        ctx.save_for_backward(x2, w, pre if pre is not None else torch.empty(0, device=x2.device))
        ctx.meta = (act, bias is not None, bias.dtype if bias is not None else None, x_part.shape)
        return y.view(*x_part.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from ..ops import cuda_ops
        ws = workspace()
        x2, w, pre = ctx.saved_tensors
        act, has_bias, bias_dtype, x_shape = ctx.meta
        g = dy.reshape(-1, dy.shape[-1]).contiguous()
        if act == "silu":
            g = cuda_ops.silu_bwd(g, pre)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = ws.gemm_rs(g, w, b_mn=True).view(x_shape)         # (g w) reduce-scattered over features
        if ctx.needs_input_grad[1]:
            x_full = _all_gather_last(x2, ws.group)
            dw, _ = cuda_ops.gemm(g, x_full, a_mn=True, b_mn=True)
        if has_bias and ctx.needs_input_grad[2]:
            db = g.sum(0, dtype=torch.float32).to(bias_dtype)
        return dx, dw, db, None


class LinearRS(torch.autograd.Function):
    """Row-parallel linear with feature-sharded output: reduce-scatter fused into the GEMM epilogue."""

    @staticmethod
    def forward(ctx, x, w):
        from ..ops import cuda_ops
        ws = workspace()
        cuda_ops.ensure_gathered(w)
        x2 = x.reshape(-1, x.shape[-1])
        y = ws.gemm_rs(x2, w)
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy_part):
        from ..ops import cuda_ops
        ws = workspace()
        x2, w = ctx.saved_tensors
        g_part = dy_part.reshape(-1, dy_part.shape[-1]).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx, _ = ws.ag_gemm(g_part, w, b_mn=True)                # [g_0 | g_1 | ...] w
            dx = dx.view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            g_full = _all_gather_last(g_part, ws.group)
            dw, _ = cuda_ops.gemm(g_full, x2, a_mn=True, b_mn=True)
        return dx, dw


def usable(x: torch.Tensor) -> bool:
    ws = workspace()
    # (a decode step's few rows take the plain layers: their collectives then go through the
    # graph-capturable small-collective kernel, and a 128-row tile would be nearly empty)
    return (ws is not None and x.is_cuda and x.dtype == ws.dtype and x.numel() // max(x.shape[-1], 1) > 16
            and x.numel() // x.shape[-1] * max(x.shape[-1], 1) <= ws.max_elems * ws.world)


def enable_tp_fused(model, max_tokens: int, timeout_s: float = 30.0) -> Optional[TensorParallelWorkspace]:
    """Route the model's tensor-parallel linears through the fused kernels.  Call on every rank of the
    model-parallel group after `build_model`; `max_tokens` bounds batch x local sequence per call."""
    from .initialize import get_model_parallel_group, get_model_parallel_world_size
    mp = get_model_parallel_world_size()
    if mp == 1:
        return None
    inner = model
    while hasattr(inner, "_wrapped"):
        inner = inner._wrapped
    device = next(model.parameters()).device
    ws = TensorParallelWorkspace(get_model_parallel_group(), device, max_tokens, inner.model_dim // mp,
                                 timeout_s=timeout_s)
    _WORKSPACE[0] = ws
    return ws


def disable_tp_fused() -> None:
    _WORKSPACE[0] = None
