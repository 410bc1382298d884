"""AdamW on the FSDP flat shards.

`build_optimizer` keeps the reference's signature and return value
(megalodon/optim/optimizer.py:24-36) but returns `FusedAdamW`: one kernel per
flat shard reads the reduced gradient shard in whatever dtype the
reduce-scatter produced (bf16 or fp32), applies clipping scale, decoupled
weight decay and the Adam update to the fp32 master shard, and writes the
compute-dtype copy that the next forward's all-gather reads - one pass over
memory instead of cast + AdamW + cast.  It also accepts ordinary parameters
with `.grad` (then it is a plain AdamW).
"""
from __future__ import annotations

import functools
import logging
from typing import Iterable

import torch
from torch import nn
from torch.optim import Optimizer

from .. import ops
from ..config import OptimConf
from .lr_scheduler import build_lr_scheduler

logger = logging.getLogger()


@torch.no_grad()
def rescale_grads(model: nn.Module, scale: float) -> None:
    """Divide every gradient by `scale` (e.g. the number of accumulated tokens)."""
    if scale == 1.0:
        return
    if hasattr(model, "finish_backward"):
        model.finish_backward()
    for p in model.parameters():
        g = getattr(p, "_grad_shard", None)
        if g is not None:
            g.div_(scale)
        if p.grad is not None:
            p.grad.div_(scale)


class FusedAdamW(Optimizer):
    def __init__(self, params: Iterable[nn.Parameter], lr: float = 1e-3, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 1e-2):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)

    def _state_of(self, p):
        st = self.state[p]
        if not st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
        return st

    def fuse_with_reduce_scatter(self, enabled: bool = True) -> int:
        """Run the update of every FSDP shard inside the peer-memory reduce-scatter kernel of its unit
        (`SymmetricReduceScatter.reduce_scatter_adamw`), during backward, instead of in `step()`.
        Only meaningful without global-norm gradient clipping - the update of a shard then depends
        on nothing but its own reduced gradient - and without gradient accumulation over several
        backward passes (an accumulating pass falls back to the separate kernels).  `step()` still
        has to be called: it advances the step counters.  Returns the number of shards switched."""
        n = 0
        for group in self.param_groups:
            for p in group["params"]:
                unit = getattr(p, "_fsdp_unit", None)
                if unit is None or not unit.mixed_precision or unit.world_size == 1:
                    continue
                p._update_in_backward = functools.partial(self._update_in_backward, p, group) if enabled else None
                n += 1
        return n

    @torch.no_grad()
    def _update_in_backward(self, p, group, reducer, flat_grad, scale, sumsq, table=None) -> None:
        unit = p._fsdp_unit
        st = self._state_of(p)
        if p._lowp_shard is None:
            p._lowp_shard = torch.empty(p.numel(), dtype=unit.compute_dtype, device=p.device)
        b1, b2 = group["betas"]
        reducer.reduce_scatter_adamw(flat_grad, p.data, st["exp_avg"], st["exp_avg_sq"], p._lowp_shard, scale, sumsq,
                                     lr=group["lr"], beta1=b1, beta2=b2, eps=group["eps"],
                                     weight_decay=group["weight_decay"], step=st["step"] + 1, table=table)
        p._updated_in_backward = True

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        roots = set()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                unit = getattr(p, "_fsdp_unit", None)
                scale_ptr = None
                if unit is not None:
                    unit._sync_comm()
                    root = getattr(unit, "_root", unit)
                    scale_ptr = root._clip_coef
                    roots.add(root)
                if getattr(p, "_updated_in_backward", False):
                    # the reduce-scatter kernel already applied this step's update
                    p._updated_in_backward = False
                    self._state_of(p)["step"] += 1
                    p._master_version = getattr(p, "_master_version", 0) + 1
                    p._lowp_version = (p._version, p._master_version)
                    continue
                grad = p.grad if p.grad is not None else getattr(p, "_grad_shard", None)
                if grad is None:
                    continue
                st = self._state_of(p)
                st["step"] += 1
                low = None
                if unit is not None and unit.mixed_precision:
                    if p._lowp_shard is None:
                        p._lowp_shard = torch.empty(p.numel(), dtype=unit.compute_dtype, device=p.device)
                    low = p._lowp_shard
                ops.adamw_step(p.data, grad, st["exp_avg"], st["exp_avg_sq"], lr=group["lr"],
                               beta1=b1, beta2=b2, eps=group["eps"],
                               weight_decay=group["weight_decay"], step=st["step"], low=low,
                               **({"scale_ptr": scale_ptr} if scale_ptr is not None else {}))
                # master weights changed behind autograd's back: bump our own counter
                p._master_version = getattr(p, "_master_version", 0) + 1
                if low is not None:
                    p._lowp_version = (p._version, p._master_version)
        for root in roots:
            root._clip_coef = None
        return loss

    def zero_grad(self, set_to_none: bool = True) -> None:
        super().zero_grad(set_to_none=True)
        for group in self.param_groups:
            for p in group["params"]:
                if hasattr(p, "_grad_shard"):
                    p._grad_shard = None


def build_optimizer(model: nn.Module, cfg: OptimConf, total_steps: int, param_dtype: str = "bf16"):
    logger.info("Starting build of optimizer...")
    optimizer = FusedAdamW(model.parameters(), lr=cfg.lr, betas=(cfg.beta1, cfg.beta2),
                           weight_decay=cfg.weight_decay, eps=cfg.epsilon)
    scheduler = build_lr_scheduler(optimizer, cfg, total_steps)
    logger.info("Done with build of optimizer.")
    return optimizer, scheduler
