"""Warm-up + decay learning-rate multipliers: `linear`, `cosine`, `constant`
(reference: megalodon/optim/lr_scheduler.py:8-75).  Each returns the factor
applied to the base learning rate at a given step."""
from __future__ import annotations

import math
from functools import partial

from torch.optim import lr_scheduler

from ..config import OptimConf


def _warmup(step: int, warmup: int, init_ratio: float) -> float:
    return init_ratio + (1.0 - init_ratio) * step / warmup


def lr_linear(step: int, warmup: int, total_steps: int, init_ratio: float, end_ratio: float) -> float:
    if step < warmup:
        return _warmup(step, warmup, init_ratio)
    if step > total_steps:
        return end_ratio
    s = (step - warmup) / max(1, total_steps - warmup)
    return s * end_ratio + (1.0 - s)


def lr_cosine(step: int, warmup: int, total_steps: int, cycles: float, init_ratio: float,
              end_ratio: float) -> float:
    if step < warmup:
        return _warmup(step, warmup, init_ratio)
    if step > total_steps:
        return end_ratio
    s = (step - warmup) / max(1, total_steps - warmup)
    return end_ratio + 0.5 * (1.0 - end_ratio) * (math.cos(math.pi * s * cycles) + 1.0)


def lr_constant(step: int, warmup: int, init_ratio: float) -> float:
    return _warmup(step, warmup, init_ratio) if step < warmup else 1.0


def build_lr_fn(cfg: OptimConf, total_steps: int):
    if cfg.scheduler == "linear":
        return partial(lr_linear, warmup=cfg.warmup, total_steps=total_steps,
                       init_ratio=cfg.lr_init_ratio, end_ratio=cfg.lr_end_ratio)
    if cfg.scheduler == "constant":
        return partial(lr_constant, warmup=cfg.warmup, init_ratio=cfg.lr_init_ratio)
    if cfg.scheduler == "cosine":
        return partial(lr_cosine, warmup=cfg.warmup, total_steps=total_steps, cycles=cfg.cycles,
                       init_ratio=cfg.lr_init_ratio, end_ratio=cfg.lr_end_ratio)
    raise NotImplementedError(f"Unknown scheduler: {cfg.scheduler}")


def build_lr_scheduler(optimizer, cfg: OptimConf, total_steps: int):
    return lr_scheduler.LambdaLR(optimizer, build_lr_fn(cfg, total_steps))
