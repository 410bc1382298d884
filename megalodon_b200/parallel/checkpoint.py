"""Activation checkpointing for one block (the role fairscale's
`checkpoint_wrapper` plays in the reference, megalodon/model/mega.py:184).

The block runs without building a graph in the forward pass; only its tensor
inputs are kept.  In the backward pass the block is run again with a graph and
differentiated.  Two things are preserved across the two runs:

* the RNG state (CPU and current CUDA device), so dropout masks agree;
* the chunk-parallel receives: tensors received from the previous rank in the
  first run are taped and replayed in the second run, and sends are skipped, so
  recomputation needs no communication.
"""
from __future__ import annotations

from typing import Any, Tuple

import torch
import torch.nn as nn

from .chunk_parallel.mappings import HandoffTape, use_tape


def _rng_snapshot(device: torch.device):
    cpu = torch.get_rng_state()
    cuda = torch.cuda.get_rng_state(device) if device.type == "cuda" else None
    return cpu, cuda


def _rng_restore(device: torch.device, snap) -> None:
    cpu, cuda = snap
    torch.set_rng_state(cpu)
    if cuda is not None:
        torch.cuda.set_rng_state(cuda, device)


class _Checkpoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_fn, n_tensors, dummy, *args):
        tensors = args[:n_tensors]
        ctx.run_fn = run_fn
        ctx.extra = args[n_tensors:]
        device = tensors[0].device
        ctx.device = device
        ctx.rng = _rng_snapshot(device)
        ctx.tape = HandoffTape()
        ctx.save_for_backward(*tensors)
        with torch.no_grad(), use_tape(ctx.tape):
            out = run_fn(*tensors, *ctx.extra)
        return out

    @staticmethod
    def backward(ctx, *grads):
        inputs = [t.detach().requires_grad_(t.requires_grad) for t in ctx.saved_tensors]
        now = _rng_snapshot(ctx.device)
        _rng_restore(ctx.device, ctx.rng)
        ctx.tape.start_replay()
        with torch.enable_grad(), use_tape(ctx.tape):
            out = ctx.run_fn(*inputs, *ctx.extra)
        _rng_restore(ctx.device, now)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads)
                 if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        in_grads = tuple(t.grad if t.requires_grad else None for t in inputs)
        return (None, None, None) + in_grads + (None,) * len(ctx.extra)


def checkpoint(fn, *args):
    """Run `fn(*args)` under activation checkpointing.  Leading tensor arguments
    are differentiated through; everything from the first non-tensor argument
    on is passed along untouched (masks, tables, `None`)."""
    n = 0
    while n < len(args) and isinstance(args[n], torch.Tensor) and args[n].is_floating_point():
        n += 1
    assert n > 0, "checkpoint needs at least one floating-point tensor argument"
    dummy = torch.empty(0, requires_grad=True, device=args[0].device)
    return _Checkpoint.apply(fn, n, dummy, *args)


class CheckpointWrapper(nn.Module):
    """Wraps a block whose forward is `block(x, freqs_cis, mask, cache)` and
    returns `(y, cache)`.  Calls with a cache (inference) or without autograd
    run the block directly."""

    _is_wrapper = True

    def __init__(self, module: nn.Module):
        super().__init__()
        self._wrapped = module

    def __getattr__(self, name: str) -> Any:
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self._modules["_wrapped"], name)

    def forward(self, x, *rest):
        cache = rest[-1] if rest else None
        if cache is not None or not torch.is_grad_enabled():
            return self._wrapped(x, *rest)

        def run(x_, *extra):
            y, _ = self._wrapped(x_, *extra)
            return y

        y = checkpoint(run, x, *rest)
        return y, None


def checkpoint_wrapper(module: nn.Module) -> CheckpointWrapper:
    return CheckpointWrapper(module)
