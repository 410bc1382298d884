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
    def forward(ctx, run_fn, spec, dummy, *tensors):
        # `spec` rebuilds the original argument list from (tensor slots, constants)
        ctx.run_fn = run_fn
        ctx.spec = spec
        device = tensors[0].device
        ctx.device = device
        ctx.rng = _rng_snapshot(device)
        ctx.tape = HandoffTape()
        ctx.save_for_backward(*tensors)
        with torch.no_grad(), use_tape(ctx.tape):
            out = run_fn(*_rebuild(spec, tensors))
        return out

    @staticmethod
    def backward(ctx, *grads):
        inputs = [t.detach().requires_grad_(t.requires_grad) for t in ctx.saved_tensors]
        now = _rng_snapshot(ctx.device)
        _rng_restore(ctx.device, ctx.rng)
        ctx.tape.start_replay()
        with torch.enable_grad(), use_tape(ctx.tape):
            out = ctx.run_fn(*_rebuild(ctx.spec, inputs))
        _rng_restore(ctx.device, now)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads)
                 if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        in_grads = tuple(t.grad if t.requires_grad else None for t in inputs)
        return (None, None, None) + in_grads


def _rebuild(spec, tensors):
    return [tensors[v] if is_slot else v for is_slot, v in spec]


def checkpoint(fn, *args):
    """Run `fn(*args)` under activation checkpointing.  Tensor arguments that
    require grad are differentiated through (real or complex); every other
    argument (masks, tables, integer tensors, `None`) is passed along as a
    constant.  `fn` must return a tensor or a flat tuple of tensors / None."""
    spec, tensors = [], []
    for a in args:
        if isinstance(a, torch.Tensor) and a.requires_grad:
            spec.append((True, len(tensors)))
            tensors.append(a)
        else:
            spec.append((False, a))
    if not tensors:
        # nothing upstream needs a gradient: still recompute for the parameters
        first = next(a for a in args if isinstance(a, torch.Tensor))
        anchor = first.detach().requires_grad_(True)
        spec[[i for i, a in enumerate(args) if a is first][0]] = (True, 0)
        tensors.append(anchor)
    dummy = torch.empty(0, requires_grad=True, device=tensors[0].device)
    return _Checkpoint.apply(fn, tuple(spec), dummy, *tensors)


class CheckpointWrapper(nn.Module):
    """Wraps a block with signature `block(x, freqs_cis, mask, cache, carry, piece)`
    returning `(y, state)`, where `state` is an inference cache, a tuple of
    carried tensors (sequence micro-batching) or None.  Calls with a cache
    (inference) or without autograd run the block directly."""

    _is_wrapper = True

    def __init__(self, module: nn.Module):
        super().__init__()
        self._wrapped = module
        # The wrapper is invisible in state dicts (like fairscale's checkpoint_wrapper, which the
        # reference uses): keys are those of the wrapped block, so a checkpoint written with
        # checkpointing loads into a model built without it and the other way round.
        self._register_state_dict_hook(_strip_wrapper_prefix)
        self._register_load_state_dict_pre_hook(_insert_wrapper_prefix)

    def __getattr__(self, name: str) -> Any:
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self._modules["_wrapped"], name)

    def forward(self, x, freqs_cis=None, mask=None, cache=None, carry=None, piece=None):
        if cache is not None or not torch.is_grad_enabled():
            return self._wrapped(x, freqs_cis, mask, cache, carry, piece)

        def run(x_, freqs_, mask_, piece_, *carry_):
            y, state = self._wrapped(x_, freqs_, mask_, None, tuple(carry_) if carry_ else None, piece_)
            return (y,) + (tuple(state) if state is not None else ())

        out = checkpoint(run, x, freqs_cis, mask, piece, *(carry or ()))
        y, state = out[0], out[1:]
        return y, (tuple(state) if state else None)


def _strip_wrapper_prefix(module, state_dict, prefix, local_metadata):
    inner = prefix + "_wrapped."
    for key in [k for k in state_dict if k.startswith(inner)]:
        state_dict[prefix + key[len(inner):]] = state_dict.pop(key)
    return state_dict


def _insert_wrapper_prefix(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
    inner = prefix + "_wrapped."
    for key in [k for k in state_dict if k.startswith(prefix) and not k.startswith(inner)]:
        state_dict[inner + key[len(prefix):]] = state_dict.pop(key)


def checkpoint_wrapper(module: nn.Module) -> CheckpointWrapper:
    return CheckpointWrapper(module)
