"""Chunk-parallel (sequence-split) region boundaries.

A sequence is cut into contiguous pieces, one per rank of the chunk group.
Only two small recurrent states cross a cut: the CEMA complex hidden state and
the TimestepNorm running statistics.  `send_to_next_…` / `recv_from_prev_…`
move them forward in the forward pass and move their gradients backward in the
backward pass (reference: megalodon/modules/chunk_parallel/mappings.py:25-191).

Two transports exist behind the same autograd functions:

* `torch.distributed` send/recv (gloo on CPU, NCCL on GPU) - the baseline;
* a peer-memory mailbox (`parallel/symm.py`): the producer's kernel stores the
  state straight into the consumer GPU's memory over NVLink and raises a flag,
  the consumer polls the flag with a bounded wait.  Selected with
  `set_handoff_transport("p2p")` once symmetric memory is set up.

Unlike the reference, the gradient arriving from the next rank is *added* to
the locally produced gradient of the sent tensor instead of overwriting it
(the reference notes this as a TODO at mappings.py:64).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..initialize import (
    get_chunk_parallel_group,
    get_chunk_parallel_next_rank,
    get_chunk_parallel_prev_rank,
    get_chunk_parallel_rank,
    get_chunk_parallel_world_size,
)
from ..utils import comm_device, all_gather_flat

_TRANSPORT = {"kind": "nccl", "mailbox": None}


def set_handoff_transport(kind: str, mailbox=None) -> None:
    """`kind` is "nccl" (torch.distributed send/recv) or "p2p" (peer mailbox)."""
    if kind not in ("nccl", "p2p"):
        raise ValueError(kind)
    if kind == "p2p" and mailbox is None:
        raise ValueError("p2p transport needs a mailbox")
    _TRANSPORT["kind"] = kind
    _TRANSPORT["mailbox"] = mailbox


def get_handoff_transport() -> str:
    return _TRANSPORT["kind"]


def should_send_to_next() -> bool:
    return get_chunk_parallel_world_size() > 1 and get_chunk_parallel_next_rank() is not None


def should_recv_from_prev() -> bool:
    return get_chunk_parallel_world_size() > 1 and get_chunk_parallel_prev_rank() is not None


def _wire(t: torch.Tensor) -> torch.Tensor:
    dev = comm_device(get_chunk_parallel_group())
    t = t.detach().contiguous()
    return t if t.device == dev else t.to(dev)


def _send(t: torch.Tensor, dst: int, direction: str) -> None:
    if _TRANSPORT["kind"] == "p2p":
        _TRANSPORT["mailbox"].send(t.detach(), direction)
    else:
        dist.send(_wire(t), dst, group=get_chunk_parallel_group())


def _recv(buf: torch.Tensor, src: int, direction: str) -> torch.Tensor:
    if _TRANSPORT["kind"] == "p2p":
        _TRANSPORT["mailbox"].recv(buf, direction)
        return buf
    w = _wire(buf)
    dist.recv(w, src, group=get_chunk_parallel_group())
    if w.data_ptr() != buf.data_ptr():
        buf.copy_(w)
    return buf


class HandoffTape:
    """Record of the tensors received during one forward of a checkpointed
    block.  When the block is recomputed for its backward pass, receives are
    served from the tape and sends are skipped, so recomputation costs no
    communication and cannot stall on a neighbour (the reference re-runs its
    blocking send/recv pair during recomputation)."""

    def __init__(self):
        self.items = []
        self.mode = "record"
        self._cursor = 0

    def push(self, t: torch.Tensor) -> None:
        self.items.append(t.detach())

    def pop(self) -> torch.Tensor:
        t = self.items[self._cursor]
        self._cursor += 1
        return t

    def start_replay(self) -> None:
        self.mode = "replay"
        self._cursor = 0


_TAPE: list = [None]


def current_tape() -> Optional[HandoffTape]:
    return _TAPE[0]


class use_tape:
    def __init__(self, tape: Optional[HandoffTape]):
        self.tape = tape

    def __enter__(self):
        self.prev = _TAPE[0]
        _TAPE[0] = self.tape
        return self.tape

    def __exit__(self, *exc):
        _TAPE[0] = self.prev
        return False


class _SendToNext(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, really_send):
        if really_send:
            _send(x, get_chunk_parallel_next_rank(), "fwd")
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        incoming = torch.empty_like(g)
        _recv(incoming, get_chunk_parallel_next_rank(), "bwd")
        return g + incoming, None


class _RecvFromPrev(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buf, replayed):
        if replayed is not None:
            return replayed.clone()
        out = torch.empty_like(buf)
        _recv(out, get_chunk_parallel_prev_rank(), "fwd")
        return out

    @staticmethod
    def backward(ctx, g):
        _send(g, get_chunk_parallel_prev_rank(), "bwd")
        return None, None


class _Attach(torch.autograd.Function):
    """Returns `x` unchanged while making `token` an autograd ancestor of the
    result, so that `token`'s producer (a send) runs its backward (a receive)
    even though its value is not used locally."""

    @staticmethod
    def forward(ctx, x, token):
        ctx.token_meta = (token.shape, token.dtype, token.device)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        shape, dtype, device = ctx.token_meta
        return g, torch.zeros(shape, dtype=dtype, device=device)


def attach_to_graph(x: torch.Tensor, token: torch.Tensor) -> torch.Tensor:
    return _Attach.apply(x, token)


def _split(x: torch.Tensor, dim: Optional[int]) -> torch.Tensor:
    world = get_chunk_parallel_world_size()
    if world == 1:
        return x
    d = x.dim() - 1 if dim is None else dim % x.dim()
    width = x.shape[d] // world
    assert width * world == x.shape[d]
    return x.narrow(d, get_chunk_parallel_rank() * width, width).contiguous()


def _gather(x: torch.Tensor, dim: Optional[int]) -> torch.Tensor:
    world = get_chunk_parallel_world_size()
    if world == 1:
        return x
    d = x.dim() - 1 if dim is None else dim % x.dim()
    x = x.contiguous()
    out = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    all_gather_flat(out, x, get_chunk_parallel_group())
    shape = list(x.shape)
    shape[d] *= world
    return out.movedim(0, d).reshape(shape)


class _GatherFromChunk(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        return _gather(x, dim)

    @staticmethod
    def backward(ctx, g):
        return _split(g, ctx.dim), None


def send_to_next_chunk_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    tape = current_tape()
    replay = tape is not None and tape.mode == "replay"
    return _SendToNext.apply(input_, not replay)


def recv_from_prev_chunk_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    """`input_` only provides shape/dtype/device (and `requires_grad`, which
    decides whether the gradient is sent back in the backward pass)."""
    tape = current_tape()
    if tape is not None and tape.mode == "replay":
        return _RecvFromPrev.apply(input_, tape.pop())
    out = _RecvFromPrev.apply(input_, None)
    if tape is not None:
        tape.push(out)
    return out


def gather_from_chunk_parallel_region(input_: torch.Tensor, dim: Optional[int] = None) -> torch.Tensor:
    return _GatherFromChunk.apply(input_, dim)
