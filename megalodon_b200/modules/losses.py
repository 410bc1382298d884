"""Token-level cross-entropy under chunk parallelism: every rank scores its own
slice of the sequence, then the per-token losses are gathered rank-major over
the chunk group so each rank returns the full [B * L] vector (reference:
megalodon/modules/losses.py:12-59)."""
from __future__ import annotations

from typing import Optional

from torch import Tensor

from .. import ops
from ..parallel.initialize import get_chunk_parallel_rank, get_chunk_parallel_world_size
from ..parallel.chunk_parallel import gather_from_chunk_parallel_region


def cross_entropy(logits: Tensor, target: Tensor, weight: Optional[Tensor] = None,
                  ignore_index: int = -100, label_smoothing: float = 0.0) -> Tensor:
    """logits [B, L_local, V]; target [B, L_total] -> losses [cp * B * L_local]."""
    _, local_len, _ = logits.shape
    cp = get_chunk_parallel_world_size()
    assert local_len * cp == target.size(1), (local_len, cp, target.size(1))
    r = get_chunk_parallel_rank()
    tgt = target[:, r * local_len:(r + 1) * local_len]
    losses = ops.cross_entropy(logits.flatten(0, 1), tgt.flatten(0, 1), weight, ignore_index,
                               label_smoothing)
    return gather_from_chunk_parallel_region(losses)
