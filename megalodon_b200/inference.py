"""Perplexity-style scoring of long inputs with bounded memory: the sequence is
streamed through the cached forward path `MAX_CHUNKS_PER_BATCH` chunks at a
time; once `TRUNCATE_CHUNKS` chunks have been consumed, the normalisation
statistics are re-derived from the most recent
`TRUNCATE_CHUNKS - MAX_CHUNKS_PER_BATCH` chunks only, which bounds the drift of
the cumulative statistics (reference: megalodon/inference.py:16-76)."""
from __future__ import annotations

import logging

import torch
import torch.nn.functional as F

from .modules.losses import cross_entropy
from .parallel.utils import reduce_scalar
from .utils import get_torch_dtype, init_cache, truncate_cache

logger = logging.getLogger()

MAX_CHUNKS_PER_BATCH = 2
TRUNCATE_CHUNKS = 8


def get_max_length(length: int) -> int:
    """Largest length over all ranks, so every rank makes the same number of calls."""
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        return int(reduce_scalar(length, op="max"))
    return length


@torch.inference_mode()
def inference(model, tokens: torch.Tensor, targets: torch.Tensor, dtype: str) -> torch.Tensor:
    """Per-token negative log-likelihood [B, L] of `targets` given `tokens`."""
    model.eval()
    bsz, length = tokens.shape
    compute_dtype = get_torch_dtype(dtype)
    c = model.chunk_size
    max_length = get_max_length(length)
    tokens = F.pad(tokens, (0, max_length - length), value=0)
    targets = F.pad(targets, (0, max_length - length), value=-100)
    n_chunks = max_length // c
    body = n_chunks * c

    cache = init_cache(bsz, model, compute_dtype, device=tokens.device) if n_chunks > 0 else None
    losses = []
    for first in range(0, n_chunks, MAX_CHUNKS_PER_BATCH):
        s = first * c
        e = min(first + MAX_CHUNKS_PER_BATCH, n_chunks) * c
        pred, cache = model(tokens[:, s:e], cache=cache)
        losses.append(cross_entropy(pred, targets[:, s:e]).view(bsz, e - s))
        more_to_come = e < body or body < max_length
        if TRUNCATE_CHUNKS * c <= e and more_to_come:
            ss = e - (TRUNCATE_CHUNKS - MAX_CHUNKS_PER_BATCH) * c
            fresh = init_cache(bsz, model, compute_dtype, truncate=True, device=tokens.device)
            _, stats_only = model(tokens[:, ss:e], cache=fresh)
            cache = truncate_cache(cache, stats_only)
    if body < max_length:
        pred, _ = model(tokens[:, body:], cache=cache)
        losses.append(cross_entropy(pred, targets[:, body:]).view(bsz, max_length - body))
    return torch.cat(losses, dim=1)[:, :length]
