"""Rotary position embedding with the interleaved-pair convention: features
(2i, 2i+1) form one complex number rotated by `pos * base^(-2i/d)`.  Positions
are counted *within a chunk*, so the table only needs `chunk_size` rows
(reference: megalodon/modules/rotary_positional_embedding.py:8-77)."""
from __future__ import annotations

import warnings
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops


class RotaryEmbedding(nn.Module):
    def __init__(self, embed_dim: int, max_positions: int, base: Optional[float] = None):
        super().__init__()
        assert embed_dim % 2 == 0
        self.embed_dim = embed_dim
        self.max_positions = max_positions
        self.base = 10000 if base is None else base
        exponents = torch.arange(0, embed_dim, 2, dtype=torch.float64) / embed_dim
        self.register_buffer("freqs", (1.0 / torch.pow(torch.tensor(float(self.base), dtype=torch.float64),
                                                        exponents)).float())
        self.freqs_cis: Optional[torch.Tensor] = None

    @torch.no_grad()
    def _table(self, n: int) -> torch.Tensor:
        self.max_positions = max(self.max_positions, n)
        t = torch.arange(self.max_positions, dtype=torch.float32, device=self.freqs.device)
        ang = torch.outer(t, self.freqs.float())
        return torch.polar(torch.ones_like(ang), ang)

    def get_freqs_cis(self, start: int, end: int) -> torch.Tensor:
        if self.freqs_cis is None or self.freqs_cis.device != self.freqs.device:
            self.freqs_cis = self._table(self.max_positions)
        if end > self.freqs_cis.shape[0]:
            warnings.warn(f"Extending rotary range from {self.freqs_cis.shape[0]} to {end}")
            self.freqs_cis = self._table(end)
        return self.freqs_cis[start:end]

    def forward(self, xq, xk, start: int):
        n = xq.shape[1]
        return apply_rotary_emb(xq, xk, self.get_freqs_cis(start, start + n), backward=False)

    def extra_repr(self) -> str:
        return f"dim={self.embed_dim}, max positions={self.max_positions}, base={self.base:.1f}"


def apply_rotary_emb(xq: torch.Tensor, xk: torch.Tensor, freqs_cis: torch.Tensor,
                     backward: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """xq, xk [B, C, H, D]; freqs_cis [C, D/2].  With `backward=True` the inputs
    are output-gradients and the conjugate rotation is applied."""
    return ops.rotary(xq, freqs_cis, backward), ops.rotary(xk, freqs_cis, backward)
