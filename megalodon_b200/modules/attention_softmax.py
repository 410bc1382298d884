"""Module wrappers around the standalone softmax / attention operators (the
reference ships them as unused helpers: modules/attention_softmax.py,
modules/fused_attention.py)."""
from __future__ import annotations

from torch import nn

from .. import ops


class AttentionSoftmax(nn.Module):
    def __init__(self, dropout: float = 0.0, use_causal_mask: bool = True):
        super().__init__()
        self.dropout = dropout
        self.use_causal_mask = use_causal_mask

    def forward(self, x):
        return ops.attention_softmax(x, self.dropout, self.use_causal_mask, self.training)

    def extra_repr(self) -> str:
        return f"dropout={self.dropout}, causal={self.use_causal_mask}"


class SwiftAttention(nn.Module):
    def __init__(self, scale: float = 1.0, dropout: float = 0.0, use_causal_mask: bool = True):
        super().__init__()
        self.scale = scale
        self.dropout = dropout
        self.use_causal_mask = use_causal_mask

    def forward(self, q, k, v):
        return ops.attention(q, k, v, self.scale, self.dropout, self.use_causal_mask, self.training)

    def extra_repr(self) -> str:
        return f"scale={self.scale}, dropout={self.dropout}, causal={self.use_causal_mask}"
