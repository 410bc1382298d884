"""Pre-normalised feed-forward block: LayerNorm -> SiLU MLP (or SwiGLU) ->
residual.  The residual added is supplied by the caller: in a Megalodon block
it is the block *input*, not the attention output (reference:
megalodon/modules/normalized_feedforward_network.py:16-98)."""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..parallel.initialize import get_model_parallel_world_size
from ..parallel.model_parallel import (
    ColumnParallelLinear,
    RowParallelLinear,
    gather_from_model_parallel_region,
)
from ..utils import get_init_fn
from .layer_norm import FusedLayerNorm


class NormalizedFeedForwardNetwork(nn.Module):
    def __init__(self, model_dim, ffn_hidden_dim, dropout=0.0, hidden_dropout=0.0, swiglu=False,
                 norm_affine=True, norm_eps=1e-5, rescale=None, init_mode="bert"):
        super().__init__()
        self.model_dim = model_dim
        self.hidden_dim = ffn_hidden_dim
        self.dropout = dropout
        self.hidden_dropout = hidden_dropout
        self.swiglu = swiglu
        self.rescale_init = rescale
        self.init_mode = init_mode
        self.norm = FusedLayerNorm(model_dim, elementwise_affine=norm_affine, eps=norm_eps)
        init_fn = get_init_fn(init_mode)
        # without SwiGLU the SiLU is fused into fc1's GEMM epilogue
        self.fc1 = ColumnParallelLinear(model_dim, ffn_hidden_dim, bias=False, input_is_parallel=False,
                                        gather_output=False, init_method=init_fn,
                                        activation=None if swiglu else "silu")
        self.fc2 = RowParallelLinear(ffn_hidden_dim, model_dim, bias=False, input_is_parallel=True,
                                     parallel_output=True, init_method=init_fn)
        self.fc3 = ColumnParallelLinear(model_dim, ffn_hidden_dim, bias=False, input_is_parallel=False,
                                        gather_output=False, init_method=init_fn) if swiglu else None
        if rescale is None:
            self.register_parameter("alpha", None)
        else:
            assert rescale > 0.0, "Layer scale init value should be positive."
            # sized like fc2's (feature-sharded) output, so layer scale also works with mp > 1
            self.alpha = nn.Parameter(torch.full((self.fc2.output_size_per_partition,), float(rescale)))

    def rescale(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.alpha is None else self.alpha * x

    def forward(self, x, residual):
        x = gather_from_model_parallel_region(x)
        x = self.norm(x)
        if self.swiglu:
            hidden = ops.swiglu(self.fc1(x), self.fc3(x))
        else:
            hidden = self.fc1(x)
        hidden = ops.memory_efficient_dropout(hidden, self.hidden_dropout, self.training)
        if (self.alpha is None and get_model_parallel_world_size() == 1
                and not (self.training and self.dropout > 0.0)):
            return ops.linear_add(hidden, self.fc2.weight, None, residual)     # residual add in the GEMM epilogue
        x = self.fc2(hidden)
        x = ops.memory_efficient_dropout(x, self.dropout, self.training)
        return self.rescale(x) + residual

    def extra_repr(self) -> str:
        return (f"dim={self.model_dim}, hdim={self.hidden_dim}, swiglu={self.swiglu}, "
                f"init={self.init_mode}, rescale={self.rescale_init}")
