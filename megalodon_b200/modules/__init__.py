"""Model building blocks.  Public names: those of the reference's `megalodon.modules`
(modules/__init__.py) plus the CEMA module and the two attention wrappers; imported on first use."""
import importlib

_WHERE = {
    "FusedLayerNorm": "layer_norm", "FusedRMSNorm": "layer_norm",
    "TimestepNorm": "timestep_norm",
    "MultiHeadComplexEMA": "complex_exponential_moving_average",
    "MovingAverageGatedAttention": "moving_average_gated_attention",
    "NormalizedFeedForwardNetwork": "normalized_feedforward_network",
    "RotaryEmbedding": "rotary_positional_embedding", "apply_rotary_emb": "rotary_positional_embedding",
    "AttentionSoftmax": "attention_softmax", "SwiftAttention": "attention_softmax",
}
__all__ = sorted(_WHERE)


def __getattr__(name):
    if name in _WHERE:
        value = getattr(importlib.import_module(f"{__name__}.{_WHERE[name]}"), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
