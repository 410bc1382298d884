from .layer_norm import FusedLayerNorm, FusedRMSNorm
from .normalized_feedforward_network import NormalizedFeedForwardNetwork
from .rotary_positional_embedding import RotaryEmbedding, apply_rotary_emb
from .moving_average_gated_attention import MovingAverageGatedAttention
from .timestep_norm import TimestepNorm
from .complex_exponential_moving_average import MultiHeadComplexEMA
from .attention_softmax import AttentionSoftmax, SwiftAttention

__all__ = [
    "FusedLayerNorm", "FusedRMSNorm", "MovingAverageGatedAttention", "MultiHeadComplexEMA",
    "NormalizedFeedForwardNetwork", "RotaryEmbedding", "apply_rotary_emb", "TimestepNorm",
    "AttentionSoftmax", "SwiftAttention",
]
