from .exponential_moving_average import MultiHeadEMA
from .complex_exponential_moving_average import MultiHeadComplexEMA
from .timestep_norm import TimestepNorm
from .sequence_norm import SequenceNorm
from .attention_softmax import AttentionSoftmax
from .efficient_attention import EfficientAttention, attention
from .fused import sequence_norm_ema, timestep_norm_ema
from .moving_average_gated_attention import MovingAverageGatedAttention, RotaryEmbedding, SimpleRelativePositionalBias

__all__ = ["MultiHeadEMA", "MultiHeadComplexEMA", "TimestepNorm", "SequenceNorm", "AttentionSoftmax", "EfficientAttention", "attention",
           "timestep_norm_ema", "sequence_norm_ema", "MovingAverageGatedAttention", "RotaryEmbedding",
           "SimpleRelativePositionalBias"]
