"""mega_b200: Mega's EMA layer, TimestepNorm and SequenceNorm on hand-written sm_100a CUDA
kernels behind the reference's module API.  Import name: ``fairseq_apollo_b200``."""
from . import ops
from ._lib import LIB_PATH, MegaError, launch_count
from .modules import (AttentionSoftmax, EfficientAttention, MovingAverageGatedAttention, MultiHeadComplexEMA, MultiHeadEMA,
                      SequenceNorm, TimestepNorm, sequence_norm_ema, timestep_norm_ema)

__all__ = ["ops", "MultiHeadEMA", "MultiHeadComplexEMA", "TimestepNorm", "SequenceNorm", "AttentionSoftmax", "EfficientAttention",
           "timestep_norm_ema", "sequence_norm_ema", "MovingAverageGatedAttention",
           "MegaError", "launch_count", "LIB_PATH"]
