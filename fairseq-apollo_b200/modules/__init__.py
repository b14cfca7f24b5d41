from .exponential_moving_average import MultiHeadEMA
from .timestep_norm import TimestepNorm
from .sequence_norm import SequenceNorm
from .fused import sequence_norm_ema, timestep_norm_ema

__all__ = ["MultiHeadEMA", "TimestepNorm", "SequenceNorm", "timestep_norm_ema", "sequence_norm_ema"]
