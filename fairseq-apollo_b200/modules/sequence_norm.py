"""SequenceNorm — drop-in for fairseq/modules/norm_layer/sequence_norm.py:55-72 on the
mega_b200 CUDA kernels: masked normalisation over the sequence axis of x (B, D, L), per
channel or per channel group; weight/bias (D) stored as offsets (effective scale weight + 1).
"""
from typing import Optional

import torch
import torch.nn as nn
from torch.nn.parameter import Parameter

from .. import ops
from ..functions import SequenceNormFunction, needs_grad
from ..incremental_state import require_no_grad


class SequenceNorm(nn.Module):
    def __init__(self, num_features: int, num_groups: Optional[int] = None, eps: float = 1e-5) -> None:
        super().__init__()
        self.num_features = num_features
        self.num_groups = num_groups
        assert self.num_groups is None or self.num_features % self.num_groups == 0
        self.register_parameter("weight", Parameter(torch.zeros(num_features), requires_grad=True))
        self.register_parameter("bias", Parameter(torch.zeros(num_features), requires_grad=True))
        self.eps = eps

    def forward(self, x: torch.Tensor, padding_mask: Optional[torch.Tensor] = None,
                length_last: bool = True) -> torch.Tensor:
        if needs_grad(x, self.weight, self.bias):
            return SequenceNormFunction.apply(x, self.weight.float() + 1.0, self.bias.float(), padding_mask,
                                              self.eps, length_last, self.num_groups)
        y, _, _, _ = ops.sequence_norm_fwd(x, self.weight.detach().float() + 1.0, self.bias, padding_mask,
                                           self.eps, length_last, self.num_groups)
        return y

    def extra_repr(self) -> str:
        return 'num_features={num_features}, num_groups={num_groups}, eps={eps}'.format(**self.__dict__)
