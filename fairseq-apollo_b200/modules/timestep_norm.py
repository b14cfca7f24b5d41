"""TimestepNorm — drop-in for fairseq/modules/norm_layer/timestep_norm.py:69-167 on the
mega_b200 CUDA kernels.

Same constructor ``(num_features, num_groups=None, prior_count=0, eps=1e-5)``, the same
buffers/parameters (prior_count int64 scalar buffer; prior_mean, prior_logv (G) — Parameters
when prior_count > 0, buffers otherwise; weight, bias (D) stored as offsets, the effective
scale is weight + 1), the same ``"norm_state"/{prev_mean, prev_var, prev_count}`` incremental
buffer and ``forward(x (B, L, D), padding_mask, incremental_state)``.

Like the reference, per-feature statistics (num_groups None or == num_features) need
prior_count > 1.  Running statistics are kept in fp32 whatever the activation dtype.
"""
from typing import Dict, Optional

import torch
import torch.nn as nn
from torch import Tensor
from torch.nn.parameter import Parameter

from .. import ops
from ..functions import TimestepNormFunction, needs_grad
from ..incremental_state import IncrementalStateMixin


class TimestepNorm(IncrementalStateMixin, nn.Module):
    def __init__(self, num_features: int, num_groups: Optional[int] = None,
                 prior_count: int = 0, eps: float = 1e-5) -> None:
        super().__init__()
        self.num_features = num_features
        self.num_groups = num_groups
        self._prior_count = prior_count

        if num_groups is None or num_groups == num_features:
            num_groups = num_features
            assert prior_count > 1
        else:
            assert self.num_features % num_groups == 0

        self.register_buffer("prior_count", torch.tensor(prior_count, dtype=torch.int64))
        if prior_count > 0:
            self.register_parameter("prior_mean", Parameter(torch.zeros(num_groups), requires_grad=True))
            self.register_parameter("prior_logv", Parameter(torch.zeros(num_groups), requires_grad=True))
        else:
            self.register_buffer("prior_mean", torch.zeros(num_groups))
            self.register_buffer("prior_logv", torch.zeros(num_groups))
        self.register_parameter("weight", Parameter(torch.zeros(num_features), requires_grad=True))
        self.register_parameter("bias", Parameter(torch.zeros(num_features), requires_grad=True))
        self.eps = eps

    def initial_statistics(self, batch_size, incremental_state=None):
        """(prev_count (B) int64, prev_mean, prev_var (B, G) fp32, saved_state or None)."""
        prev_mean = prev_var = prev_count = saved_state = None
        if incremental_state is not None:
            saved_state = self._get_input_buffer(incremental_state)
            if 'prev_mean' in saved_state:
                assert 'prev_var' in saved_state and 'prev_count' in saved_state
                prev_mean = saved_state['prev_mean']
                prev_var = saved_state['prev_var']
                prev_count = saved_state['prev_count']
        if prev_count is None:
            prev_count = self.prior_count.expand(batch_size).clone()
        # fresh tensors: a (1, G) expand of an fp32 parameter is a view of the parameter itself, and
        # the decode step updates its statistics in place
        if prev_mean is None:
            prev_mean = self.prior_mean.detach().float().expand(batch_size, -1).clone()
        if prev_var is None:
            prev_var = torch.exp(self.prior_logv.detach().float()).expand(batch_size, -1).clone()
        return prev_count, prev_mean, prev_var, saved_state

    def store_statistics(self, incremental_state, saved_state, count, mean, var):
        if incremental_state is not None:
            saved_state['prev_mean'] = mean
            saved_state['prev_var'] = var
            saved_state['prev_count'] = count
            self._set_input_buffer(incremental_state, saved_state)

    def forward(self, x: torch.Tensor, padding_mask: Optional[torch.Tensor] = None,
                incremental_state: Optional[Dict[str, Dict[str, Optional[Tensor]]]] = None) -> torch.Tensor:
        groups = None if (self.num_groups is None or self.num_groups == self.num_features) else self.num_groups
        if needs_grad(x, self.weight, self.bias, self.prior_mean, self.prior_logv):
            # differentiable path (norm_layer/timestep_norm.py:100-139 with the autograd Function)
            if incremental_state is not None:
                raise NotImplementedError("the incremental state is an inference feature: use torch.no_grad()")
            bsz = x.size(0)
            out, _, _, _ = TimestepNormFunction.apply(
                x, self.prior_count.expand(bsz).contiguous(), self.prior_mean.float().expand(bsz, -1),
                torch.exp(self.prior_logv.float()).expand(bsz, -1), self.weight.float() + 1.0, self.bias.float(),
                padding_mask, groups, self.eps)
            return out
        prev_count, prev_mean, prev_var, saved_state = self.initial_statistics(x.size(0), incremental_state)
        out, count, mean, var = ops.timestep_norm_fwd(x, prev_count, prev_mean, prev_var,
                                                      self.weight.detach().float() + 1.0, self.bias,
                                                      padding_mask, self.eps, groups)
        self.store_statistics(incremental_state, saved_state, count, mean, var)
        return out

    def _get_input_buffer(self, incremental_state):
        result = self.get_incremental_state(incremental_state, "norm_state")
        return result if result is not None else {}

    def _set_input_buffer(self, incremental_state, buffer):
        return self.set_incremental_state(incremental_state, "norm_state", buffer)

    def reorder_incremental_state(self, incremental_state, new_order: Tensor):
        return self._reorder_buffer(incremental_state, "norm_state", new_order)

    def extra_repr(self) -> str:
        return 'num_features={num_features}, num_groups={num_groups}, prior_count={_prior_count}, eps={eps}'.format(
            **self.__dict__)
