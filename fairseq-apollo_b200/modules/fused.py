"""Fused TimestepNorm -> EMA, the drop-in for the three statements
``x = self.norm(x, ...); mx = self.move(x.transpose(1, 2), ...); mx = move_act(mx.transpose(1, 2))``
of MovingAverageGatedAttention.forward (fairseq/modules/moving_average_gated_attention.py:306-316).
"""
from typing import Dict, Optional

import torch
from torch import Tensor

from .. import ops
from ..incremental_state import require_no_grad
from .exponential_moving_average import MultiHeadEMA
from .timestep_norm import TimestepNorm


def timestep_norm_ema(norm: TimestepNorm, move: MultiHeadEMA, x: Tensor,
                      padding_mask: Optional[Tensor] = None,
                      incremental_state: Optional[Dict[str, Dict[str, Optional[Tensor]]]] = None,
                      activation: Optional[str] = None, return_normed: bool = False):
    """x (B, L, D) -> mx (B, L, D) [, normed x (B, L, D)].

    One pass over x when the norm keeps per-feature statistics and the EMA is causal;
    otherwise the two modules run back to back.  Both modules' incremental buffers are read
    and updated exactly as their own ``forward`` would.
    """
    require_no_grad(x, norm.weight, move.alpha)
    assert activation in (None, 'silu')
    per_feature = norm.num_groups is None or norm.num_groups == norm.num_features
    if not per_feature or move.bidirectional:
        xn = norm(x, padding_mask, incremental_state)
        mx = move(xn.transpose(1, 2), padding_mask, incremental_state, activation).transpose(1, 2)
        return (mx, xn) if return_normed else mx
    prev_count, prev_mean, prev_var, nstate = norm.initial_statistics(x.size(0), incremental_state)
    p, q, g = move.coeffs()
    h_in = None
    estate = None
    if incremental_state is not None:
        estate = move._get_input_buffer(incremental_state)
        h_in = estate.get('prev_state')
    res = ops.tsn_ema_forward(x, prev_count, prev_mean, prev_var, norm.weight.detach().float() + 1.0, norm.bias,
                              norm.eps, p.squeeze(-1), q.squeeze(-1), g, move.omega, padding_mask, h_in,
                              want_state=incremental_state is not None, silu=activation == 'silu',
                              want_normed=return_normed)
    norm.store_statistics(incremental_state, nstate, res["count"], res["mean"], res["var"])
    if incremental_state is not None:
        estate['prev_state'] = res["h"]
        move._set_input_buffer(incremental_state, estate)
    return (res["y"], res["xn"]) if return_normed else res["y"]
