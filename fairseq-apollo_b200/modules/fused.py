"""Fused TimestepNorm -> EMA, the drop-in for the three statements
``x = self.norm(x, ...); mx = self.move(x.transpose(1, 2), ...); mx = move_act(mx.transpose(1, 2))``
of MovingAverageGatedAttention.forward (fairseq/modules/moving_average_gated_attention.py:306-316).
"""
from typing import Dict, Optional

import torch
from torch import Tensor

from .. import ops
from ..functions import needs_grad
from .exponential_moving_average import MultiHeadEMA
from .sequence_norm import SequenceNorm
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
    assert activation in (None, 'silu')
    per_feature = norm.num_groups is None or norm.num_groups == norm.num_features
    train = needs_grad(x, *norm.parameters(), *move.parameters())
    if train or not per_feature or move.bidirectional:
        # training, grouped statistics or a bidirectional layer: the two modules in turn
        xn = norm(x, padding_mask, incremental_state)
        mx = move(xn.transpose(1, 2), padding_mask, incremental_state, activation).transpose(1, 2)
        return (mx, xn) if return_normed else mx
    if (incremental_state is not None and x.size(1) == 1 and padding_mask is None and x.is_contiguous()
            and (not move.complex or move.ndim in (2, 4, 8, 16, 32))):
        return _decode_step(norm, move, x, incremental_state, activation, return_normed)
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
                              want_normed=return_normed, complex_poles=move.complex)
    norm.store_statistics(incremental_state, nstate, res["count"], res["mean"], res["var"])
    if incremental_state is not None:
        estate['prev_state'] = res["h"]
        move._set_input_buffer(incremental_state, estate)
    return (res["y"], res["xn"]) if return_normed else res["y"]


def sequence_norm_ema(norm: SequenceNorm, move: MultiHeadEMA, x: Tensor, padding_mask: Optional[Tensor] = None,
                      activation: Optional[str] = None):
    """x (B, D, L) -> EMA(SequenceNorm(x)) (B, D, L): the bidirectional branch of the Mega block
    (moving_average_gated_attention.py:298-303, 313).  One kernel, one pass over x, when the norm
    is per channel and the rows fit the row-resident kernel; otherwise the two modules in turn."""
    assert activation in (None, 'silu')
    train = needs_grad(x, *norm.parameters(), *move.parameters())
    if not train and not move.complex and norm.num_groups is None and move.truncation is None:
        p, q, g = move.coeffs()
        y = ops.sqn_ema_forward(x, norm.weight.detach().float() + 1.0, norm.bias, norm.eps, p.squeeze(-1),
                                q.squeeze(-1), g, move.omega, padding_mask, move.bidirectional, move.shift,
                                silu=activation == 'silu')
        if y is not None:
            return y
    return move(norm(x, padding_mask), padding_mask, None, activation)


def _fp32_params(norm: TimestepNorm, move: MultiHeadEMA):
    """fp32, contiguous copies of everything the decode kernel reads, cached until a parameter
    is modified (checked through the tensors' version counters)."""
    third = move.theta if move.complex else move.beta
    tensors = (norm.weight, norm.bias, move.alpha, move.delta, third, move.gamma, move.omega)
    key = tuple((t.data_ptr(), t._version) for t in tensors)
    cache = getattr(move, "_decode_cache", None)
    if cache is None or cache[0] != key:
        if move.complex:   # q, g complex64 (K, N): the kernel reads them as interleaved (re, im) floats
            p, q, g = ops.cema_coeffs(move.alpha, move.delta, move.theta, move.gamma)
            p, q, g = p.reshape(p.shape[0], -1).contiguous(), q.reshape(q.shape[0], -1).contiguous(), g.contiguous()
        else:
            p, q, g = ops.ema_coeffs(move.alpha, move.delta, move.beta, move.gamma)
        cache = (key, (norm.weight.detach().float() + 1.0).contiguous(), norm.bias.detach().float().contiguous(),
                 p, q, g, move.omega.detach().float().reshape(-1).contiguous())
        move._decode_cache = cache
    return cache[1:]


def _decode_step(norm, move, x, incremental_state, activation, return_normed):
    """Single-token step (x: (B, 1, D)): one fused kernel, running state updated in place."""
    bsz, _, dim = x.shape
    gamma, beta, p, q, g, omega = _fp32_params(norm, move)
    nstate = norm._get_input_buffer(incremental_state)
    if 'prev_mean' not in nstate:
        count, mean, var, nstate = norm.initial_statistics(bsz, incremental_state)
        nstate['prev_count'], nstate['prev_mean'], nstate['prev_var'] = count.clone(), mean, var
        norm._set_input_buffer(incremental_state, nstate)
    for k in ('prev_mean', 'prev_var'):
        t = nstate[k]
        if t.dtype != torch.float32 or not t.is_contiguous():
            nstate[k] = t.float().contiguous()
    estate = move._get_input_buffer(incremental_state)
    h = estate.get('prev_state')
    sdtype = torch.complex64 if move.complex else torch.float32
    if h is None:
        h = torch.zeros(bsz, dim, move.ndim, device=x.device, dtype=sdtype)
    elif h.dtype != sdtype or not h.is_contiguous():
        h = h.to(sdtype).contiguous()
    estate['prev_state'] = h
    move._set_input_buffer(incremental_state, estate)
    y = torch.empty_like(x)
    xn = torch.empty_like(x) if return_normed else None
    step = ops.tsn_cema_step_ if move.complex else ops.tsn_ema_step_
    step(x.view(bsz, dim), y.view(bsz, dim), nstate['prev_count'], nstate['prev_mean'],
         nstate['prev_var'], gamma, beta, norm.eps, p, q, g, omega, h,
         silu=activation == 'silu', xn_out=None if xn is None else xn.view(bsz, dim))
    return (y, xn) if return_normed else y
