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
    # the decode fast path first: one token, an incremental state, inference
    if (incremental_state is not None and x.size(1) == 1 and padding_mask is None and per_feature
            and not move.bidirectional and not torch.is_grad_enabled() and x.is_contiguous()
            and (not move.complex or move.ndim in (2, 4, 8, 16, 32))):
        return _decode_step(norm, move, x, incremental_state, activation, return_normed)
    train = torch.is_grad_enabled() and needs_grad(x, *norm.parameters(), *move.parameters())
    if train or not per_feature or move.bidirectional:
        # training, grouped statistics or a bidirectional layer: the two modules in turn
        xn = norm(x, padding_mask, incremental_state)
        mx = move(xn.transpose(1, 2), padding_mask, incremental_state, activation).transpose(1, 2)
        return (mx, xn) if return_normed else mx
    if (incremental_state is not None and x.size(1) == 1 and padding_mask is None and x.is_contiguous()
            and (not move.complex or move.ndim in (2, 4, 8, 16, 32))):
        return _decode_step(norm, move, x, incremental_state, activation, return_normed)
    prev_count, prev_mean, prev_var, nstate = norm.initial_statistics(x.size(0), incremental_state)
    if move.complex:
        p, q, g = move.coeffs()
        p, q, gamma_eff, beta, omega = p.squeeze(-1), q.squeeze(-1), norm.weight.detach().float() + 1.0, norm.bias, move.omega
    else:
        # inference: coefficients and the effective scale come from the cache that the single-token step
        # uses too (rebuilt when a parameter's version counter moves), not from a kernel launch per call
        gamma_eff, beta, p, q, g, omega = _fp32_params(norm, move)
    h_in = None
    estate = None
    if incremental_state is not None:
        estate = move._get_input_buffer(incremental_state)
        h_in = estate.get('prev_state')
    res = ops.tsn_ema_forward(x, prev_count, prev_mean, prev_var, gamma_eff, beta,
                              norm.eps, p, q, g, omega, padding_mask, h_in,
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
    # (in-place updates bump the version counters; a parameter that was replaced has a new identity)
    key = (norm.weight._version, norm.bias._version, move.alpha._version, move.delta._version, third._version,
           move.gamma._version, move.omega._version)
    cache = getattr(move, "_decode_cache", None)
    if cache is not None and (cache[0] != key or any(a is not b for a, b in zip(cache[-1], tensors))):
        cache = None
    if cache is None:
        if move.complex:   # q, g complex64 (K, N): the kernel reads them as interleaved (re, im) floats
            p, q, g = ops.cema_coeffs(move.alpha, move.delta, move.theta, move.gamma)
            p, q, g = p.reshape(p.shape[0], -1).contiguous(), q.reshape(q.shape[0], -1).contiguous(), g.contiguous()
        else:
            p, q, g = ops.ema_coeffs(move.alpha, move.delta, move.beta, move.gamma)
        cache = (key, (norm.weight.detach().float() + 1.0).contiguous(), norm.bias.detach().float().contiguous(),
                 p, q, g, move.omega.detach().float().reshape(-1).contiguous(), tensors)
        move._decode_cache = cache
    return cache[1:7]


_current_device = getattr(torch._C, "_cuda_getDevice", torch.cuda.current_device)

try:   # the raw handle of the current stream without building a torch.cuda.Stream object
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:   # pragma: no cover - older / newer torch
    def _raw_stream(index):
        return torch.cuda.current_stream(index).cuda_stream


class _StepPlan:
    """Everything a single-token step passes to the C entry point, converted once: the ctypes
    argument list with the pointers of the parameters and of the running state, and a second count
    array (the step writes the bumped counts there from its one launch; the two arrays alternate).
    Valid for as long as the parameters (identity and version counters), the state tensors, the batch
    size, the dtype and the options stay the same; the caller rebuilds it otherwise (new generation,
    reordered beams, an optimiser step, ...)."""

    __slots__ = ("key", "fn", "args", "count_ptr", "count_cur", "count_alt", "keep", "params", "pver", "nkey", "ekey",
                 "dev")

    def __init__(self, key, fn, args, count_cur, count_alt, keep, params, pver, nkey, ekey, dev):
        self.key, self.fn, self.args, self.count_cur, self.count_alt, self.keep = key, fn, args, count_cur, count_alt, keep
        self.count_ptr = count_cur.data_ptr()
        self.params, self.pver, self.nkey, self.ekey, self.dev = params, pver, nkey, ekey, dev


def _param_tensors(norm, move):
    """The seven parameter tensors the step depends on, fetched from the modules' parameter dicts
    (several times cheaper than attribute access through nn.Module.__getattr__)."""
    np_, mp_ = norm._parameters, move._parameters
    return (np_['weight'], np_['bias'], mp_['alpha'], mp_['delta'], mp_['theta' if move.complex else 'beta'],
            mp_['gamma'], mp_['omega'])


def _decode_step(norm, move, x, incremental_state, activation, return_normed, _fresh_plan=False):
    """Single-token step (x: (B, 1, D)): one fused kernel, one launch, running state updated in place."""
    plan = move.__dict__.get("_step_plan")
    if plan is not None:
        nstate = incremental_state.get(plan.nkey)
        estate = incremental_state.get(plan.ekey)
        if nstate is not None and estate is not None:
            count, mean, var, h = nstate.get('prev_count'), nstate.get('prev_mean'), nstate.get('prev_var'), \
                estate.get('prev_state')
            ps = _param_tensors(norm, move)
            pp = plan.params
            if (mean is not None and h is not None and ps[0] is pp[0] and ps[1] is pp[1] and ps[2] is pp[2]
                    and ps[3] is pp[3] and ps[4] is pp[4] and ps[5] is pp[5] and ps[6] is pp[6]
                    and (ps[0]._version, ps[1]._version, ps[2]._version, ps[3]._version, ps[4]._version,
                         ps[5]._version, ps[6]._version) == plan.pver
                    and mean is plan.keep[6] and var is plan.keep[7] and h is plan.keep[8] and count is plan.count_cur
                    and plan.key == (x.shape[0], x.dtype, activation, return_normed, x.device.index)):
                args = plan.args
                y = torch.empty_like(x)
                args[0].value = x.data_ptr()
                args[1].value = y.data_ptr()
                xn = None
                if return_normed:
                    xn = torch.empty_like(x)
                    args[2].value = xn.data_ptr()
                # counts: read from the state's array, written to the other one, which becomes the state's
                alt = plan.count_alt
                args[6].value = plan.count_ptr
                args[7].value = alt.data_ptr()
                args[20].value = _raw_stream(plan.dev)
                if _current_device() == plan.dev:
                    rc = plan.fn(*args)
                else:
                    with torch.cuda.device(plan.dev):
                        rc = plan.fn(*args)
                if rc != 0:
                    from .. import _lib
                    _lib.check(rc, "tsn_ema_step")
                nstate['prev_count'] = alt
                plan.count_alt, plan.count_cur, plan.count_ptr = count, alt, args[7].value
                return (y, xn) if return_normed else y
    if _fresh_plan:
        raise RuntimeError("single-token step: a freshly built plan does not match its own inputs")
    return _decode_step_plan(norm, move, x, incremental_state, activation, return_normed)


def _decode_step_plan(norm, move, x, incremental_state, activation, return_normed):
    """Builds (or rebuilds) the plan of the single-token step, then takes the step through it."""
    import ctypes
    from .. import _lib
    bsz, _, dim = x.shape
    nkey = norm._get_full_incremental_state_key("norm_state")
    ekey = move._get_full_incremental_state_key("ema_state")
    nstate = incremental_state.get(nkey)
    estate = incremental_state.get(ekey)
    if nstate is None or estate is None or 'prev_mean' not in nstate or estate.get('prev_state') is None:
        nstate, estate = _seed_decode_state(norm, move, bsz, dim, x.device, incremental_state)
    count, mean, var, h = nstate['prev_count'], nstate['prev_mean'], nstate['prev_var'], estate['prev_state']
    sdtype = torch.complex64 if move.complex else torch.float32
    if (mean.dtype != torch.float32 or not mean.is_contiguous() or var.dtype != torch.float32
            or not var.is_contiguous() or h.dtype != sdtype or not h.is_contiguous()
            or count.dtype != torch.int64 or not count.is_contiguous()):
        nstate['prev_mean'], nstate['prev_var'] = mean.float().contiguous(), var.float().contiguous()
        nstate['prev_count'] = count.long().contiguous()
        estate['prev_state'] = h.to(sdtype).contiguous()
        count, mean, var, h = nstate['prev_count'], nstate['prev_mean'], nstate['prev_var'], estate['prev_state']
    gamma, beta, p, q, g, omega = _fp32_params(norm, move)
    params = _param_tensors(norm, move)
    pver = tuple(t._version for t in params)
    # (the state tensors themselves are compared by identity: keep[6:9] and count_cur)
    key = (bsz, x.dtype, activation, return_normed, x.device.index)
    lib = _lib.lib()
    fn = lib.mega_tsn_cema_step if move.complex else lib.mega_tsn_ema_step
    vp, ci = ctypes.c_void_p, ctypes.c_int
    count_alt = torch.empty_like(count)
    # x, y, xn_out, dtype, B, D, count, count_next, mean, var, gamma, beta, eps, p, q, g, omega, N, h, flags, stream
    args = [vp(0), vp(0), vp(None), ci(ops._dt(x)), ci(bsz), ci(dim), vp(count.data_ptr()),
            vp(count_alt.data_ptr()), vp(mean.data_ptr()), vp(var.data_ptr()), vp(gamma.data_ptr()),
            vp(beta.data_ptr()), ctypes.c_double(norm.eps), vp(p.data_ptr()), vp(q.data_ptr()), vp(g.data_ptr()),
            vp(omega.data_ptr()), ci(p.shape[1]), vp(h.data_ptr()),
            ctypes.c_uint(ops.EMA_SILU if activation == 'silu' else 0), vp(0)]
    move._step_plan = _StepPlan(key, fn, args, count, count_alt, (gamma, beta, p, q, g, omega, mean, var, h),
                                params, pver, nkey, ekey, x.device.index)
    return _decode_step(norm, move, x, incremental_state, activation, return_normed, _fresh_plan=True)


def _seed_decode_state(norm, move, bsz, dim, device, incremental_state):
    """First single-token call of a generation: running statistics from the priors (fresh tensors,
    never views of the parameters: the step updates them in place) and zero pole states."""
    nstate = norm._get_input_buffer(incremental_state)
    if 'prev_mean' not in nstate:
        count, mean, var, nstate = norm.initial_statistics(bsz, incremental_state)
        nstate['prev_count'], nstate['prev_mean'], nstate['prev_var'] = count.clone(), mean.clone(), var.clone()
        norm._set_input_buffer(incremental_state, nstate)
    estate = move._get_input_buffer(incremental_state)
    if estate.get('prev_state') is None:
        sdtype = torch.complex64 if move.complex else torch.float32
        estate['prev_state'] = torch.zeros(bsz, dim, move.ndim, device=device, dtype=sdtype)
    move._set_input_buffer(incremental_state, estate)
    return nstate, estate
