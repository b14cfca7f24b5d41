"""Operator level of the package: torch tensors in, torch tensors out, every op a call into
libmega_b200.so on the current CUDA stream.

The functions mirror the operator surface the reference's Python wrappers expect from
``fairseq.mega2_extension.ops`` (fairseq/modules/fused_ops/*.py,
fairseq/modules/norm_layer/*.py), with the FFT convolution, its bias and the hidden-state
update folded into one ``ema_forward``.  Outputs are allocated here with torch (device
memory plumbing); the library itself allocates nothing.
"""
from typing import Optional, Tuple

import torch

from . import _lib

F32, BF16, F16 = 0, 1, 2
EMA_BIDIRECTIONAL, EMA_NO_SHIFT, EMA_SILU = 1, 2, 4
_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


def _dt(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError("mega_b200 supports float32, bfloat16 and float16 activations, got %s" % t.dtype)


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("mega_b200 ops run on CUDA tensors only (there is no CPU fallback)")


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def _f32c(t):
    """fp32, contiguous (parameters, statistics, states are tiny)."""
    if t is None:
        return None
    t = t.detach()
    if t.dtype != torch.float32:
        t = t.float()
    return t.contiguous()


def _mask_u8(mask, bsz, length):
    if mask is None:
        return None
    if mask.shape != (bsz, length):
        raise ValueError("padding_mask must be (batch, length) = (%d, %d), got %s" % (bsz, length, tuple(mask.shape)))
    if mask.dtype == torch.bool:
        return mask.contiguous().view(torch.uint8)
    return (mask != 0).contiguous().view(torch.uint8)


# ----------------------------------------------------------------------------- EMA
def ema_coeffs(alpha, delta, beta, gamma):
    """(p, q, gamma_hat), each (K, N) fp32 — MultiHeadEMA._calc_coeffs."""
    _cuda(alpha, delta, beta, gamma)
    k, n = alpha.shape[0], alpha.shape[1]
    dt = alpha.dtype
    args = [t.detach().to(dt).contiguous() for t in (alpha, delta, beta, gamma)]
    p = torch.empty(k, n, device=alpha.device, dtype=torch.float32)
    q = torch.empty_like(p)
    g = torch.empty_like(p)
    with torch.cuda.device(alpha.device):
        _lib.check(_lib.lib().mega_ema_coeffs(*[a.data_ptr() for a in args], _dt(args[0]), k, n,
                                              p.data_ptr(), q.data_ptr(), g.data_ptr(), _stream()), "ema_coeffs")
    return p, q, g


def ema_kernel(p, q, g, length):
    """k (K, L) fp32: the materialised convolution kernel."""
    _cuda(p, q, g)
    p, q, g = _f32c(p), _f32c(q), _f32c(g)
    k, n = p.shape
    out = torch.empty(k, length, device=p.device, dtype=torch.float32)
    with torch.cuda.device(p.device):
        _lib.check(_lib.lib().mega_ema_kernel(p.data_ptr(), q.data_ptr(), g.data_ptr(), k, n, length,
                                              out.data_ptr(), _stream()), "ema_kernel")
    return out


def ema_bias(q, g, h, length):
    """(B, D, L) fp32 output term of a carried state h (B, D, N)."""
    _cuda(q, g, h)
    q, g, h = _f32c(q), _f32c(g), _f32c(h)
    b, d, n = h.shape
    out = torch.empty(b, d, length, device=h.device, dtype=torch.float32)
    with torch.cuda.device(h.device):
        _lib.check(_lib.lib().mega_ema_bias(q.data_ptr(), g.data_ptr(), h.data_ptr(), b, d, n, length,
                                            out.data_ptr(), _stream()), "ema_bias")
    return out


def _trunc(truncation):
    return 0 if truncation is None or truncation < 1 else int(truncation)


def ema_forward(x, p, q, g, omega, padding_mask=None, h_in=None, want_state=False,
                bidirectional=False, shift=True, truncation=None, silu=False, out=None):
    """EMA layer forward on x (B, D, L) with any strides (a transposed view of (B, L, D)
    memory is addressed in place).  Returns y shaped and strided like x, and the new state
    (B, D, N) when ``want_state``."""
    _cuda(x, p, q, g, omega, padding_mask, h_in)
    bsz, dim, length = x.shape
    p, q, g, omega = _f32c(p), _f32c(q), _f32c(g), _f32c(omega)
    n = p.shape[1]
    if p.shape[0] != (2 * dim if bidirectional else dim):
        raise ValueError("coefficient rows %d do not match embed_dim %d" % (p.shape[0], dim))
    mask = _mask_u8(padding_mask, bsz, length)
    if out is None:
        out = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device) \
            if _dense(x) else torch.empty_like(x, memory_format=torch.contiguous_format)
    h_in = _f32c(h_in)
    h_out = torch.empty(bsz, dim, n, device=x.device, dtype=torch.float32) if want_state else None
    flags = (EMA_BIDIRECTIONAL if bidirectional else 0) | (0 if shift else EMA_NO_SHIFT) | (EMA_SILU if silu else 0)
    trunc = 0 if truncation is None or truncation < 1 else int(truncation)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_ema_fwd(
            x.data_ptr(), out.data_ptr(), _dt(x), bsz, dim, length, *x.stride(), *out.stride(),
            p.data_ptr(), q.data_ptr(), g.data_ptr(), omega.data_ptr(), n,
            _ptr(mask), _ptr(h_in), _ptr(h_out), flags, trunc, _stream()), "ema_fwd")
    return (out, h_out) if want_state else out


def _dense(t):
    """True when t's strides describe a permutation of a contiguous block."""
    exp = 1
    for size, stride in sorted(zip(t.shape, t.stride()), key=lambda v: v[1]):
        if size == 1:
            continue
        if stride != exp:
            return False
        exp *= size
    return True


def ema_step(x, p, q, g, omega, h=None, silu=False):
    """One decode step.  x (B, D) or (B, D, 1); returns (y like x, h' (B, D, N))."""
    _cuda(x, p, q, g, omega, h)
    shape = x.shape
    x2 = x.reshape(shape[0], shape[1]).contiguous()
    bsz, dim = x2.shape
    p, q, g, omega = _f32c(p), _f32c(q), _f32c(g), _f32c(omega)
    n = p.shape[1]
    h = _f32c(h)
    h_out = torch.empty(bsz, dim, n, device=x.device, dtype=torch.float32)
    y = torch.empty_like(x2)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_ema_step(x2.data_ptr(), y.data_ptr(), _dt(x2), bsz, dim, p.data_ptr(),
                                            q.data_ptr(), g.data_ptr(), omega.data_ptr(), n, _ptr(h),
                                            h_out.data_ptr(), EMA_SILU if silu else 0, _stream()), "ema_step")
    return y.view(shape), h_out


# --------------------------------------------------------------------------- norms
def timestep_norm_fwd(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask=None,
                      eps=1e-5, num_groups=None, out=None):
    """x (B, L, D) any strides -> (y, count (B) int64, mean, var (B, G) fp32).
    gamma is the effective scale (module weight + 1)."""
    _cuda(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask)
    bsz, length, dim = x.shape
    groups = dim if num_groups is None else int(num_groups)
    prev_count = prev_count.detach().to(torch.int64).contiguous()
    prev_mean, prev_var = _f32c(prev_mean), _f32c(prev_var)
    if prev_mean.shape != (bsz, groups) or prev_var.shape != (bsz, groups):
        raise ValueError("prev_mean/prev_var must be (batch, groups) = (%d, %d)" % (bsz, groups))
    gamma, beta = _f32c(gamma), _f32c(beta)
    mask = _mask_u8(padding_mask, bsz, length)
    if out is None:
        out = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device) \
            if _dense(x) else torch.empty_like(x, memory_format=torch.contiguous_format)
    count = torch.empty(bsz, device=x.device, dtype=torch.int64)
    mean = torch.empty(bsz, groups, device=x.device, dtype=torch.float32)
    var = torch.empty_like(mean)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_timestep_norm_fwd(
            x.data_ptr(), out.data_ptr(), _dt(x), bsz, length, dim, *x.stride(), *out.stride(),
            prev_count.data_ptr(), prev_mean.data_ptr(), prev_var.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
            _ptr(mask), groups, float(eps), count.data_ptr(), mean.data_ptr(), var.data_ptr(), _stream()),
            "timestep_norm_fwd")
    return out, count, mean, var


def sequence_norm_fwd(x, gamma, beta, padding_mask=None, eps=1e-5, length_last=True, num_groups=None, out=None):
    """x (B, D, L) when ``length_last`` else (B, L, D); any strides.
    Returns (y, count (B) int64, mean, rstd (B, G) fp32)."""
    _cuda(x, gamma, beta, padding_mask)
    if length_last:
        bsz, dim, length = x.shape
    else:
        bsz, length, dim = x.shape
    groups = dim if num_groups is None else int(num_groups)
    gamma, beta = _f32c(gamma), _f32c(beta)
    mask = _mask_u8(padding_mask, bsz, length)
    if out is None:
        out = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device) \
            if _dense(x) else torch.empty_like(x, memory_format=torch.contiguous_format)
    xs, ys = x.stride(), out.stride()
    if not length_last:
        xs = (xs[0], xs[2], xs[1])
        ys = (ys[0], ys[2], ys[1])
    count = torch.empty(bsz, device=x.device, dtype=torch.int64)
    mean = torch.empty(bsz, groups, device=x.device, dtype=torch.float32)
    rstd = torch.empty_like(mean)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_sequence_norm_fwd(
            x.data_ptr(), out.data_ptr(), _dt(x), bsz, dim, length, *xs, *ys, gamma.data_ptr(), beta.data_ptr(),
            _ptr(mask), groups, float(eps), count.data_ptr(), mean.data_ptr(), rstd.data_ptr(), _stream()),
            "sequence_norm_fwd")
    return out, count, mean, rstd


def tsn_ema_forward(x, prev_count, prev_mean, prev_var, gamma, beta, eps, p, q, g, omega,
                    padding_mask=None, h_in=None, want_state=False, silu=False, want_normed=False,
                    complex_poles=False):
    """Fused per-feature TimestepNorm -> causal EMA on x (B, L, D).
    Returns dict(y, count, mean, var[, h][, xn]); y and xn are (B, L, D) like x.
    ``complex_poles``: q, g (and the states) are complex64, the layer is MultiHeadComplexEMA's."""
    _cuda(x, prev_count, prev_mean, prev_var, gamma, beta, p, q, g, omega, padding_mask, h_in)
    bsz, length, dim = x.shape
    prev_count = prev_count.detach().to(torch.int64).contiguous()
    prev_mean, prev_var, gamma, beta = _f32c(prev_mean), _f32c(prev_var), _f32c(gamma), _f32c(beta)
    if complex_poles:
        p, q, g, omega, h_in = _f32c(p), _c64(q), _c64(g), _f32c(omega).reshape(-1), _c64(h_in)
    else:
        p, q, g, omega = _f32c(p), _f32c(q), _f32c(g), _f32c(omega)
    n = p.shape[1]
    mask = _mask_u8(padding_mask, bsz, length)
    y = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device) \
        if _dense(x) else torch.empty_like(x, memory_format=torch.contiguous_format)
    xn = torch.empty_strided(y.shape, y.stride(), dtype=x.dtype, device=x.device) if want_normed else None
    count = torch.empty(bsz, device=x.device, dtype=torch.int64)
    mean = torch.empty(bsz, dim, device=x.device, dtype=torch.float32)
    var = torch.empty_like(mean)
    if complex_poles:
        h_out = torch.empty(bsz, dim, n, 2, device=x.device, dtype=torch.float32) if want_state else None
        entry, what = _lib.lib().mega_tsn_cema_fwd, "tsn_cema_fwd"
    else:
        h_in = _f32c(h_in)
        h_out = torch.empty(bsz, dim, n, device=x.device, dtype=torch.float32) if want_state else None
        entry, what = _lib.lib().mega_tsn_ema_fwd, "tsn_ema_fwd"
    with torch.cuda.device(x.device):
        _lib.check(entry(
            x.data_ptr(), y.data_ptr(), _ptr(xn), _dt(x), bsz, length, dim, *x.stride(), *y.stride(),
            prev_count.data_ptr(), prev_mean.data_ptr(), prev_var.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
            float(eps), count.data_ptr(), mean.data_ptr(), var.data_ptr(),
            p.data_ptr(), q.data_ptr(), g.data_ptr(), omega.data_ptr(), n, _ptr(mask), _ptr(h_in), _ptr(h_out),
            EMA_SILU if silu else 0, _stream()), what)
    res = {"y": y, "count": count, "mean": mean, "var": var}
    if want_state:
        res["h"] = torch.view_as_complex(h_out) if complex_poles else h_out
    if want_normed:
        res["xn"] = xn
    return res


def sqn_ema_forward(x, gamma, beta, eps, p, q, g, omega, padding_mask=None, bidirectional=False, shift=True,
                    silu=False):
    """Fused per-channel SequenceNorm -> EMA on x (B, D, L) with contiguous length.  Returns y, or
    None when the call is outside the fused kernel's envelope (the caller then runs the two ops)."""
    _cuda(x, gamma, beta, p, q, g, omega, padding_mask)
    bsz, dim, length = x.shape
    if x.stride(2) != 1:
        return None
    gamma, beta, p, q, g, omega = _f32c(gamma), _f32c(beta), _f32c(p), _f32c(q), _f32c(g), _f32c(omega)
    mask = _mask_u8(padding_mask, bsz, length)
    y = torch.empty_like(x, memory_format=torch.contiguous_format)
    flags = (EMA_BIDIRECTIONAL if bidirectional else 0) | (0 if shift else EMA_NO_SHIFT) | (EMA_SILU if silu else 0)
    with torch.cuda.device(x.device):
        rc = _lib.lib().mega_sqn_ema_fwd(x.data_ptr(), y.data_ptr(), _dt(x), bsz, dim, length, *x.stride(), *y.stride(),
                                         gamma.data_ptr(), beta.data_ptr(), float(eps), None, None, None,
                                         p.data_ptr(), q.data_ptr(), g.data_ptr(), omega.data_ptr(), p.shape[1],
                                         _ptr(mask), flags, _stream())
    if rc == 7:  # MEGA_ERR_UNSUPPORTED: outside the envelope
        return None
    _lib.check(rc, "sqn_ema_fwd")
    return y


def tsn_ema_step_(x, y, count, mean, var, gamma, beta, eps, p, q, g, omega, h, silu=False, xn_out=None,
                  count_next=None):
    """In-place decode step: x, y (B, D) contiguous; count (B) int64, mean/var (B, D) fp32 and
    h (B, D, N) fp32 are UPDATED IN PLACE (pass count=None to skip the norm).  All parameter
    tensors must already be fp32 and contiguous: nothing is converted or allocated here.
    With ``count_next`` (a second (B) int64 tensor) the bumped counts go there from the same launch
    and ``count`` stays as it was; without it a second launch bumps ``count`` in place."""
    bsz, dim = x.shape
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_tsn_ema_step(
            x.data_ptr(), y.data_ptr(), _ptr(xn_out), _dt(x), bsz, dim, _ptr(count), _ptr(count_next), _ptr(mean),
            _ptr(var),
            _ptr(gamma), _ptr(beta), float(eps), p.data_ptr(), q.data_ptr(), g.data_ptr(), omega.data_ptr(),
            p.shape[1], h.data_ptr(), EMA_SILU if silu else 0, _stream()), "tsn_ema_step")
    return y


def tsn_cema_step_(x, y, count, mean, var, gamma, beta, eps, p, q, g, omega, h, silu=False, xn_out=None,
                   count_next=None):
    """tsn_ema_step_ for the complex layer: q, g (K, N, 2) and h (B, D, N, 2) are fp32 views of the
    complex64 tensors; everything is updated in place, nothing is converted or allocated."""
    bsz, dim = x.shape
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_tsn_cema_step(
            x.data_ptr(), y.data_ptr(), _ptr(xn_out), _dt(x), bsz, dim, count.data_ptr(), _ptr(count_next),
            mean.data_ptr(),
            var.data_ptr(), gamma.data_ptr(), beta.data_ptr(), float(eps), p.data_ptr(), q.data_ptr(), g.data_ptr(),
            omega.data_ptr(), p.shape[1], h.data_ptr(), EMA_SILU if silu else 0, _stream()), "tsn_cema_step")
    return y


# --------------------------------------------------------------------------- gates
def _rows(t):
    """View t (..., cols) as `rows` rows of `cols` elements with one row pitch; copies only
    when the memory is not a uniform-pitch row-major matrix (e.g. after a transpose)."""
    cols = t.shape[-1]
    if t.dim() == 1:
        t = t.unsqueeze(0)
    ok = t.stride(-1) == 1 or cols == 1
    ld = t.stride(-2) if t.shape[-2] > 1 else max(cols, t.stride(-2))
    exp = ld
    for size, stride in zip(reversed(t.shape[:-1]), reversed(t.stride()[:-1])):
        if size != 1 and stride != exp:
            ok = False
        exp *= size
    if not ok or ld < cols:
        t = t.contiguous()
        ld = cols
    return t, t.numel() // cols, cols, ld


def gate_silu(a, b=None):
    """silu(a [+ b]) elementwise; a, b may be column slices of wider row-major matrices."""
    _cuda(a, b)
    a_, rows, cols, lda = _rows(a)
    ldb, b_ = 0, None
    if b is not None:
        b_, _, _, ldb = _rows(b)
    y = torch.empty(a.shape, dtype=a.dtype, device=a.device)
    with torch.cuda.device(a.device):
        _lib.check(_lib.lib().mega_gate_silu(a_.data_ptr(), lda, _ptr(b_), ldb, y.data_ptr(), cols, _dt(a),
                                             rows, cols, _stream()), "gate_silu")
    return y


def gate_mul_silu(a, r):
    """a * silu(r)."""
    _cuda(a, r)
    a_, rows, cols, lda = _rows(a)
    r_, _, _, ldr = _rows(r)
    y = torch.empty(a.shape, dtype=a.dtype, device=a.device)
    with torch.cuda.device(a.device):
        _lib.check(_lib.lib().mega_gate_mul_silu(a_.data_ptr(), lda, r_.data_ptr(), ldr, y.data_ptr(), cols,
                                                 _dt(a), rows, cols, _stream()), "gate_mul_silu")
    return y


def gate_output(residual, u, hx, h_lin):
    """residual + sigmoid(u) * (silu(hx + h_lin) - residual); u is the PRE-sigmoid gate."""
    _cuda(residual, u, hx, h_lin)
    r_, rows, cols, ldr = _rows(residual)
    u_, _, _, ldu = _rows(u)
    x_, _, _, ldx = _rows(hx)
    h_, _, _, ldh = _rows(h_lin)
    y = torch.empty(residual.shape, dtype=residual.dtype, device=residual.device)
    with torch.cuda.device(residual.device):
        _lib.check(_lib.lib().mega_gate_output(r_.data_ptr(), ldr, u_.data_ptr(), ldu, x_.data_ptr(), ldx,
                                               h_.data_ptr(), ldh, y.data_ptr(), cols, _dt(residual), rows, cols,
                                               _stream()), "gate_output")
    return y


def gate_qk(z, gamma, beta, eps=1e-5):
    """Query and key of the Mega block from the shared representation z (..., S):
    zn = z / max(||z||_2, eps); returns (zn * (gamma[0] + 1) + beta[0], zn * (gamma[1] + 1) + beta[1]).
    gamma, beta are (2, S); z may be a column slice of the mx_proj output.
    Mirrors fairseq/modules/moving_average_gated_attention.py:324-328."""
    _cuda(z, gamma, beta)
    z_, rows, cols, ldz = _rows(z)
    g = gamma.detach().to(torch.float32).contiguous()
    b = beta.detach().to(torch.float32).contiguous()
    if g.shape != (2, cols) or b.shape != (2, cols):
        raise ValueError("gate_qk: gamma and beta must be (2, %d)" % cols)
    q = torch.empty(z.shape, dtype=z.dtype, device=z.device)
    k = torch.empty(z.shape, dtype=z.dtype, device=z.device)
    with torch.cuda.device(z.device):
        _lib.check(_lib.lib().mega_gate_qk(z_.data_ptr(), ldz, g.data_ptr(), b.data_ptr(), q.data_ptr(), cols,
                                           k.data_ptr(), cols, _dt(z), rows, cols, float(eps), _stream()),
                   "gate_qk")
    return q, k


def gate_qk_rotary(z, gamma, beta, rot, period, q_offset=0, eps=1e-5):
    """gate_qk with the block's rotary embedding applied to both results in the same kernel.
    rot: complex64 (positions, S / 2) unit phasors (the table RotaryEmbedding keeps) or their float32
    (positions, S / 2, 2) view; row r of the flattened z is position r % period (+ q_offset for the query).
    Returns (q, k) in z's dtype."""
    _cuda(z, gamma, beta, rot)
    z_, rows, cols, ldz = _rows(z)
    g = gamma.detach().to(torch.float32).contiguous()
    b = beta.detach().to(torch.float32).contiguous()
    if g.shape != (2, cols) or b.shape != (2, cols):
        raise ValueError("gate_qk_rotary: gamma and beta must be (2, %d)" % cols)
    r = torch.view_as_real(rot) if rot.is_complex() else rot
    r = r.to(torch.float32).contiguous()
    if r.dim() != 3 or r.shape[1] * 2 != cols or r.shape[2] != 2:
        raise ValueError("gate_qk_rotary: rot must be (positions, %d) complex or (positions, %d, 2) float" % (cols // 2, cols // 2))
    q = torch.empty(z.shape, dtype=z.dtype, device=z.device)
    k = torch.empty(z.shape, dtype=z.dtype, device=z.device)
    with torch.cuda.device(z.device):
        _lib.check(_lib.lib().mega_gate_qk_rotary(z_.data_ptr(), ldz, g.data_ptr(), b.data_ptr(), r.data_ptr(),
                                                  r.shape[0], int(period), int(q_offset), q.data_ptr(), cols,
                                                  k.data_ptr(), cols, _dt(z), rows, cols, float(eps), _stream()),
                   "gate_qk_rotary")
    return q, k


# ------------------------------------------------------------------------ training
def _like(x):
    return torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device) \
        if _dense(x) else torch.empty_like(x, memory_format=torch.contiguous_format)


def timestep_norm_fwd_train(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask=None, eps=1e-5,
                            num_groups=None):
    """timestep_norm_fwd that also returns what the backward needs, like the reference op:
    (y, count, mean, var, cummean, cumrstd, group_mean); the saves are (B, L, G) fp32 and
    group_mean is None for the per-feature form."""
    _cuda(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask)
    bsz, length, dim = x.shape
    groups = dim if num_groups is None else int(num_groups)
    prev_count = prev_count.detach().to(torch.int64).contiguous()
    prev_mean, prev_var, gamma, beta = _f32c(prev_mean), _f32c(prev_var), _f32c(gamma), _f32c(beta)
    if prev_mean.shape != (bsz, groups) or prev_var.shape != (bsz, groups):
        raise ValueError("prev_mean/prev_var must be (batch, groups) = (%d, %d)" % (bsz, groups))
    mask = _mask_u8(padding_mask, bsz, length)
    out = _like(x)
    count = torch.empty(bsz, device=x.device, dtype=torch.int64)
    mean = torch.empty(bsz, groups, device=x.device, dtype=torch.float32)
    var = torch.empty_like(mean)
    cummean = torch.empty(bsz, length, groups, device=x.device, dtype=torch.float32)
    cumrstd = torch.empty_like(cummean)
    group_mean = torch.empty_like(cummean) if groups != dim else None
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_timestep_norm_fwd_train(
            x.data_ptr(), out.data_ptr(), _dt(x), bsz, length, dim, *x.stride(), *out.stride(),
            prev_count.data_ptr(), prev_mean.data_ptr(), prev_var.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
            _ptr(mask), groups, float(eps), count.data_ptr(), mean.data_ptr(), var.data_ptr(),
            cummean.data_ptr(), cumrstd.data_ptr(), _ptr(group_mean), _stream()), "timestep_norm_fwd_train")
    return out, count, mean, var, cummean, cumrstd, group_mean


def timestep_norm_bwd(dy, dmean, dvar, x, prev_mean, count, cummean, cumrstd, group_mean, gamma,
                      padding_mask=None, num_groups=None):
    """Gradients of TimestepNorm: (dx, dprev_mean, dprev_var, dgamma, dbeta); the argument order
    follows the reference's timestep_norm_bwd / group_timestep_norm_bwd."""
    _cuda(dy, dmean, dvar, x, prev_mean, count, cummean, cumrstd, group_mean, gamma, padding_mask)
    bsz, length, dim = x.shape
    groups = dim if num_groups is None else int(num_groups)
    if dy.dtype != x.dtype:
        dy = dy.to(x.dtype)
    dmean, dvar, prev_mean, gamma = _f32c(dmean), _f32c(dvar), _f32c(prev_mean), _f32c(gamma)
    mask = _mask_u8(padding_mask, bsz, length)
    dx = _like(x)
    dpm = torch.empty(bsz, groups, device=x.device, dtype=torch.float32)
    dpv = torch.empty_like(dpm)
    dgamma = torch.empty(dim, device=x.device, dtype=torch.float32)
    dbeta = torch.empty_like(dgamma)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_timestep_norm_bwd(
            dy.data_ptr(), x.data_ptr(), dx.data_ptr(), _dt(x), bsz, length, dim, *dy.stride(), *x.stride(),
            *dx.stride(), _ptr(dmean), _ptr(dvar), prev_mean.data_ptr(), count.data_ptr(), cummean.data_ptr(),
            cumrstd.data_ptr(), _ptr(group_mean), gamma.data_ptr(), _ptr(mask), groups, dpm.data_ptr(),
            dpv.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), _stream()), "timestep_norm_bwd")
    return dx, dpm, dpv, dgamma, dbeta


def sequence_norm_bwd(dy, x, count, mean, rstd, gamma, padding_mask=None, length_last=True, num_groups=None):
    """Gradients of SequenceNorm (per channel, or per group with ``num_groups``): (dx, dgamma, dbeta)."""
    _cuda(dy, x, count, mean, rstd, gamma, padding_mask)
    if length_last:
        bsz, dim, length = x.shape
    else:
        bsz, length, dim = x.shape
    if dy.dtype != x.dtype:
        dy = dy.to(x.dtype)
    mean, rstd, gamma = _f32c(mean), _f32c(rstd), _f32c(gamma)
    mask = _mask_u8(padding_mask, bsz, length)
    dx = _like(x)
    gs, xs, ds = dy.stride(), x.stride(), dx.stride()
    if not length_last:
        gs, xs, ds = (gs[0], gs[2], gs[1]), (xs[0], xs[2], xs[1]), (ds[0], ds[2], ds[1])
    dgamma = torch.empty(dim, device=x.device, dtype=torch.float32)
    dbeta = torch.empty_like(dgamma)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_sequence_norm_bwd(
            dy.data_ptr(), x.data_ptr(), dx.data_ptr(), _dt(x), bsz, dim, length, *gs, *xs, *ds,
            count.data_ptr(), mean.data_ptr(), rstd.data_ptr(), gamma.data_ptr(), _ptr(mask),
            dim if num_groups is None else int(num_groups), dgamma.data_ptr(), dbeta.data_ptr(), _stream()),
            "sequence_norm_bwd")
    return dx, dgamma, dbeta


def ema_backward(dy, x, p, q, g, omega, padding_mask=None, h_in=None, dh_out=None, bidirectional=False,
                 shift=True, want_dh_in=False, truncation=None):
    """Gradients of ema_forward (no activation) on (B, D, L) tensors with any strides:
    (dx, dp, dq, dgamma_hat, domega, dh_in or None).  ``truncation``: kernel support of a
    bidirectional layer, as in the forward."""
    _cuda(dy, x, p, q, g, omega, padding_mask, h_in, dh_out)
    bsz, dim, length = x.shape
    if dy.dtype != x.dtype:
        dy = dy.to(x.dtype)
    p, q, g, omega, h_in, dh_out = _f32c(p), _f32c(q), _f32c(g), _f32c(omega), _f32c(h_in), _f32c(dh_out)
    n = p.shape[1]
    mask = _mask_u8(padding_mask, bsz, length)
    dx = _like(x)
    dp = torch.empty_like(p)
    dq = torch.empty_like(p)
    dg = torch.empty_like(p)
    dom = torch.empty(dim, device=x.device, dtype=torch.float32)
    dh_in = torch.empty(bsz, dim, n, device=x.device, dtype=torch.float32) if want_dh_in else None
    flags = (EMA_BIDIRECTIONAL if bidirectional else 0) | (0 if shift else EMA_NO_SHIFT)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_ema_bwd(
            dy.data_ptr(), x.data_ptr(), dx.data_ptr(), _dt(x), bsz, dim, length, *dy.stride(), *x.stride(),
            *dx.stride(), p.data_ptr(), q.data_ptr(), g.data_ptr(), omega.data_ptr(), n, _ptr(mask), _ptr(h_in),
            _ptr(dh_out), flags, _trunc(truncation), dp.data_ptr(), dq.data_ptr(), dg.data_ptr(), dom.data_ptr(),
            _ptr(dh_in),
            _stream()), "ema_bwd")
    return dx, dp, dq, dg, dom, dh_in


def ema_coeffs_bwd(alpha, delta, beta, dp, dq, dg):
    """(dalpha, ddelta, dbeta (K, N, 1), dgamma (K, N)) from the coefficient gradients."""
    _cuda(alpha, delta, beta, dp, dq, dg)
    k, n = alpha.shape[0], alpha.shape[1]
    a, d, b = _f32c(alpha).view(k, n), _f32c(delta).view(k, n), _f32c(beta).view(k, n)
    dp, dq, dg = _f32c(dp), _f32c(dq), _f32c(dg)
    outs = [torch.empty(k, n, device=alpha.device, dtype=torch.float32) for _ in range(4)]
    with torch.cuda.device(alpha.device):
        _lib.check(_lib.lib().mega_ema_coeffs_bwd(a.data_ptr(), d.data_ptr(), b.data_ptr(), dp.data_ptr(),
                                                  dq.data_ptr(), dg.data_ptr(), k, n,
                                                  *[o.data_ptr() for o in outs], _stream()), "ema_coeffs_bwd")
    return outs[0].unsqueeze(-1), outs[1].unsqueeze(-1), outs[2].unsqueeze(-1), outs[3]


# --------------------------------------------------------------------- complex EMA
def cema_coeffs(alpha, delta, theta, gamma):
    """(p (K, N) fp32, q (K, N) complex64, gamma_hat (K, N) complex64) of the complex EMA."""
    _cuda(alpha, delta, theta, gamma)
    k, n = alpha.shape[0], alpha.shape[1]
    dt = alpha.dtype
    args = [t.detach().to(dt).contiguous() for t in (alpha, delta, theta, gamma)]
    p = torch.empty(k, n, device=alpha.device, dtype=torch.float32)
    q = torch.empty(k, n, 2, device=alpha.device, dtype=torch.float32)
    g = torch.empty_like(q)
    with torch.cuda.device(alpha.device):
        _lib.check(_lib.lib().mega_cema_coeffs(*[a.data_ptr() for a in args], _dt(args[0]), k, n,
                                               p.data_ptr(), q.data_ptr(), g.data_ptr(), _stream()), "cema_coeffs")
    return p, torch.view_as_complex(q), torch.view_as_complex(g)


def _c64(t):
    """complex64 contiguous tensor -> its interleaved float view (no copy when already so)."""
    if t is None:
        return None
    t = t.detach()
    if not t.is_complex():
        t = t.to(torch.complex64)
    elif t.dtype != torch.complex64:
        t = t.to(torch.complex64)
    return torch.view_as_real(t.contiguous())


def cema_kernel(p, q, g, length):
    """k (K, L) fp32 = Re(sum_n p gamma_hat q^l)."""
    _cuda(p, q, g)
    p, q, g = _f32c(p), _c64(q), _c64(g)
    k, n = p.shape
    out = torch.empty(k, length, device=p.device, dtype=torch.float32)
    with torch.cuda.device(p.device):
        _lib.check(_lib.lib().mega_cema_kernel(p.data_ptr(), q.data_ptr(), g.data_ptr(), k, n, length,
                                               out.data_ptr(), _stream()), "cema_kernel")
    return out


def cema_forward(x, p, q, g, omega, padding_mask=None, h_in=None, want_state=False, bidirectional=False,
                 shift=True, truncation=None, silu=False):
    """Complex EMA layer forward on x (B, D, L) with any strides; q, g complex64 (K, N); the state
    is complex64 (B, D, N).  Returns y like x, and the new state when ``want_state``."""
    _cuda(x, p, q, g, omega, padding_mask, h_in)
    bsz, dim, length = x.shape
    p, q, g, omega = _f32c(p), _c64(q), _c64(g), _f32c(omega).reshape(-1)
    n = p.shape[1]
    if p.shape[0] != (2 * dim if bidirectional else dim):
        raise ValueError("coefficient rows %d do not match embed_dim %d" % (p.shape[0], dim))
    mask = _mask_u8(padding_mask, bsz, length)
    out = _like(x)
    h_in = _c64(h_in)
    h_out = torch.empty(bsz, dim, n, 2, device=x.device, dtype=torch.float32) if want_state else None
    flags = (EMA_BIDIRECTIONAL if bidirectional else 0) | (0 if shift else EMA_NO_SHIFT) | (EMA_SILU if silu else 0)
    trunc = 0 if truncation is None or truncation < 1 else int(truncation)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_cema_fwd(
            x.data_ptr(), out.data_ptr(), _dt(x), bsz, dim, length, *x.stride(), *out.stride(),
            p.data_ptr(), q.data_ptr(), g.data_ptr(), omega.data_ptr(), n,
            _ptr(mask), _ptr(h_in), _ptr(h_out), flags, trunc, _stream()), "cema_fwd")
    return (out, torch.view_as_complex(h_out)) if want_state else out


def cema_step(x, p, q, g, omega, h=None, silu=False):
    """One decode step.  x (B, D) or (B, D, 1); returns (y like x, h' (B, D, N) complex64)."""
    _cuda(x, p, q, g, omega, h)
    shape = x.shape
    x2 = x.reshape(shape[0], shape[1]).contiguous()
    bsz, dim = x2.shape
    p, q, g, omega = _f32c(p), _c64(q), _c64(g), _f32c(omega).reshape(-1)
    n = p.shape[1]
    h = _c64(h)
    h_out = torch.empty(bsz, dim, n, 2, device=x.device, dtype=torch.float32)
    y = torch.empty_like(x2)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_cema_step(x2.data_ptr(), y.data_ptr(), _dt(x2), bsz, dim, p.data_ptr(),
                                             q.data_ptr(), g.data_ptr(), omega.data_ptr(), n, _ptr(h),
                                             h_out.data_ptr(), EMA_SILU if silu else 0, _stream()), "cema_step")
    return y.view(shape), torch.view_as_complex(h_out)


def cema_backward(dy, x, p, q, g, omega, padding_mask=None, bidirectional=False, shift=True, truncation=None):
    """Gradients of cema_forward (no activation, no carried state; ``truncation`` as in the forward):
    (dx, dp (K, N), dq (K, N) complex64 = dL/dRe q + i dL/dIm q, dgamma_hat likewise, domega (D))."""
    _cuda(dy, x, p, q, g, omega, padding_mask)
    bsz, dim, length = x.shape
    if dy.dtype != x.dtype:
        dy = dy.to(x.dtype)
    p, q, g, omega = _f32c(p), _c64(q), _c64(g), _f32c(omega).reshape(-1)
    n = p.shape[1]
    mask = _mask_u8(padding_mask, bsz, length)
    dx = _like(x)
    dp = torch.empty_like(p)
    dq = torch.empty_like(q)
    dg = torch.empty_like(g)
    dom = torch.empty(dim, device=x.device, dtype=torch.float32)
    flags = (EMA_BIDIRECTIONAL if bidirectional else 0) | (0 if shift else EMA_NO_SHIFT)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_cema_bwd(
            dy.data_ptr(), x.data_ptr(), dx.data_ptr(), _dt(x), bsz, dim, length, *dy.stride(), *x.stride(),
            *dx.stride(), p.data_ptr(), q.data_ptr(), g.data_ptr(), omega.data_ptr(), n, _ptr(mask), flags,
            _trunc(truncation), dp.data_ptr(), dq.data_ptr(), dg.data_ptr(), dom.data_ptr(), _stream()), "cema_bwd")
    return dx, dp, torch.view_as_complex(dq), torch.view_as_complex(dg), dom


def cema_coeffs_bwd(alpha, delta, theta, q, dp, dq, dg):
    """(dalpha, ddelta (K, N, 1), dtheta (K, 1, 1), dgamma (K, N, 2)) from the coefficient gradients."""
    _cuda(alpha, delta, theta, q, dp, dq, dg)
    k, n = alpha.shape[0], alpha.shape[1]
    a, d, t = _f32c(alpha).view(k, n), _f32c(delta).view(k, n), _f32c(theta).view(k)
    q, dp, dq, dg = _c64(q), _f32c(dp), _c64(dq), _c64(dg)
    da = torch.empty(k, n, device=alpha.device, dtype=torch.float32)
    dd = torch.empty_like(da)
    dt = torch.empty(k, device=alpha.device, dtype=torch.float32)
    dgm = torch.empty(k, n, 2, device=alpha.device, dtype=torch.float32)
    with torch.cuda.device(alpha.device):
        _lib.check(_lib.lib().mega_cema_coeffs_bwd(a.data_ptr(), d.data_ptr(), t.data_ptr(), q.data_ptr(),
                                                   dp.data_ptr(), dq.data_ptr(), dg.data_ptr(), k, n, da.data_ptr(),
                                                   dd.data_ptr(), dt.data_ptr(), dgm.data_ptr(), _stream()),
                   "cema_coeffs_bwd")
    return da.unsqueeze(-1), dd.unsqueeze(-1), dt.view(k, 1, 1), dgm


# ----------------------------------------------------------------------- attention
def attention_softmax_fwd(x, causal=True):
    """softmax over the last axis of the score tensor x (..., C_q, C_k); with ``causal`` row r keeps
    its first C_k - C_q + r + 1 columns (the rest is 0).  A row of -inf scores gives zeros."""
    _cuda(x)
    xc = x.contiguous()
    outer, inner = xc.shape[-2], xc.shape[-1]
    batch = xc.numel() // (outer * inner)
    y = torch.empty_like(xc)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_attention_softmax_fwd(xc.data_ptr(), y.data_ptr(), _dt(xc), batch, outer, inner,
                                                         1 if causal else 0, _stream()), "attention_softmax_fwd")
    return y


def attention_dropkey_softmax_fwd(x, dropout, causal=True, seed=0, offset=0):
    """attention_softmax_fwd with DropKey: every kept score is masked with probability ``dropout``
    before the softmax (no rescaling).  The mask is a function of (seed, offset, row, column)."""
    _cuda(x)
    xc = x.contiguous()
    outer, inner = xc.shape[-2], xc.shape[-1]
    batch = xc.numel() // (outer * inner)
    y = torch.empty_like(xc)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mega_attention_dropkey_softmax_fwd(
            xc.data_ptr(), y.data_ptr(), _dt(xc), batch, outer, inner, 1 if causal else 0, float(dropout),
            int(seed) & 0xFFFFFFFFFFFFFFFF, int(offset) & 0xFFFFFFFFFFFFFFFF, _stream()), "attention_dropkey_softmax_fwd")
    return y


def attention_softmax_bwd(dy, y, causal=True):
    """Gradient of attention_softmax_fwd with respect to the scores."""
    _cuda(dy, y)
    yc = y.contiguous()
    dyc = dy.to(yc.dtype).contiguous()
    outer, inner = yc.shape[-2], yc.shape[-1]
    batch = yc.numel() // (outer * inner)
    dx = torch.empty_like(yc)
    with torch.cuda.device(y.device):
        _lib.check(_lib.lib().mega_attention_softmax_bwd(dyc.data_ptr(), yc.data_ptr(), dx.data_ptr(), _dt(yc), batch,
                                                         outer, inner, 1 if causal else 0, _stream()),
                   "attention_softmax_bwd")
    return dx
