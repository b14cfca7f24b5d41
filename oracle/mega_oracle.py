"""TEST INFRASTRUCTURE ONLY — CPU restatement of the Mega EMA hot path.

This module is the checker for the CUDA kernels.  Only tests, the smoke check
and the CPU-baseline leg of the benchmark may import it; the product package
never does and fails loudly without its CUDA library.

Every function restates one piece of the reference (paths are relative to the
fairseq-apollo checkout) and says which lines it follows.

Parity pin: the reference ships no test, golden vector or known-answer file
for this path.  The restatement is therefore pinned against outputs of the
reference itself: (1) the reference's CPU C++ ops compiled by
``oracle/build_ref.py`` and (2) the reference's Python modules imported from
the checkout; both were run by ``tests/golden/make_golden.py`` and the results
are committed under ``tests/golden/``.  ``tests/test_oracle_vs_golden.py``
checks this file against those fixtures.

Deviations from the literal ``MultiHeadEMA`` class, which does not run in the
reference snapshot (its omega has shape (D,) but multiplies a (B,D,L) tensor,
and its ``_compute_kernel`` has a stale signature):
  * omega is broadcast per channel, as ``omega.view(D, 1)``;
  * the kernel routine returns ``(k, bias)`` like the working complex class.
The real EMA equals ``MultiHeadComplexEMA`` with the rotation switched off
(theta -> -inf, gamma' = gamma * beta); the golden vectors use that mapping.
"""
import math
from typing import Optional, Tuple

import torch


# --------------------------------------------------------------------------
# EMA coefficients and kernel
# --------------------------------------------------------------------------
def ema_coeffs(alpha, delta, beta, gamma, dtype=torch.float32):
    """p, q, gamma_hat from the raw parameters.

    fairseq/modules/exponential_moving_average.py:71-80:
      p = sigmoid(alpha) * beta ; q = 1 - sigmoid(alpha) * sigmoid(delta) ;
      gamma_hat = gamma * sqrt(1 / ndim).
    Shapes: alpha, delta, beta (K, N, 1); gamma (K, N).  Returns p, q (K, N) and
    gamma_hat (K, N).
    """
    n = alpha.shape[1]
    a = torch.sigmoid(alpha.to(dtype))
    d = torch.sigmoid(delta.to(dtype))
    q = 1.0 - a * d
    p = a * beta.to(dtype)
    g = gamma.to(dtype) * math.sqrt(1.0 / n)
    return p.squeeze(-1), q.squeeze(-1), g


def ema_kernel(p, q, g, length):
    """k[d, l] = sum_n p*gamma_hat*exp(l*log q), l < length.

    fairseq/modules/exponential_moving_average.py:82-90 (Vandermonde through
    exp(arange * log q), then einsum over the ndim axis).
    """
    ar = torch.arange(length, dtype=q.dtype).view(1, 1, length)
    vander = torch.exp(ar * torch.log(q).unsqueeze(-1))
    return torch.einsum("dnl,dn->dl", p.unsqueeze(-1) * vander, g)


def ema_bias(q, g, h, length):
    """Output term of a carried state: b[b,d,l] = sum_n q^(l+1) gamma_hat h[b,d,n].

    fairseq/csrc/ops/ema_parameters.cc:54-77 with real q (the complex op's
    real part), equivalently base_moving_average.py:75-79.
    """
    ar = torch.arange(1, length + 1, dtype=q.dtype).view(1, 1, length)
    vander = torch.exp(ar * torch.log(q).unsqueeze(-1))  # D N L
    return torch.einsum("bdn,dnl->bdl", h.to(q.dtype), vander * g.unsqueeze(-1))


def ema_hidden(x, p, q, h):
    """State after a chunk: h' = q^L h + p * sum_l q^(L-1-l) x_l.

    fairseq/csrc/ops/ema_hidden.cc:31-63 with real q; x is (B, D, L) and is
    expected to be already zeroed at padded positions.
    """
    length = x.shape[-1]
    ar = torch.arange(length - 1, -1, -1, dtype=q.dtype).view(1, 1, length)
    vander = torch.exp(ar * torch.log(q).unsqueeze(-1))  # D N L : q^(L-1-l)
    out = torch.einsum("bdl,dnl->bdn", x.to(q.dtype), vander) * p
    if h is not None:
        out = out + torch.exp(length * torch.log(q)) * h.to(q.dtype)
    return out


def _fftconv(x, k):
    """Causal convolution through a zero-padded FFT.

    fairseq/modules/fused_ops/fftconv.py:45-61 (the path taken on CPU and, on
    GPU, for L < 32 or L > 8192): FFT length 2 * next_pow2(L), kernel
    transformed with norm="forward", inverse with norm="forward".
    """
    length = x.size(-1)
    n = length if (length & (length - 1)) == 0 else (1 << length.bit_length())
    dtype = x.dtype
    if dtype in (torch.float16, torch.bfloat16):
        x = x.float()
    x_f = torch.fft.rfft(x, n=2 * n)
    k_f = torch.fft.rfft(k, n=2 * n, norm="forward")
    y = torch.fft.irfft(x_f * k_f, n=2 * n, norm="forward")[..., :length]
    if dtype in (torch.float16, torch.bfloat16):
        y = y.to(dtype)
    return y


def _bidirectional_fftconv(x, k, shift):
    """fairseq/modules/fused_ops/fftconv.py:85-100.

    k is (2D, K): rows [0, D) are the causal half, rows [D, 2D) the anti-causal
    half.  With shift=True the anti-causal half starts at lag 1 (its tap j
    weighs x[t+j+1]); with shift=False its tap 0 sits at lag 0.
    """
    _, embed_dim, seq_len = x.size()
    kernel_size = k.size(1)
    fft_len = seq_len + kernel_size
    k1, k2 = torch.split(k, [embed_dim, embed_dim], dim=0)
    pad = torch.nn.functional.pad
    if shift:
        kk = pad(k1, (0, seq_len)) + pad(k2.flip(-1), (seq_len, 0))
    else:
        kk = (pad(k1, (0, seq_len)) + pad(k2[:, :1], (0, fft_len - 1))
              + pad(k2[:, 1:].flip(-1), (seq_len + 1, 0)))
    k_f = torch.fft.rfft(kk, n=fft_len, norm="forward")
    x_f = torch.fft.rfft(x.float(), n=fft_len)
    return torch.fft.irfft(x_f * k_f, n=fft_len, norm="forward")[..., :seq_len].to(x)


def ema_forward_fft(x, alpha, delta, beta, gamma, omega, padding_mask=None,
                    bidirectional=False, shift=True, truncation=None,
                    h=None, return_state=False):
    """The reference's own forward flow with its FFT convolution (CPU path).

    fairseq/modules/base_moving_average.py:120-172: residual = x * omega (from
    the UNMASKED x); x is zeroed at pads; k, b = kernel(L, h); causal or
    bidirectional FFT convolution; + bias of a carried state; + residual.
    x is (B, D, L); padding_mask (B, L) with True/1 at pads.  When
    ``return_state`` the new state (ema_hidden) is returned as well.
    """
    bsz, dim, length = x.shape
    p, q, g = ema_coeffs(alpha, delta, beta, gamma)
    residual = x * omega.view(dim, 1).to(x.dtype if x.dtype == torch.float64 else torch.float32)
    if padding_mask is not None:
        x = x * (1.0 - padding_mask.unsqueeze(1).to(x))
    ksize = length if truncation is None or truncation < 1 else min(truncation, length)
    k = ema_kernel(p, q, g, ksize)
    if bidirectional:
        assert h is None and not return_state
        out = _bidirectional_fftconv(x, k, shift)
    else:
        out = _fftconv(x, k)
        if h is not None:
            out = out + ema_bias(q, g, h, length)
    out = out + residual
    if return_state:
        return out, ema_hidden(x, p, q, h)
    return out


def ema_forward_recurrence(x, alpha, delta, beta, gamma, omega, padding_mask=None,
                           bidirectional=False, shift=True, truncation=None,
                           h=None, return_state=False, silu=False):
    """Independent ground truth in float64: the diagonal recurrence itself.

    h_t = q h_{t-1} + p x~_t,  y_t = sum_n gamma_hat_n h_{n,t} + omega x_t with
    x~ = x zeroed at pads (base_moving_average.py:105-118 ``one_step`` applied
    L times; residual from the unmasked x as in :138).  Bidirectional: rows
    [D, 2D) of the parameters run anti-causally, starting at lag 1 when
    ``shift`` (fused_ops/fftconv.py:91-94).  A positive ``truncation`` limits
    the kernel support to its first ``truncation`` taps
    (base_moving_average.py:60-62).
    """
    x64 = x.double()
    bsz, dim, length = x64.shape
    p, q, g = ema_coeffs(alpha, delta, beta, gamma, dtype=torch.float64)
    xm = x64
    if padding_mask is not None:
        xm = x64 * (1.0 - padding_mask.unsqueeze(1).double())
    ksize = length if truncation is None or truncation < 1 else min(truncation, length)

    def scan(xs, pp, qq, gg, h0):
        # xs (B, D, L) -> outputs (B, D, L), final state (B, D, N)
        st = torch.zeros(bsz, dim, pp.shape[1], dtype=torch.float64) if h0 is None else h0.double().clone()
        ys = torch.empty_like(xs)
        hist = []
        qk = qq ** ksize
        for t in range(length):
            st = qq * st + pp * xs[:, :, t:t + 1]
            if ksize < length:
                hist.append(st)
                eff = st - (qk * hist[t - ksize] if t >= ksize else 0.0)
            else:
                eff = st
            ys[:, :, t] = (eff * gg).sum(-1)
        return ys, st

    if not bidirectional:
        y, st = scan(xm, p, q, g, h)
    else:
        assert h is None and not return_state
        y, _ = scan(xm, p[:dim], q[:dim], g[:dim], None)
        xr = xm.flip(-1)
        if shift:
            xr = torch.nn.functional.pad(xr, (1, 0))[..., :length]
        yb, _ = scan(xr, p[dim:], q[dim:], g[dim:], None)
        y = y + yb.flip(-1)
    y = y + x64 * omega.double().view(dim, 1)
    if silu:
        y = y * torch.sigmoid(y)
    if return_state:
        return y, st
    return y


def ema_one_step(x, p, q, g, h):
    """Single-token update: h' = p x + q h ; y = sum_n gamma_hat h'.

    fairseq/modules/base_moving_average.py:105-118.  x (B, D) or (B, D, 1).
    Returns y (B, D) WITHOUT the omega residual (the module adds it) and h'.
    """
    x = x.reshape(x.shape[0], x.shape[1], 1).to(q.dtype)
    hn = p * x
    if h is not None:
        hn = hn + q * h.to(q.dtype)
    return (hn * g).sum(-1), hn


# --------------------------------------------------------------------------
# Complex EMA (MultiHeadComplexEMA)
# --------------------------------------------------------------------------
def cema_coeffs(alpha, delta, theta, gamma, dtype=torch.float32):
    """p (K, N) real, q (K, N) complex, gamma_hat (K, N) complex.

    fairseq/modules/complex_exponential_moving_average.py:79-96:
      theta_n = n * sigmoid(theta) * 2 pi / N for n = 1..N ;
      p = sigmoid(alpha) ; q = polar(1 - sigmoid(alpha) sigmoid(delta), theta_n) ;
      gamma_hat = (gamma[..., 0] + i gamma[..., 1]) * sqrt(1 / N).
    """
    n = alpha.shape[1]
    th = torch.sigmoid(theta.to(dtype)) * (2 * math.pi / n)          # K 1 1
    wave = torch.arange(1, n + 1, dtype=dtype).view(1, n, 1)
    th = wave * th                                                    # K N 1
    a = torch.sigmoid(alpha.to(dtype))
    d = torch.sigmoid(delta.to(dtype))
    q = torch.polar(1.0 - a * d, th)
    g = torch.view_as_complex(gamma.to(dtype).contiguous()) * math.sqrt(1.0 / n)
    return a.squeeze(-1), q.squeeze(-1), g


def cema_forward_recurrence(x, alpha, delta, theta, gamma, omega, padding_mask=None,
                            bidirectional=False, shift=True, truncation=None,
                            h=None, return_state=False, silu=False):
    """Complex EMA layer in float64 as the recurrence itself.

    h_t = q h_{t-1} + p x~_t (complex), y_t = Re(sum_n gamma_hat_n h_{n,t}) + omega x_t:
    base_moving_average.py:105-118 (``one_step``) applied L times with the complex
    coefficients; mask, residual, bidirectional halves, shift and truncation as in
    ``ema_forward_recurrence``.  omega is (D, 1) or (D,).
    """
    x64 = x.double()
    bsz, dim, length = x64.shape
    p, q, g = cema_coeffs(alpha, delta, theta, gamma, dtype=torch.float64)
    xm = x64
    if padding_mask is not None:
        xm = x64 * (1.0 - padding_mask.unsqueeze(1).double())
    ksize = length if truncation is None or truncation < 1 else min(truncation, length)

    def scan(xs, pp, qq, gg, h0):
        st = torch.zeros(bsz, dim, pp.shape[1], dtype=torch.complex128) if h0 is None else h0.to(torch.complex128)
        ys = torch.empty_like(xs)
        hist = []
        qk = qq ** ksize
        for t in range(length):
            st = qq * st + pp * xs[:, :, t:t + 1]
            if ksize < length:
                hist.append(st)
                eff = st - (qk * hist[t - ksize] if t >= ksize else 0.0)
            else:
                eff = st
            ys[:, :, t] = (eff * gg).sum(-1).real
        return ys, st

    if not bidirectional:
        y, st = scan(xm, p, q, g, h)
    else:
        assert h is None and not return_state
        y, _ = scan(xm, p[:dim], q[:dim], g[:dim], None)
        xr = xm.flip(-1)
        if shift:
            xr = torch.nn.functional.pad(xr, (1, 0))[..., :length]
        yb, _ = scan(xr, p[dim:], q[dim:], g[dim:], None)
        y = y + yb.flip(-1)
    y = y + x64 * omega.double().view(dim, 1)
    if silu:
        y = y * torch.sigmoid(y)
    if return_state:
        return y, st
    return y


# --------------------------------------------------------------------------
# Welford helpers (fairseq/csrc/utils.h:56-76)
# --------------------------------------------------------------------------
def _welford_update(m0, m1, m2, x):
    m0 = m0 + 1
    coef = 1.0 / m0.to(m1.dtype) if torch.is_tensor(m0) else 1.0 / m0
    d1 = x - m1
    m1n = m1 + coef * d1
    d2 = d1 * (x - m1n) - m2
    m2n = m2 + coef * d2
    return m0, m1n, m2n


def _welford_combine(a0, a1, a2, b0, b1, b2):
    m0 = a0 + b0
    dt = a1.dtype
    m0f = m0.to(dt)
    safe = torch.where(m0 == 0, torch.ones_like(m0f), m0f)
    c1 = torch.where(m0 == 0, torch.zeros_like(m0f), a0.to(dt) / safe)
    c2 = torch.where(m0 == 0, torch.zeros_like(m0f), b0.to(dt) / safe)
    d = b1 - a1
    m1 = c1 * a1 + c2 * b1
    m2 = c1 * a2 + c2 * b2 + (c1 * d) * (c2 * d)
    return m0, m1, m2


# --------------------------------------------------------------------------
# TimestepNorm
# --------------------------------------------------------------------------
def timestep_norm(x, prev_count, prev_mean, prev_var, gamma, beta,
                  padding_mask=None, eps=1e-5, acc_dtype=torch.float32):
    """Causal cumulative normalisation, one statistic per (batch, feature).

    fairseq/csrc/ops/timestep_norm.cc:23-103.  x (B, L, H); prev_count (B,)
    int64; prev_mean, prev_var (B, H); gamma is the EFFECTIVE scale (the module
    passes weight + 1, norm_layer/timestep_norm.py:130).  Per step: Welford
    update of (count, mean, var) with x_t, y_t = (x_t - mean_t) * rstd_t *
    gamma + beta with rstd_t = 1/sqrt(var_t + eps); at a padded step the output
    is 0 and the statistics do not advance.  Returns (y, count, mean, var).
    """
    bsz, length, feat = x.shape
    xa = x.to(acc_dtype)
    w = gamma.to(acc_dtype)
    b = beta.to(acc_dtype)
    m0 = prev_count.clone().view(bsz, 1)
    u = prev_mean.to(acc_dtype).clone()
    v = prev_var.to(acc_dtype).clone()
    y = torch.empty_like(xa)
    for t in range(length):
        xt = xa[:, t]
        _, m1, m2 = _welford_update(m0, u, v, xt)
        rstd = 1.0 / torch.sqrt(m2 + eps)
        yt = (xt - m1) * rstd * w + b
        if padding_mask is not None:
            mk = padding_mask[:, t].bool().view(bsz, 1)
            yt = torch.where(mk, torch.zeros_like(yt), yt)
            u = torch.where(mk, u, m1)
            v = torch.where(mk, v, m2)
            m0 = m0 + (~mk).to(m0.dtype)
        else:
            u, v = m1, m2
            m0 = m0 + 1
        y[:, t] = yt
    return y.to(x.dtype), m0.view(bsz), u.to(x.dtype), v.to(x.dtype)


def _rowwise_moments(x):
    """Population mean / variance over the last axis (utils.h:79-118 computes
    the same quantity with a cascade of Welford chunks; the closed form differs
    from it only by rounding)."""
    m = x.mean(-1)
    v = ((x - m.unsqueeze(-1)) ** 2).mean(-1)
    return m, v


def group_timestep_norm(x, prev_count, prev_mean, prev_var, gamma, beta,
                        padding_mask=None, num_groups=1, eps=1e-5,
                        acc_dtype=torch.float32):
    """Grouped variant: statistics pooled over the H/G features of a group.

    fairseq/csrc/ops/timestep_norm.cc:218-316: per (b, t, g) moments over the
    group's features, then a cumulative WelfordCombine(state, count=1, mu, var)
    over time; count still counts timesteps.  prev_mean/prev_var are (B, G).
    """
    bsz, length, feat = x.shape
    gsz = feat // num_groups
    xa = x.to(acc_dtype).view(bsz, length, num_groups, gsz)
    w = gamma.to(acc_dtype).view(num_groups, gsz)
    b = beta.to(acc_dtype).view(num_groups, gsz)
    gm, gv = _rowwise_moments(xa)  # B L G
    m0 = prev_count.clone().view(bsz, 1)
    u = prev_mean.to(acc_dtype).clone()
    v = prev_var.to(acc_dtype).clone()
    y = torch.empty_like(xa)
    one = torch.ones_like(m0)
    for t in range(length):
        _, m1, m2 = _welford_combine(m0, u, v, one, gm[:, t], gv[:, t])
        rstd = 1.0 / torch.sqrt(m2 + eps)
        yt = (xa[:, t] - m1.unsqueeze(-1)) * rstd.unsqueeze(-1) * w + b
        if padding_mask is not None:
            mk = padding_mask[:, t].bool().view(bsz, 1)
            yt = torch.where(mk.unsqueeze(-1), torch.zeros_like(yt), yt)
            u = torch.where(mk, u, m1)
            v = torch.where(mk, v, m2)
            m0 = m0 + (~mk).to(m0.dtype)
        else:
            u, v = m1, m2
            m0 = m0 + 1
        y[:, t] = yt
    return (y.view(bsz, length, feat).to(x.dtype), m0.view(bsz),
            u.to(x.dtype), v.to(x.dtype))


# --------------------------------------------------------------------------
# SequenceNorm
# --------------------------------------------------------------------------
def sequence_norm(x, gamma, beta, padding_mask=None, num_groups=None, eps=1e-5,
                  length_last=True, acc_dtype=torch.float32):
    """Masked normalisation over the sequence axis.

    fairseq/csrc/ops/sequence_norm.cc:322-372 (length last, x (B, H, L)),
    :258-320 (x (B, L, H)), :531-655 (grouped).  Per (batch, channel) — or per
    (batch, group), pooling the group's channels — population mean/variance
    over the unmasked positions; y = (x - mean) * rstd * gamma + beta, 0 at
    pads; gamma is the effective scale (module passes weight + 1).  Returns
    (y, count (B,), mean, rstd) with mean/rstd (B, H) or (B, G).
    """
    xa = x.to(acc_dtype)
    if not length_last:
        xa = xa.transpose(1, 2)
    bsz, feat, length = xa.shape
    if padding_mask is not None:
        keep = (~padding_mask.bool()).to(acc_dtype).view(bsz, 1, length)
    else:
        keep = torch.ones(bsz, 1, length, dtype=acc_dtype)
    cnt = keep.sum(-1)  # B 1
    safe = cnt.clamp(min=1.0)
    if num_groups is None:
        mean = (xa * keep).sum(-1) / safe
        var = (((xa - mean.unsqueeze(-1)) ** 2) * keep).sum(-1) / safe
        mean = torch.where(cnt == 0, torch.zeros_like(mean), mean)
        var = torch.where(cnt == 0, torch.zeros_like(var), var)
        rstd = 1.0 / torch.sqrt(var + eps)
        mu_b, rs_b = mean.unsqueeze(-1), rstd.unsqueeze(-1)
    else:
        gsz = feat // num_groups
        xg = xa.view(bsz, num_groups, gsz, length)
        kg = keep.view(bsz, 1, 1, length)
        tot = (safe * gsz).view(bsz, 1)
        mean = (xg * kg).sum((-1, -2)) / tot
        var = (((xg - mean.view(bsz, num_groups, 1, 1)) ** 2) * kg).sum((-1, -2)) / tot
        mean = torch.where(cnt == 0, torch.zeros_like(mean), mean)
        var = torch.where(cnt == 0, torch.zeros_like(var), var)
        rstd = 1.0 / torch.sqrt(var + eps)
        mu_b = mean.repeat_interleave(gsz, dim=1).unsqueeze(-1)
        rs_b = rstd.repeat_interleave(gsz, dim=1).unsqueeze(-1)
    y = (xa - mu_b) * rs_b * gamma.to(acc_dtype).view(1, feat, 1) + beta.to(acc_dtype).view(1, feat, 1)
    y = y * keep
    if not length_last:
        y = y.transpose(1, 2)
    return (y.to(x.dtype).contiguous(), cnt.view(bsz).to(torch.int64), mean, rstd)


# --------------------------------------------------------------------------
# Mega gate elementwise ops
# --------------------------------------------------------------------------
def mega_gate_split(base, zdim, hdim, embed_dim, z_gamma, z_beta, norm_eps=1e-5):
    """Post-projection gates of the Mega block.

    fairseq/modules/moving_average_gated_attention.py:319-330: ``base`` is the
    output of mx_proj, split as (u, z, r, hx) = (D, Z, H, D); u = sigmoid(u);
    r = silu(r); z is L2-normalised over its last axis and expanded to query
    and key by a (2, Z) affine: z.unsqueeze(-2) * (gamma + 1) + beta.
    """
    u, z, r, hx = torch.split(base, [embed_dim, zdim, hdim, embed_dim], dim=-1)
    u = torch.sigmoid(u)
    r = torch.nn.functional.silu(r)
    z = torch.nn.functional.normalize(z, p=2, dim=-1, eps=norm_eps)
    zz = z.unsqueeze(-2) * (z_gamma + 1.0) + z_beta
    qq, kk = torch.unbind(zz, dim=-2)
    return u, qq, kk, r, hx


def mega_gate_output(residual, u, hx, h_lin):
    """fairseq/modules/moving_average_gated_attention.py:407-412:
    h = silu(hx + h_lin); out = residual + u * (h - residual)."""
    h = torch.nn.functional.silu(hx + h_lin)
    return torch.addcmul(residual, u, h - residual)


# --------------------------------------------------------------------------
# Attention-weight softmax
# --------------------------------------------------------------------------
def attention_softmax(x, use_causal_mask=True):
    """fairseq/csrc/softmax.cuh:90-153 (AttentionSoftmaxFwdKernel): softmax over the last axis of
    x (..., C_q, C_k); with the causal mask row r keeps its first C_k - C_q + r + 1 columns and the
    rest of the row is 0; a row whose kept scores are all -inf is all zeros."""
    outer, inner = x.shape[-2], x.shape[-1]
    xs = x.double()
    if use_causal_mask:
        cols = torch.arange(inner).view(1, inner)
        keep = cols < (inner - outer + torch.arange(outer).view(outer, 1) + 1)
        xs = xs.masked_fill(~keep, float("-inf"))
    m = xs.max(dim=-1, keepdim=True).values
    dead = torch.isinf(m) & (m < 0)
    e = torch.exp(xs - torch.where(dead, torch.zeros_like(m), m))
    e = torch.where(dead.expand_as(e), torch.zeros_like(e), e)
    d = e.sum(-1, keepdim=True)
    return torch.where(d == 0, torch.zeros_like(e), e / torch.where(d == 0, torch.ones_like(d), d))


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3",
    SC'11) on numpy uint64 arrays holding 32-bit words; returns the four output words."""
    import numpy as np
    m32 = np.uint64(0xFFFFFFFF)
    c0, c1, c2, c3 = [np.asarray(c, dtype=np.uint64) & m32 for c in np.broadcast_arrays(c0, c1, c2, c3)]
    k0, k1 = np.uint64(k0) & m32, np.uint64(k1) & m32
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & m32
        hi1, lo1 = p1 >> np.uint64(32), p1 & m32
        c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
        k0 = (k0 + np.uint64(0x9E3779B9)) & m32
        k1 = (k1 + np.uint64(0xBB67AE85)) & m32
    return c0, c1, c2, c3


def dropkey_mask(rows, inner, dropout, seed, offset=0):
    """The DropKey mask of the CUDA kernel (True = score dropped), shape (rows, inner): column c of
    row i is dropped when word c % 4 of Philox4x32-10(counter (c // 4, i, offset lo, offset hi),
    key (seed lo, seed hi)) is below dropout * 2^32.  The reference (fairseq/csrc/softmax.cuh:
    155-186) drops with the same probability from curand's Philox stream in its own thread
    order; only the distribution is shared."""
    import numpy as np
    groups = (inner + 3) // 4
    cg = np.arange(groups, dtype=np.uint64).reshape(1, groups)
    ri = np.arange(rows, dtype=np.uint64).reshape(rows, 1)
    w = philox4x32_10(cg, ri, np.uint64(offset & 0xFFFFFFFF), np.uint64((offset >> 32) & 0xFFFFFFFF),
                      seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    bits = np.stack(w, axis=-1).reshape(rows, groups * 4)[:, :inner]
    return torch.from_numpy(bits < np.uint64(int(dropout * 4294967296.0)))


def attention_dropkey_softmax(x, dropout, use_causal_mask, seed, offset=0):
    """fairseq/csrc/softmax.cuh:155-232 (AttentionDropKeySoftmaxFwdKernel) with the mask of
    ``dropkey_mask``: dropped scores become -inf before the softmax, nothing is rescaled."""
    outer, inner = x.shape[-2], x.shape[-1]
    rows = x.numel() // inner
    drop = dropkey_mask(rows, inner, dropout, seed, offset).view(x.shape)
    return attention_softmax(x.double().masked_fill(drop, float("-inf")), use_causal_mask)
