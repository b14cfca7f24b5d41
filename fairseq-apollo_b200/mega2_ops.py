"""Operator-level stand-in for ``fairseq.mega2_extension.ops`` (fairseq/csrc/mega2_extension.cc:14-24).

The reference's Python wrappers call the native extension by these names
(fairseq/modules/norm_layer/timestep_norm.py:29-66, norm_layer/sequence_norm.py:25-51,
attention_softmax.py:21-38, efficient_attention.py:22-40).  Binding this module in place of the
extension (``sys.modules["fairseq.mega2_extension.ops"] = fairseq_apollo_b200.mega2_ops``) lets those
wrappers and their autograd Functions run unchanged on this library's kernels: same argument order,
same tuple of results, gamma already the effective scale (weight + 1) as the wrappers pass it.

Statistics come back in float32 whatever the activation dtype (the reference returns them in the
activation dtype); they are cast where a caller's contract needs the activation dtype.

The EMA operators (``ema_parameters_fwd/bwd``, ``ema_hidden_fwd/bwd``, ``rfft``, ``fftconv_fwd/bwd``)
are NOT offered at this level: their interface is the reference's algorithm (a Vandermonde tensor
saved for backward, kernels in the frequency domain), which this build replaces as a whole by one
scan kernel.  The swap point for the EMA is the module class (``MultiHeadEMA`` /
``MultiHeadComplexEMA``); calling one of those names here raises with that explanation.
"""
import torch

from . import ops

__all__ = ["timestep_norm_fwd", "timestep_norm_bwd", "group_timestep_norm_fwd", "group_timestep_norm_bwd",
           "sequence_norm_fwd", "sequence_norm_bwd", "group_sequence_norm_fwd", "group_sequence_norm_bwd",
           "attention_softmax_fwd", "attention_softmax_bwd", "attention_fwd", "attention_bwd"]


def _stats_like(x, *ts):
    return tuple(None if t is None else t.to(x.dtype) for t in ts)


# ------------------------------------------------------------------ TimestepNorm (timestep_norm.cc:700-707)
def timestep_norm_fwd(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask, eps):
    """-> (y, count, mean, var, cummean, cumrstd)"""
    y, count, mean, var, cummean, cumrstd, _ = ops.timestep_norm_fwd_train(
        x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask, eps, None)
    return (y, count) + _stats_like(x, mean, var) + (cummean, cumrstd)


def group_timestep_norm_fwd(x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask, num_groups, eps):
    """-> (y, count, mean, var, group_mean, cummean, cumrstd)"""
    y, count, mean, var, cummean, cumrstd, group_mean = ops.timestep_norm_fwd_train(
        x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask, eps, num_groups)
    return (y, count) + _stats_like(x, mean, var) + (group_mean, cummean, cumrstd)


def timestep_norm_bwd(y_grad, mean_grad, var_grad, x, prev_mean, count, cummean, cumrstd, gamma, padding_mask):
    """-> (x_grad, prev_mean_grad, prev_var_grad, gamma_grad, beta_grad)"""
    dx, dpm, dpv, dg, db = ops.timestep_norm_bwd(y_grad, mean_grad, var_grad, x, prev_mean, count, cummean, cumrstd,
                                                 None, gamma, padding_mask, None)
    return (dx,) + _stats_like(prev_mean, dpm, dpv) + _stats_like(gamma, dg, db)


def group_timestep_norm_bwd(y_grad, mean_grad, var_grad, x, prev_mean, count, group_mean, cummean, cumrstd, gamma,
                            padding_mask, num_groups):
    dx, dpm, dpv, dg, db = ops.timestep_norm_bwd(y_grad, mean_grad, var_grad, x, prev_mean, count, cummean, cumrstd,
                                                 group_mean, gamma, padding_mask, num_groups)
    return (dx,) + _stats_like(prev_mean, dpm, dpv) + _stats_like(gamma, dg, db)


# ------------------------------------------------------------------ SequenceNorm (sequence_norm.cc:1066-1075)
def sequence_norm_fwd(x, gamma, beta, padding_mask, eps, length_last):
    """-> (y, count, mean, rstd)"""
    return ops.sequence_norm_fwd(x, gamma, beta, padding_mask, eps, length_last, None)


def group_sequence_norm_fwd(x, gamma, beta, padding_mask, num_groups, eps, length_last):
    return ops.sequence_norm_fwd(x, gamma, beta, padding_mask, eps, length_last, num_groups)


def sequence_norm_bwd(y_grad, x, count, mean, rstd, gamma, padding_mask, length_last):
    """-> (x_grad, gamma_grad, beta_grad)"""
    dx, dg, db = ops.sequence_norm_bwd(y_grad, x, count, mean, rstd, gamma, padding_mask, length_last, None)
    return (dx,) + _stats_like(gamma, dg, db)


def group_sequence_norm_bwd(y_grad, x, count, mean, rstd, gamma, padding_mask, num_groups, length_last):
    dx, dg, db = ops.sequence_norm_bwd(y_grad, x, count, mean, rstd, gamma, padding_mask, length_last, num_groups)
    return (dx,) + _stats_like(gamma, dg, db)


# ------------------------------------------------------------------ attention (attention_softmax.cc:20-23, attention.cc:28-31)
def attention_softmax_fwd(x, dropout, use_causal_mask):
    if dropout > 0.0:
        seed = int(torch.randint(0, 2 ** 62, (1,)).item())
        return ops.attention_dropkey_softmax_fwd(x, dropout, use_causal_mask, seed, 0)
    return ops.attention_softmax_fwd(x, use_causal_mask)


def attention_softmax_bwd(y_grad, y, use_causal_mask):
    return ops.attention_softmax_bwd(y_grad, y, use_causal_mask)


def attention_fwd(q, k, v, scale, dropout, use_causal_mask):
    """q, k (B, L, N, H1), v (B, L, N, H2) -> (y (B, L, N, H2), w (B, N, L, L)): library GEMMs around
    this library's softmax, the weights materialised as the reference operator does."""
    if q.dtype != v.dtype or k.dtype != v.dtype:
        q, k = q.to(v.dtype), k.to(v.dtype)
    s = torch.matmul(q.transpose(1, 2), k.transpose(1, 2).transpose(-1, -2))
    if scale != 1.0:
        s = s * scale
    w = attention_softmax_fwd(s, dropout, use_causal_mask)
    return torch.matmul(w, v.transpose(1, 2)).transpose(1, 2).contiguous(), w


def attention_bwd(y_grad, q, k, v, w, scale, use_causal_mask):
    """-> (q_grad, k_grad, v_grad)"""
    qh, kh, vh = q.to(v.dtype).transpose(1, 2), k.to(v.dtype).transpose(1, 2), v.transpose(1, 2)
    gh = y_grad.transpose(1, 2)
    v_grad = torch.matmul(w.transpose(-1, -2), gh)
    s_grad = ops.attention_softmax_bwd(torch.matmul(gh, vh.transpose(-1, -2)), w, use_causal_mask)
    if scale != 1.0:
        s_grad = s_grad * scale
    q_grad = torch.matmul(s_grad, kh).transpose(1, 2).contiguous().to(q.dtype)
    k_grad = torch.matmul(s_grad.transpose(-1, -2), qh).transpose(1, 2).contiguous().to(k.dtype)
    return q_grad, k_grad, v_grad.transpose(1, 2).contiguous()


def _not_at_this_level(name):
    def f(*args, **kwargs):
        raise NotImplementedError(
            "%s: the EMA operators of the reference extension (Vandermonde / frequency-domain interface) have no "
            "counterpart at operator level in this library; swap the module classes MultiHeadEMA / "
            "MultiHeadComplexEMA instead (one scan kernel replaces ema_parameters + fftconv + ema_hidden)" % name)
    f.__name__ = name
    return f


for _n in ("ema_parameters_fwd", "ema_parameters_bwd", "ema_hidden_fwd", "ema_hidden_bwd", "rfft", "fftconv_fwd",
           "fftconv_bwd"):
    globals()[_n] = _not_at_this_level(_n)
