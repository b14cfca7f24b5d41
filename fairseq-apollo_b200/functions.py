"""autograd Functions of the training path: forward and backward both run on the library's
kernels; what is saved between them follows the reference's Functions
(fairseq/modules/norm_layer/timestep_norm.py:14-66, sequence_norm.py:12-52,
fairseq/modules/fused_ops/{fftconv,ema_parameters,ema_hidden}.py)."""
import torch

from . import ops


def needs_grad(*tensors):
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


class EMAFunction(torch.autograd.Function):
    """y = EMA(x) for x (B, D, L): coefficients, convolution, mask and omega residual in one
    forward kernel; one backward kernel for (dx, dp, dq, dgamma_hat, domega) and a small one for
    the chain rule to (alpha, delta, beta, gamma)."""

    @staticmethod
    def forward(ctx, x, alpha, delta, beta, gamma, omega, padding_mask, bidirectional, shift, truncation=None):
        p, q, g = ops.ema_coeffs(alpha, delta, beta, gamma)
        y = ops.ema_forward(x, p, q, g, omega, padding_mask, None, False, bidirectional=bidirectional,
                            shift=shift, truncation=truncation)
        ctx.save_for_backward(x, alpha, delta, beta, omega, padding_mask, p, q, g)
        ctx.bidirectional, ctx.shift, ctx.truncation = bidirectional, shift, truncation
        return y

    @staticmethod
    def backward(ctx, dy):
        x, alpha, delta, beta, omega, padding_mask, p, q, g = ctx.saved_tensors
        dx, dp, dq, dg, dom, _ = ops.ema_backward(dy, x, p, q, g, omega, padding_mask,
                                                  bidirectional=ctx.bidirectional, shift=ctx.shift,
                                                  truncation=ctx.truncation)
        da, dd, db, dgm = ops.ema_coeffs_bwd(alpha, delta, beta, dp, dq, dg)
        return (dx, da.to(alpha.dtype), dd.to(delta.dtype), db.to(beta.dtype), dgm.to(alpha.dtype),
                dom.to(omega.dtype), None, None, None, None)


class ComplexEMAFunction(torch.autograd.Function):
    """y = complex EMA(x) for x (B, D, L); parameters alpha, delta (K, N, 1), theta (K, 1, 1),
    gamma (K, N, 2), omega (D, 1) as in MultiHeadComplexEMA."""

    @staticmethod
    def forward(ctx, x, alpha, delta, theta, gamma, omega, padding_mask, bidirectional, shift, truncation=None):
        p, q, g = ops.cema_coeffs(alpha, delta, theta, gamma)
        y = ops.cema_forward(x, p, q, g, omega, padding_mask, None, False, bidirectional=bidirectional, shift=shift,
                             truncation=truncation)
        ctx.save_for_backward(x, alpha, delta, theta, omega, padding_mask, p, q, g)
        ctx.bidirectional, ctx.shift, ctx.truncation = bidirectional, shift, truncation
        ctx.gamma_dtype = gamma.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, alpha, delta, theta, omega, padding_mask, p, q, g = ctx.saved_tensors
        dx, dp, dq, dg, dom = ops.cema_backward(dy, x, p, q, g, omega, padding_mask,
                                                bidirectional=ctx.bidirectional, shift=ctx.shift,
                                                truncation=ctx.truncation)
        da, dd, dt, dgm = ops.cema_coeffs_bwd(alpha, delta, theta, q, dp, dq, dg)
        return (dx, da.to(alpha.dtype), dd.to(delta.dtype), dt.to(theta.dtype), dgm.to(ctx.gamma_dtype),
                dom.view_as(omega).to(omega.dtype), None, None, None, None)


class TimestepNormFunction(torch.autograd.Function):
    """(y, count, mean, var) = TimestepNorm(x (B, L, D)); gamma is the effective scale."""

    @staticmethod
    def forward(ctx, x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask, num_groups, eps):
        y, count, mean, var, cummean, cumrstd, group_mean = ops.timestep_norm_fwd_train(
            x, prev_count, prev_mean, prev_var, gamma, beta, padding_mask, eps, num_groups)
        ctx.save_for_backward(x, prev_mean, count, cummean, cumrstd, group_mean, gamma, padding_mask)
        ctx.num_groups = num_groups
        ctx.dtypes = (prev_mean.dtype, prev_var.dtype, gamma.dtype, beta.dtype)
        ctx.mark_non_differentiable(count)
        return y, count, mean, var

    @staticmethod
    def backward(ctx, dy, _, dmean, dvar):
        x, prev_mean, count, cummean, cumrstd, group_mean, gamma, padding_mask = ctx.saved_tensors
        dx, dpm, dpv, dgamma, dbeta = ops.timestep_norm_bwd(dy, dmean, dvar, x, prev_mean, count, cummean,
                                                            cumrstd, group_mean, gamma, padding_mask,
                                                            ctx.num_groups)
        t = ctx.dtypes
        return dx, None, dpm.to(t[0]), dpv.to(t[1]), dgamma.to(t[2]), dbeta.to(t[3]), None, None, None


class SequenceNormFunction(torch.autograd.Function):
    """y = SequenceNorm(x), per channel or per channel group; gamma is the effective scale."""

    @staticmethod
    def forward(ctx, x, gamma, beta, padding_mask, eps, length_last, num_groups=None):
        y, count, mean, rstd = ops.sequence_norm_fwd(x, gamma, beta, padding_mask, eps, length_last, num_groups)
        ctx.save_for_backward(x, count, mean, rstd, gamma, padding_mask)
        ctx.length_last = length_last
        ctx.num_groups = num_groups
        ctx.dtypes = (gamma.dtype, beta.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, count, mean, rstd, gamma, padding_mask = ctx.saved_tensors
        dx, dgamma, dbeta = ops.sequence_norm_bwd(dy, x, count, mean, rstd, gamma, padding_mask, ctx.length_last,
                                                  ctx.num_groups)
        return dx, dgamma.to(ctx.dtypes[0]), dbeta.to(ctx.dtypes[1]), None, None, None, None
