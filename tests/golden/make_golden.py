"""Generates tests/golden/*.npz by running the REFERENCE ITSELF on CPU.

Run in a container where the reference checkout is mounted (default
/root/reference, override with MEGA_REFERENCE_ROOT).  It needs
``oracle/_ref/mega_ref_cpu.so`` (python oracle/build_ref.py).  The fixtures are
committed; nothing at test time reads the reference checkout.

Usage: python tests/golden/make_golden.py [all|forward|backward|cema|cema_backward|backward_truncated].

What runs:
  * the reference's CPU C++ ops (timestep_norm_fwd, group_timestep_norm_fwd,
    sequence_norm_fwd, group_sequence_norm_fwd, ema_parameters_fwd,
    ema_hidden_fwd) through oracle/_ref;
  * the reference's Python modules MultiHeadComplexEMA, TimestepNorm and
    SequenceNorm, imported by file path under placeholder parent packages
    (the full ``fairseq`` package does not import without its Cython parts).

The real-valued EMA is produced by MultiHeadComplexEMA with the rotation
switched off: theta = -1e4 (sigmoid -> 0), gamma'[..., 0] = gamma * beta,
gamma'[..., 1] = 0, omega' = omega.view(D, 1).  MultiHeadEMA itself does not
run in the reference snapshot.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("MEGA_REFERENCE_ROOT", "/root/reference")
sys.path.insert(0, ROOT)

from oracle.build_ref import load_ref  # noqa: E402


def import_reference():
    ref = load_ref()
    if ref is None:
        raise SystemExit("build oracle/_ref first: python oracle/build_ref.py")
    ops = ref.ops
    fs = os.path.join(REF, "fairseq")

    def pkg(name, path=None):
        m = types.ModuleType(name)
        m.__path__ = [path] if path else []
        sys.modules[name] = m
        return m

    pkg("fairseq", fs)
    ext = pkg("fairseq.mega2_extension")
    ext.ops = ops
    sys.modules["fairseq.mega2_extension.ops"] = ops
    for n in ("rfft", "fftconv_fwd", "fftconv_bwd"):  # CUDA-only in the reference
        if not hasattr(ops, n):
            setattr(ops, n, None)
    pkg("fairseq.modules", fs + "/modules")
    pkg("fairseq.modules.fused_ops", fs + "/modules/fused_ops")
    pkg("fairseq.modules.norm_layer", fs + "/modules/norm_layer")

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(fs, rel))
        m = importlib.util.module_from_spec(spec)
        sys.modules[name] = m
        spec.loader.exec_module(m)
        return m

    load("fairseq.incremental_decoding_utils", "incremental_decoding_utils.py")
    load("fairseq.modules.fused_ops.fftconv", "modules/fused_ops/fftconv.py")
    load("fairseq.modules.fused_ops.ema_hidden", "modules/fused_ops/ema_hidden.py")
    load("fairseq.modules.fused_ops.ema_parameters", "modules/fused_ops/ema_parameters.py")
    load("fairseq.modules.base_moving_average", "modules/base_moving_average.py")
    cema = load("fairseq.modules.complex_exponential_moving_average",
                "modules/complex_exponential_moving_average.py")
    tsn = load("fairseq.modules.norm_layer.timestep_norm", "modules/norm_layer/timestep_norm.py")
    sqn = load("fairseq.modules.norm_layer.sequence_norm", "modules/norm_layer/sequence_norm.py")
    return ops, cema, tsn, sqn


def ema_params(gen, dim, ndim, bidirectional):
    k = 2 * dim if bidirectional else dim
    alpha = torch.randn(k, ndim, 1, generator=gen) * 0.2
    delta = torch.randn(k, ndim, 1, generator=gen) * 0.2
    val = torch.ones(ndim, 1)
    val[1::2] = -1.0
    beta = torch.randn(k, ndim, 1, generator=gen) * 0.02 + val
    gamma = torch.randn(k, ndim, generator=gen)
    omega = torch.randn(dim, generator=gen)
    return alpha, delta, beta, gamma, omega


def right_pad_mask(gen, bsz, length, frac):
    mask = torch.zeros(bsz, length, dtype=torch.bool)
    for b in range(bsz):
        n = int(torch.rand((), generator=gen).item() * frac * length)
        if n:
            mask[b, length - n:] = True
    return mask


def cema_from_real(cema, dim, ndim, params, **kw):
    alpha, delta, beta, gamma, omega = params
    m = cema.MultiHeadComplexEMA(dim, ndim=ndim, **kw).eval()
    with torch.no_grad():
        m.alpha.copy_(alpha)
        m.delta.copy_(delta)
        m.theta.fill_(-1e4)
        m.gamma[:, :, 0] = gamma * beta.squeeze(-1)
        m.gamma[:, :, 1] = 0.0
        m.omega.copy_(omega.view(dim, 1))
    return m


def npz(name, **arrs):
    out = {}
    for k, v in arrs.items():
        if torch.is_tensor(v):
            v = v.detach().cpu().numpy()
        out[k] = np.asarray(v)
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **out)
    print(name, os.path.getsize(path), "bytes")


def main():
    ops, cema, tsn, sqn = import_reference()
    gen = torch.Generator().manual_seed(20251125)

    # ---- EMA, non-incremental, through the reference module ------------------
    for tag, (bsz, dim, length, ndim, bidir, shift, trunc, pad) in {
        "ema_uni_n16": (3, 8, 50, 16, False, True, None, 0.25),
        "ema_uni_n2": (2, 5, 33, 2, False, True, None, 0.0),
        "ema_uni_pow2": (2, 4, 64, 16, False, True, None, 0.5),
        "ema_bidir_shift": (3, 6, 41, 16, True, True, None, 0.5),
        "ema_bidir_noshift": (2, 6, 32, 16, True, False, None, 0.3),
        "ema_bidir_trunc": (2, 4, 40, 16, True, True, 7, 0.3),
    }.items():
        params = ema_params(gen, dim, ndim, bidir)
        x = torch.randn(bsz, dim, length, generator=gen)
        mask = right_pad_mask(gen, bsz, length, pad) if pad > 0 else None
        m = cema_from_real(cema, dim, ndim, params, bidirectional=bidir, truncation=trunc, shift=shift)
        with torch.no_grad():
            y = m(x, mask, None)
        npz(tag, x=x, alpha=params[0], delta=params[1], beta=params[2], gamma=params[3], omega=params[4],
            mask=(mask if mask is not None else np.zeros((0,), bool)), y=y,
            bidirectional=bidir, shift=shift, truncation=(-1 if trunc is None else trunc))

    # ---- EMA incremental through the reference CPU ops ------------------------
    bsz, dim, length, ndim, chunk = 3, 6, 48, 16, 16
    params = ema_params(gen, dim, ndim, False)
    x = torch.randn(bsz, dim, length, generator=gen)
    m = cema_from_real(cema, dim, ndim, params)
    fftconv = sys.modules["fairseq.modules.fused_ops.fftconv"]._fftconv_fwd
    with torch.no_grad():
        pc, qc, gc = m._calc_coeffs()
        hh, ys, hs = None, [], []
        for i in range(0, length, chunk):
            xc = x[..., i:i + chunk].contiguous()
            w, b, _ = ops.ema_parameters_fwd(pc, qc.log(), gc, hh, chunk)
            yy = fftconv(xc, w)[0]
            if b is not None:
                yy = yy + b
            hh, _ = ops.ema_hidden_fwd(xc, pc, qc.log(), hh)
            ys.append(yy + xc * m.omega)
            hs.append(hh.real.clone())          # state convention: p folded in (cema: p = sigmoid(alpha))
        # closed-form single step from the reference base class
        y1, h1 = m.one_step(x[..., :1], hx=None)
        y2, h2 = m.one_step(x[..., 1:2], hx=h1)
    npz("ema_incremental", x=x, alpha=params[0], delta=params[1], beta=params[2], gamma=params[3],
        omega=params[4], chunk=chunk, y=torch.cat(ys, -1), states=torch.stack(hs),
        imag_max=max(float(h.abs().max()) for h in [hh.imag]),
        step_y1=y1, step_h1=h1.real, step_y2=y2, step_h2=h2.real)

    # ---- TimestepNorm through the reference CPU op ---------------------------------
    for tag, (bsz, length, feat, groups, pad, prior) in {
        "tsn_plain": (3, 37, 10, None, 0.4, 2),
        "tsn_plain_nomask": (2, 64, 7, None, 0.0, 0),
        "tsn_group2": (3, 29, 12, 2, 0.4, 0),
        "tsn_group_prior": (2, 16, 15, 5, 0.0, 3),
    }.items():
        x = torch.randn(bsz, length, feat, generator=gen) * 1.7 + 0.3
        mask = right_pad_mask(gen, bsz, length, pad) if pad > 0 else None
        if mask is not None:
            mask[0, 3] = True          # an interior pad as well
            mask[bsz - 1, :] = True    # one fully padded row
        ng = feat if groups is None else groups
        prev_count = torch.full((bsz,), prior, dtype=torch.int64)
        prev_mean = torch.randn(bsz, ng, generator=gen) * 0.1 if prior else torch.zeros(bsz, ng)
        prev_var = torch.rand(bsz, ng, generator=gen) + 0.5 if prior else torch.ones(bsz, ng)
        gamma = torch.randn(feat, generator=gen) * 0.1 + 1.0
        beta = torch.randn(feat, generator=gen) * 0.1
        if groups is None:
            y, cnt, mean, var, cm, cr = ops.timestep_norm_fwd(x, prev_count, prev_mean, prev_var, gamma, beta, mask, 1e-5)
        else:
            y, cnt, mean, var, gm, cm, cr = ops.group_timestep_norm_fwd(x, prev_count, prev_mean, prev_var, gamma, beta, mask, groups, 1e-5)
        npz(tag, x=x, mask=(mask if mask is not None else np.zeros((0,), bool)), prev_count=prev_count,
            prev_mean=prev_mean, prev_var=prev_var, gamma=gamma, beta=beta, groups=(-1 if groups is None else groups),
            y=y, count=cnt, mean=mean, var=var)

    # ---- SequenceNorm through the reference CPU op -----------------------------------
    for tag, (bsz, feat, length, groups, length_last, pad) in {
        "sqn_bhl": (3, 6, 45, None, True, 0.5),
        "sqn_blh": (3, 6, 45, None, False, 0.5),
        "sqn_bhl_group": (3, 12, 33, 3, True, 0.5),
        "sqn_blh_group": (2, 12, 33, 4, False, 0.0),
    }.items():
        shape = (bsz, feat, length) if length_last else (bsz, length, feat)
        x = torch.randn(*shape, generator=gen) * 2.0 - 0.5
        mask = right_pad_mask(gen, bsz, length, pad) if pad > 0 else None
        if mask is not None:
            mask[bsz - 1, :] = True
        gamma = torch.randn(feat, generator=gen) * 0.1 + 1.0
        beta = torch.randn(feat, generator=gen) * 0.1
        if groups is None:
            y, cnt, mean, rstd = ops.sequence_norm_fwd(x, gamma, beta, mask, 1e-5, length_last)
        else:
            y, cnt, mean, rstd = ops.group_sequence_norm_fwd(x, gamma, beta, mask, groups, 1e-5, length_last)
        npz(tag, x=x, mask=(mask if mask is not None else np.zeros((0,), bool)), gamma=gamma, beta=beta,
            groups=(-1 if groups is None else groups), length_last=length_last, y=y, count=cnt, mean=mean, rstd=rstd)

    # ---- module level: state dicts and forward of the reference norm modules --------
    t = tsn.TimestepNorm(10, num_groups=None, prior_count=2).eval()
    with torch.no_grad():
        t.prior_mean.normal_(0, 0.1, generator=gen)
        t.prior_logv.normal_(0, 0.1, generator=gen)
        t.weight.normal_(0, 0.1, generator=gen)
        t.bias.normal_(0, 0.1, generator=gen)
        x = torch.randn(2, 24, 10, generator=gen)
        st = {}
        y_a = t(x[:, :16].contiguous(), None, st)
        y_b = t(x[:, 16:].contiguous(), None, st)
        y_full = t(x, None, None)
    sd = {("sd_" + k): v for k, v in t.state_dict().items()}
    npz("tsn_module", x=x, y_full=y_full, y_chunked=torch.cat([y_a, y_b], 1), **sd)

    s = sqn.SequenceNorm(6, num_groups=None).eval()
    with torch.no_grad():
        s.weight.normal_(0, 0.1, generator=gen)
        s.bias.normal_(0, 0.1, generator=gen)
        x = torch.randn(2, 6, 20, generator=gen)
        mask = right_pad_mask(gen, 2, 20, 0.5)
        y = s(x, mask)
    sd = {("sd_" + k): v for k, v in s.state_dict().items()}
    npz("sqn_module", x=x, mask=mask, y=y, **sd)

    m = cema.MultiHeadComplexEMA(4, ndim=16)
    print("cema state_dict:", {k: tuple(v.shape) for k, v in m.state_dict().items()})


def backward_fixtures():
    """Gradients produced by the reference: its CPU backward ops for the norms, and autograd
    through MultiHeadComplexEMA (ema_parameters_bwd C++ op + the Python FFT convolution) for the
    EMA.  Real-EMA parameter gradients follow from the rotation-off mapping: the kernel depends
    on gamma * beta only, so dgamma = dgamma'[..., 0] * beta and dbeta = dgamma'[..., 0] * gamma."""
    ops, cema, tsn, sqn = import_reference()
    gen = torch.Generator().manual_seed(20251126)

    for tag, (bsz, dim, length, ndim, bidir, shift, pad) in {
        "ema_bwd_uni": (3, 6, 45, 16, False, True, 0.3),
        "ema_bwd_uni_n3": (2, 5, 40, 3, False, True, 0.0),
        "ema_bwd_bidir_shift": (2, 5, 37, 16, True, True, 0.4),
        "ema_bwd_bidir_noshift": (2, 4, 32, 16, True, False, 0.3),
    }.items():
        params = ema_params(gen, dim, ndim, bidir)
        x = torch.randn(bsz, dim, length, generator=gen).requires_grad_(True)
        dy = torch.randn(bsz, dim, length, generator=gen)
        mask = right_pad_mask(gen, bsz, length, pad) if pad > 0 else None
        m = cema_from_real(cema, dim, ndim, params, bidirectional=bidir, truncation=None, shift=shift).train()
        y = m(x, mask, None)
        (y * dy).sum().backward()
        g0 = m.gamma.grad[:, :, 0]
        alpha, delta, beta, gamma, omega = params
        npz(tag, x=x, dy=dy, alpha=alpha, delta=delta, beta=beta, gamma=gamma, omega=omega,
            mask=(mask if mask is not None else np.zeros((0,), bool)), bidirectional=bidir, shift=shift, y=y,
            dx=x.grad, dalpha=m.alpha.grad, ddelta=m.delta.grad, dbeta=(g0 * gamma).unsqueeze(-1),
            dgamma=g0 * beta.squeeze(-1), domega=m.omega.grad.view(dim))

    for tag, (bsz, length, feat, groups, pad, prior) in {
        "tsn_bwd_plain": (3, 33, 9, None, 0.4, 2),
        "tsn_bwd_plain_nomask": (2, 40, 6, None, 0.0, 3),
        "tsn_bwd_group": (3, 27, 12, 3, 0.4, 0),
        "tsn_bwd_group_prior": (2, 18, 70, 2, 0.0, 2),
    }.items():
        x = torch.randn(bsz, length, feat, generator=gen) * 1.5 + 0.2
        dy = torch.randn(bsz, length, feat, generator=gen)
        mask = right_pad_mask(gen, bsz, length, pad) if pad > 0 else None   # right padding only
        ng = feat if groups is None else groups
        prev_count = torch.full((bsz,), prior, dtype=torch.int64)
        prev_mean = torch.randn(bsz, ng, generator=gen) * 0.1 if prior else torch.zeros(bsz, ng)
        prev_var = torch.rand(bsz, ng, generator=gen) + 0.5 if prior else torch.ones(bsz, ng)
        gamma = torch.randn(feat, generator=gen) * 0.1 + 1.0
        beta = torch.randn(feat, generator=gen) * 0.1
        dmean = torch.randn(bsz, ng, generator=gen)
        dvar = torch.randn(bsz, ng, generator=gen)
        if groups is None:
            y, cnt, mean, var, cm, cr = ops.timestep_norm_fwd(x, prev_count, prev_mean, prev_var, gamma, beta, mask, 1e-5)
            dx, dpm, dpv, dg, db = ops.timestep_norm_bwd(dy, dmean, dvar, x, prev_mean, cnt, cm, cr, gamma, mask)
        else:
            y, cnt, mean, var, gm, cm, cr = ops.group_timestep_norm_fwd(x, prev_count, prev_mean, prev_var, gamma,
                                                                        beta, mask, groups, 1e-5)
            dx, dpm, dpv, dg, db = ops.group_timestep_norm_bwd(dy, dmean, dvar, x, prev_mean, cnt, gm, cm, cr,
                                                               gamma, mask, groups)
        npz(tag, x=x, dy=dy, mask=(mask if mask is not None else np.zeros((0,), bool)), prev_count=prev_count,
            prev_mean=prev_mean, prev_var=prev_var, gamma=gamma, beta=beta, dmean=dmean, dvar=dvar,
            groups=(-1 if groups is None else groups), dx=dx, dprev_mean=dpm, dprev_var=dpv, dgamma=dg, dbeta=db)

    for tag, (bsz, feat, length, length_last, groups) in {
        "sqn_bwd_bhl_group": (3, 12, 41, True, 3),
        "sqn_bwd_blh_group": (2, 12, 38, False, 4),
    }.items():
        shape = (bsz, feat, length) if length_last else (bsz, length, feat)
        x = torch.randn(*shape, generator=gen) * 2.0 - 0.5
        dy = torch.randn(*shape, generator=gen)
        mask = right_pad_mask(gen, bsz, length, 0.5)
        gamma = torch.randn(feat, generator=gen) * 0.1 + 1.0
        beta = torch.randn(feat, generator=gen) * 0.1
        y, cnt, mean, rstd = ops.group_sequence_norm_fwd(x, gamma, beta, mask, groups, 1e-5, length_last)
        dx, dg, db = ops.group_sequence_norm_bwd(dy, x, cnt, mean, rstd, gamma, mask, groups, length_last)
        npz(tag, x=x, dy=dy, mask=mask, gamma=gamma, beta=beta, length_last=length_last, groups=groups, dx=dx,
            dgamma=dg, dbeta=db)

    for tag, (bsz, feat, length, length_last, pad) in {
        "sqn_bwd_bhl": (3, 6, 41, True, 0.5),
        "sqn_bwd_blh": (3, 7, 38, False, 0.5),
    }.items():
        shape = (bsz, feat, length) if length_last else (bsz, length, feat)
        x = torch.randn(*shape, generator=gen) * 2.0 - 0.5
        dy = torch.randn(*shape, generator=gen)
        mask = right_pad_mask(gen, bsz, length, pad)
        gamma = torch.randn(feat, generator=gen) * 0.1 + 1.0
        beta = torch.randn(feat, generator=gen) * 0.1
        y, cnt, mean, rstd = ops.sequence_norm_fwd(x, gamma, beta, mask, 1e-5, length_last)
        dx, dg, db = ops.sequence_norm_bwd(dy, x, cnt, mean, rstd, gamma, mask, length_last)
        npz(tag, x=x, dy=dy, mask=mask, gamma=gamma, beta=beta, length_last=length_last, dx=dx, dgamma=dg, dbeta=db)


def cema_fixtures():
    """MultiHeadComplexEMA as the reference ships it (rotation on, default init)."""
    ops, cema, tsn, sqn = import_reference()
    gen = torch.Generator().manual_seed(20251127)
    torch.manual_seed(20251127)   # reset_parameters draws from the global generator

    def params_of(m):
        return dict(alpha=m.alpha, delta=m.delta, theta=m.theta, gamma=m.gamma, omega=m.omega)

    for tag, (bsz, dim, length, ndim, bidir, shift, trunc, pad) in {
        "cema_uni_n16": (3, 8, 50, 16, False, True, None, 0.25),
        "cema_uni_n3": (2, 5, 33, 3, False, True, None, 0.0),
        "cema_bidir_shift": (3, 6, 41, 16, True, True, None, 0.5),
        "cema_bidir_noshift": (2, 6, 32, 16, True, False, None, 0.3),
        "cema_bidir_trunc": (2, 4, 40, 16, True, True, 7, 0.3),
    }.items():
        m = cema.MultiHeadComplexEMA(dim, ndim=ndim, bidirectional=bidir, truncation=trunc, shift=shift).eval()
        with torch.no_grad():
            m.gamma[:, :, 1].normal_(0, 1, generator=gen)   # exercise the imaginary output weights too
            x = torch.randn(bsz, dim, length, generator=gen)
            mask = right_pad_mask(gen, bsz, length, pad) if pad > 0 else None
            y = m(x, mask, None)
            k, _ = m.kernel(length, None)
        npz(tag, x=x, mask=(mask if mask is not None else np.zeros((0,), bool)), y=y, kernel=k,
            bidirectional=bidir, shift=shift, truncation=(-1 if trunc is None else trunc), **params_of(m))

    # incremental: chunks through the reference CPU ops, then the closed-form single step
    bsz, dim, length, ndim, chunk = 3, 6, 48, 16, 16
    m = cema.MultiHeadComplexEMA(dim, ndim=ndim).eval()
    fftconv = sys.modules["fairseq.modules.fused_ops.fftconv"]._fftconv_fwd
    with torch.no_grad():
        m.gamma[:, :, 1].normal_(0, 1, generator=gen)
        x = torch.randn(bsz, dim, length, generator=gen)
        pc, qc, gc = m._calc_coeffs()
        hh, ys, hs = None, [], []
        for i in range(0, length, chunk):
            xc = x[..., i:i + chunk].contiguous()
            w, b, _ = ops.ema_parameters_fwd(pc, qc.log(), gc, hh, chunk)
            yy = fftconv(xc, w)[0]
            if b is not None:
                yy = yy + b
            hh, _ = ops.ema_hidden_fwd(xc, pc, qc.log(), hh)
            ys.append(yy + xc * m.omega)
            hs.append(torch.view_as_real(hh).clone())
        y1, h1 = m.one_step(x[..., :1], hx=None)
        y2, h2 = m.one_step(x[..., 1:2], hx=h1)
        y_full = m(x, None, None)
    npz("cema_incremental", x=x, chunk=chunk, y=torch.cat(ys, -1), y_full=y_full, states=torch.stack(hs),
        step_y1=y1, step_h1=torch.view_as_real(h1), step_y2=y2, step_h2=torch.view_as_real(h2), **params_of(m))


def cema_backward_fixtures():
    """Gradients of MultiHeadComplexEMA by autograd through the reference module itself
    (ema_parameters_bwd C++ op + the Python FFT convolution backward)."""
    ops, cema, tsn, sqn = import_reference()
    gen = torch.Generator().manual_seed(20251128)
    torch.manual_seed(20251128)
    for tag, (bsz, dim, length, ndim, bidir, shift, pad) in {
        "cema_bwd_uni": (3, 6, 45, 16, False, True, 0.3),
        "cema_bwd_uni_n3": (2, 5, 40, 3, False, True, 0.0),
        "cema_bwd_bidir_shift": (2, 5, 37, 16, True, True, 0.4),
        "cema_bwd_bidir_noshift": (2, 4, 32, 16, True, False, 0.3),
    }.items():
        m = cema.MultiHeadComplexEMA(dim, ndim=ndim, bidirectional=bidir, shift=shift).train()
        with torch.no_grad():
            m.gamma[:, :, 1].normal_(0, 1, generator=gen)
        x = torch.randn(bsz, dim, length, generator=gen).requires_grad_(True)
        dy = torch.randn(bsz, dim, length, generator=gen)
        mask = right_pad_mask(gen, bsz, length, pad) if pad > 0 else None
        y = m(x, mask, None)
        (y * dy).sum().backward()
        npz(tag, x=x, dy=dy, mask=(mask if mask is not None else np.zeros((0,), bool)), bidirectional=bidir,
            shift=shift, y=y, alpha=m.alpha, delta=m.delta, theta=m.theta, gamma=m.gamma, omega=m.omega,
            dx=x.grad, dalpha=m.alpha.grad, ddelta=m.delta.grad, dtheta=m.theta.grad, dgamma=m.gamma.grad,
            domega=m.omega.grad)


def truncated_backward_fixtures():
    """Gradients of the bidirectional layers with a truncated kernel (autograd through the reference
    module: the kernel is built for min(truncation, L) taps, fused_ops/fftconv.py does the rest)."""
    ops, cema, tsn, sqn = import_reference()
    gen = torch.Generator().manual_seed(20251129)
    bsz, dim, length, ndim, trunc = 2, 5, 40, 16, 7
    for tag, shift, pad in (("ema_bwd_bidir_trunc", True, 0.3), ("ema_bwd_bidir_trunc_noshift", False, 0.0)):
        params = ema_params(gen, dim, ndim, True)
        x = torch.randn(bsz, dim, length, generator=gen).requires_grad_(True)
        dy = torch.randn(bsz, dim, length, generator=gen)
        mask = right_pad_mask(gen, bsz, length, pad) if pad > 0 else None
        m = cema_from_real(cema, dim, ndim, params, bidirectional=True, truncation=trunc, shift=shift).train()
        y = m(x, mask, None)
        (y * dy).sum().backward()
        g0 = m.gamma.grad[:, :, 0]
        alpha, delta, beta, gamma, omega = params
        npz(tag, x=x, dy=dy, alpha=alpha, delta=delta, beta=beta, gamma=gamma, omega=omega,
            mask=(mask if mask is not None else np.zeros((0,), bool)), bidirectional=True, shift=shift,
            truncation=trunc, y=y, dx=x.grad, dalpha=m.alpha.grad, ddelta=m.delta.grad,
            dbeta=(g0 * gamma).unsqueeze(-1), dgamma=g0 * beta.squeeze(-1), domega=m.omega.grad.view(dim))
    for tag, shift, pad in (("cema_bwd_bidir_trunc", True, 0.3), ("cema_bwd_bidir_trunc_noshift", False, 0.0)):
        m = cema.MultiHeadComplexEMA(dim, ndim=ndim, bidirectional=True, truncation=trunc, shift=shift).train()
        with torch.no_grad():
            m.alpha.normal_(0, 0.2, generator=gen)
            m.delta.normal_(0, 0.2, generator=gen)
            m.theta.normal_(0, 1.0, generator=gen)
            m.gamma.normal_(0, 1, generator=gen)
            m.omega.normal_(0, 1, generator=gen)
        x = torch.randn(bsz, dim, length, generator=gen).requires_grad_(True)
        dy = torch.randn(bsz, dim, length, generator=gen)
        mask = right_pad_mask(gen, bsz, length, pad) if pad > 0 else None
        y = m(x, mask, None)
        (y * dy).sum().backward()
        npz(tag, x=x, dy=dy, mask=(mask if mask is not None else np.zeros((0,), bool)), bidirectional=True,
            shift=shift, truncation=trunc, y=y, alpha=m.alpha, delta=m.delta, theta=m.theta, gamma=m.gamma,
            omega=m.omega, dx=x.grad, dalpha=m.alpha.grad, ddelta=m.delta.grad, dtheta=m.theta.grad,
            dgamma=m.gamma.grad, domega=m.omega.grad)


def block_fixtures():
    """The reference's own MovingAverageGatedAttention (the Mega block that calls the EMA layer, the
    norm and the attention softmax), built from the reference's unmodified Python on top of its own
    modules and CPU operators: input, state dict and output in fp32.  The GPU test rebuilds the same
    block class on top of this package's modules from the same state dict.

    Configuration: moving_layer='cema' (the reference's real-valued MultiHeadEMA does not run in the
    snapshot), moving_act='silu', grouped TimestepNorm (the per-feature form cannot be constructed
    through the block, whose TimestepNorm call leaves prior_count at 0), rotary positions, chunked
    causal softmax attention with the causal mask passed as attn_mask, as the decoder layer does."""
    ops, cema, tsn, sqn = import_reference()
    import types
    import torch.nn.functional as F
    fs = os.path.join(REF, "fairseq")

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(fs, rel))
        m = importlib.util.module_from_spec(spec)
        sys.modules[name] = m
        spec.loader.exec_module(m)
        return m

    utils = types.ModuleType("fairseq.utils")
    utils.softmax = lambda x, dim, onnx_trace=False: F.softmax(x.float(), dim=dim, dtype=torch.float32)
    sys.modules["fairseq.utils"] = utils
    sys.modules["fairseq"].utils = utils
    load("fairseq.modules.fairseq_dropout", "modules/fairseq_dropout.py")
    load("fairseq.modules.relative_positional_bias", "modules/relative_positional_bias.py")
    load("fairseq.modules.norm_layer.layer_norm", "modules/norm_layer/layer_norm.py")
    load("fairseq.modules.exponential_moving_average", "modules/exponential_moving_average.py")
    load("fairseq.modules.efficient_attention", "modules/efficient_attention.py")
    load("fairseq.modules.attention_softmax", "modules/attention_softmax.py")
    mag = load("fairseq.modules.moving_average_gated_attention", "modules/moving_average_gated_attention.py")
    nffn = load("fairseq.modules.normalized_feedforward_network", "modules/normalized_feedforward_network.py")

    dim, zdim, hdim, ndim, chunk, groups = 64, 16, 128, 16, 32, 8
    for name, bsz, length, padded in (("mega_block_causal", 2, 96, False), ("mega_block_causal_padded", 3, 64, True)):
        torch.manual_seed(20 + length)
        gen = torch.Generator().manual_seed(77 + length)
        blk = mag.MovingAverageGatedAttention(dim, zdim, hdim, ndim, chunk_size=chunk, moving_layer='cema',
                                              moving_act='silu', norm_num_groups=groups, rel_pos_bias='rotary',
                                              efficient_attn=False).eval()
        with torch.no_grad():   # leave the all-zero initialisations so that every parameter matters
            blk.norm.weight.normal_(0, 0.1, generator=gen)
            blk.norm.bias.normal_(0, 0.1, generator=gen)
            blk.gamma.normal_(0, 0.2, generator=gen)
            blk.beta.normal_(0, 0.2, generator=gen)
            blk.v_proj.bias.normal_(0, 0.1, generator=gen)
            blk.mx_proj.bias.normal_(0, 0.1, generator=gen)
            blk.mx_proj.weight.mul_(8.0)
            blk.v_proj.weight.mul_(8.0)
            blk.h_proj.weight.mul_(8.0)
        x = torch.randn(bsz, length, dim, generator=gen)
        mask = right_pad_mask(gen, bsz, length, 0.4) if padded else None
        causal = torch.tril(torch.ones(chunk, chunk))
        attn_mask = torch.zeros(chunk, chunk).masked_fill(causal == 0, float("-inf"))
        with torch.no_grad():
            y, _ = blk(x, padding_mask=mask, attn_mask=attn_mask)
        arrs = {"x": x, "y": y, "mask": mask if mask is not None else torch.zeros(0),
                "dims": torch.tensor([dim, zdim, hdim, ndim, chunk, groups])}
        for k, v in blk.state_dict().items():
            arrs["sd." + k] = v
        npz(name, **arrs)
    # the normalised feed-forward network that follows the block in a Mega layer (layer norm, SiLU MLP)
    torch.manual_seed(5)
    gen = torch.Generator().manual_seed(5)
    ff = nffn.NormalizedFeedForwardNetwork(dim, 96, norm_type='layernorm').eval()
    with torch.no_grad():
        for prm in ff.parameters():
            if prm.dim() == 1:
                prm.normal_(0, 0.1, generator=gen)
    x = torch.randn(2, 40, dim, generator=gen)
    with torch.no_grad():
        y = ff(x)
    arrs = {"x": x, "y": y}
    for k, v in ff.state_dict().items():
        arrs["sd." + k] = v
    npz("mega_nffn", **arrs)


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    if which in ("all", "block"):
        block_fixtures()
    if which in ("all", "backward_truncated"):
        truncated_backward_fixtures()
    if which in ("all", "cema_backward"):
        cema_backward_fixtures()
    if which in ("all", "cema"):
        cema_fixtures()
    if which in ("all", "forward"):
        main()
    if which in ("all", "backward"):
        backward_fixtures()
