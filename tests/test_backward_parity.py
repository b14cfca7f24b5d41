"""GPU parity of the backward kernels (through the C ABI) against the reference's gradients
(golden fixtures) and against torch autograd through the float64 oracle.
Tolerances (relative L2): fp32 input gradients 2e-5, fp32 parameter gradients 1e-4 (sums over
batch and length in fp32 with atomic adds), bf16 activations 2e-2."""
import pytest
import torch

from _util import golden, make_ema_params, opt_mask, rel_l2, right_pad_mask

pytestmark = pytest.mark.gpu


def _mods():
    import fairseq_apollo_b200 as M
    from oracle import mega_oracle as O
    return M, O


def _leaf(t):
    return t.double().clone().requires_grad_(True)


def _ema_module(M, dim, ndim, params, bidirectional=False, shift=True, truncation=None):
    m = M.MultiHeadEMA(dim, ndim=ndim, bidirectional=bidirectional, shift=shift, truncation=truncation).cuda().train()
    with torch.no_grad():
        for dst, src in zip((m.alpha, m.delta, m.beta, m.gamma, m.omega), params):
            dst.copy_(src)
    return m


@pytest.mark.parametrize("name", ["ema_bwd_uni", "ema_bwd_uni_n3", "ema_bwd_bidir_shift", "ema_bwd_bidir_noshift",
                                  "ema_bwd_bidir_trunc", "ema_bwd_bidir_trunc_noshift"])
def test_ema_golden(name):
    M, _ = _mods()
    g = golden(name)
    params = [g[k] for k in ("alpha", "delta", "beta", "gamma", "omega")]
    m = _ema_module(M, g["x"].shape[1], g["alpha"].shape[1], params, bool(g["bidirectional"]), bool(g["shift"]),
                    g.get("truncation"))
    x = g["x"].cuda().requires_grad_(True)
    mask = opt_mask(g["mask"])
    y = m(x, None if mask is None else mask.cuda())
    assert rel_l2(y, g["y"]) < 1e-5
    (y * g["dy"].cuda()).sum().backward()
    assert rel_l2(x.grad, g["dx"]) < 2e-5
    for t, k in ((m.alpha, "dalpha"), (m.delta, "ddelta"), (m.beta, "dbeta"), (m.gamma, "dgamma"),
                 (m.omega, "domega")):
        assert rel_l2(t.grad, g[k]) < 1e-4, k


@pytest.mark.parametrize("bsz,dim,length,ndim,bidir,shift", [
    (1, 1, 1, 16, False, True), (2, 7, 33, 16, False, True), (3, 5, 130, 2, False, True),
    (2, 9, 65, 32, False, True), (2, 6, 40, 16, True, True), (2, 3, 31, 5, True, False), (9, 33, 17, 1, True, True),
    # channel counts the streamed (TMA) backward kernel accepts: rows of 16-byte multiples
    (2, 16, 70, 16, False, True), (3, 72, 257, 3, False, True), (2, 136, 33, 16, False, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ema_grid(bsz, dim, length, ndim, bidir, shift, dtype):
    """Module autograd against autograd through the fp64 recurrence; interior pads; x given as the
    (B, D, L) view of (B, L, D) memory, as the Mega block hands it over."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(dim * 100 + length)
    params = make_ema_params(gen, dim, ndim, bidir)
    x0 = torch.randn(bsz, length, dim, generator=gen).to(dtype)
    dy = torch.randn(bsz, dim, length, generator=gen).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.4)
    if length > 4:
        mask[0, 2] = True
    leaves = [_leaf(t) for t in params]
    xr = _leaf(x0.float().transpose(1, 2))
    yr = O.ema_forward_recurrence(xr, *leaves, mask, bidirectional=bidir, shift=shift)
    (yr * dy.double()).sum().backward()
    m = _ema_module(M, dim, ndim, params, bidir, shift)
    xd = x0.cuda().requires_grad_(True)
    y = m(xd.transpose(1, 2), mask.cuda())
    (y.float() * dy.cuda().float()).sum().backward()
    tol_x, tol_p = (2e-5, 1e-4) if dtype == torch.float32 else (2e-2, 2e-2)
    assert rel_l2(y.float(), yr) < (1e-5 if dtype == torch.float32 else 1e-2)
    assert rel_l2(xd.grad.float().transpose(1, 2), xr.grad) < tol_x
    for t, r, k in zip((m.alpha, m.delta, m.beta, m.gamma, m.omega), leaves, "adbgo"):
        assert rel_l2(t.grad, r.grad) < tol_p, k

@pytest.mark.parametrize("bsz,dim,length,ndim,shift,trunc", [(2, 6, 40, 16, True, 5), (3, 5, 33, 3, False, 9),
                                                             (2, 9, 70, 32, True, 1), (2, 4, 20, 16, True, 64)])
@pytest.mark.parametrize("complex_poles", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_truncated_kernel_grid(bsz, dim, length, ndim, shift, trunc, complex_poles, dtype):
    """Bidirectional layers with a truncated kernel (taps 0 .. trunc - 1; trunc >= L is the full
    kernel) under autograd against autograd through the fp64 recurrence, interior pads included."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(dim * 100 + length + trunc)
    torch.manual_seed(dim * 100 + length + trunc)
    x0 = torch.randn(bsz, length, dim, generator=gen).to(dtype)
    dy = torch.randn(bsz, dim, length, generator=gen).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.4)
    mask[0, 2] = True
    if complex_poles:
        m = M.MultiHeadComplexEMA(dim, ndim=ndim, bidirectional=True, shift=shift, truncation=trunc).cuda().train()
        with torch.no_grad():
            m.gamma[:, :, 1].normal_(0, 1)
        names = ("alpha", "delta", "theta", "gamma", "omega")
        ref_fn = O.cema_forward_recurrence
    else:
        m = _ema_module(M, dim, ndim, make_ema_params(gen, dim, ndim, True), True, shift, trunc)
        names = ("alpha", "delta", "beta", "gamma", "omega")
        ref_fn = O.ema_forward_recurrence
    leaves = [_leaf(getattr(m, k).detach().cpu()) for k in names]
    xr = _leaf(x0.float().transpose(1, 2))
    yr = ref_fn(xr, *leaves, mask, bidirectional=True, shift=shift, truncation=trunc)
    (yr * dy.double()).sum().backward()
    xd = x0.cuda().requires_grad_(True)
    y = m(xd.transpose(1, 2), mask.cuda())
    (y.float() * dy.cuda().float()).sum().backward()
    tol_x, tol_p = (2e-5, 1e-4) if dtype == torch.float32 else (2e-2, 2e-2)
    assert rel_l2(y.float(), yr) < (1e-5 if dtype == torch.float32 else 1e-2)
    assert rel_l2(xd.grad.float().transpose(1, 2), xr.grad) < tol_x
    for k, r in zip(names, leaves):
        assert rel_l2(getattr(m, k).grad, r.grad) < tol_p, k


@pytest.mark.parametrize("dim,channel_contiguous", [(6, False), (16, True)])
def test_ema_state_gradients(dim, channel_contiguous):
    """Carried state in, state out: gradients w.r.t. the incoming state and through the returned
    one (operator level; the module keeps states out of autograd); the generic kernel and, on
    (B, L, D) memory, the streamed one."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(5)
    bsz, length, ndim = 2, 29, 16
    params = make_ema_params(gen, dim, ndim)
    x = torch.randn(bsz, dim, length, generator=gen)
    h0 = torch.randn(bsz, dim, ndim, generator=gen) * 0.3
    dy = torch.randn(bsz, dim, length, generator=gen)
    dh = torch.randn(bsz, dim, ndim, generator=gen)
    mask = right_pad_mask(gen, bsz, length, 0.3)
    leaves = [_leaf(t) for t in params]
    xr, hr = _leaf(x), _leaf(h0)
    yr, hn = O.ema_forward_recurrence(xr, *leaves, mask, h=hr, return_state=True)
    ((yr * dy.double()).sum() + (hn * dh.double()).sum()).backward()
    p, q, g = O.ema_coeffs(*[t.detach() for t in leaves[:4]], dtype=torch.float64)
    pr, qr, gr = [_leaf(t) for t in (p, q, g)]
    # coefficient-level gradients of the oracle for comparison with the kernel's (dp, dq, dgamma_hat)
    xs = x.double() * (1.0 - mask.unsqueeze(1).double())
    st = h0.double()
    tot = 0.0
    for t in range(length):
        st = qr * st + pr * xs[:, :, t:t + 1]
        tot = tot + ((st * gr).sum(-1) * dy[:, :, t].double()).sum()
    (tot + (st * dh.double()).sum()).backward()
    xd, dyd = x.cuda(), dy.cuda()
    if channel_contiguous:  # (B, D, L) views of (B, L, D) memory
        xd = xd.transpose(1, 2).contiguous().transpose(1, 2)
        dyd = dyd.transpose(1, 2).contiguous().transpose(1, 2)
    dx, dp, dq, dg, dom, dh_in = M.ops.ema_backward(dyd, xd, p.float().cuda(), q.float().cuda(),
                                                    g.float().cuda(), params[4].cuda(), mask.cuda(), h0.cuda(),
                                                    dh.cuda(), want_dh_in=True)
    assert rel_l2(dx, xr.grad) < 2e-5
    assert rel_l2(dh_in, hr.grad) < 2e-5
    assert rel_l2(dp, pr.grad) < 1e-4 and rel_l2(dq, qr.grad) < 1e-4 and rel_l2(dg, gr.grad) < 1e-4
    assert rel_l2(dom, leaves[4].grad) < 1e-4


@pytest.mark.parametrize("name", ["tsn_bwd_plain", "tsn_bwd_plain_nomask", "tsn_bwd_group", "tsn_bwd_group_prior"])
def test_tsn_golden(name):
    M, _ = _mods()
    g = golden(name)
    mask = opt_mask(g["mask"])
    groups = None if g["groups"] < 0 else g["groups"]
    md = None if mask is None else mask.cuda()
    y, cnt, mean, var, cm, cr, gm = M.ops.timestep_norm_fwd_train(
        g["x"].cuda(), g["prev_count"].cuda(), g["prev_mean"].cuda(), g["prev_var"].cuda(), g["gamma"].cuda(),
        g["beta"].cuda(), md, 1e-5, groups)
    dx, dpm, dpv, dgamma, dbeta = M.ops.timestep_norm_bwd(
        g["dy"].cuda(), g["dmean"].cuda(), g["dvar"].cuda(), g["x"].cuda(), g["prev_mean"].cuda(), cnt, cm, cr, gm,
        g["gamma"].cuda(), md, groups)
    assert rel_l2(dx, g["dx"]) < 2e-5
    assert rel_l2(dpm, g["dprev_mean"]) < 2e-5 and rel_l2(dpv, g["dprev_var"]) < 2e-5
    assert rel_l2(dgamma, g["dgamma"]) < 1e-4 and rel_l2(dbeta, g["dbeta"]) < 1e-4
    if mask is not None:
        assert (dx.cpu()[mask] == 0).all()


@pytest.mark.parametrize("bsz,length,feat,groups", [(1, 1, 1, None), (2, 130, 33, None), (9, 17, 128, None),
                                                     (2, 50, 64, 4), (3, 33, 96, 3), (2, 20, 70, 1),
                                                     (2, 70, 128, 16), (2, 257, 128, 2), (3, 100, 192, 6)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_tsn_module_grid(bsz, length, feat, groups, dtype):
    """Module autograd (prior statistics, weight, bias and x) against autograd through the fp64
    oracle, with interior pads."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(length * 7 + feat)
    x = (torch.randn(bsz, length, feat, generator=gen) * 1.5 + 0.2).to(dtype)
    dy = torch.randn(bsz, length, feat, generator=gen).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.4)
    if length > 4:
        mask[0, 2] = True
    ng = feat if groups is None else groups
    prior = 2
    mod = M.TimestepNorm(feat, groups, prior_count=prior).cuda().train()
    with torch.no_grad():
        mod.prior_mean.copy_(torch.randn(ng, generator=gen) * 0.1)
        mod.prior_logv.copy_(torch.randn(ng, generator=gen) * 0.1)
        mod.weight.copy_(torch.randn(feat, generator=gen) * 0.1)
        mod.bias.copy_(torch.randn(feat, generator=gen) * 0.1)
    pm, plv, w, b = [_leaf(t.detach().cpu()) for t in (mod.prior_mean, mod.prior_logv, mod.weight, mod.bias)]
    xr = _leaf(x.float())
    args = (xr, torch.full((bsz,), prior, dtype=torch.int64), pm.expand(bsz, -1), torch.exp(plv).expand(bsz, -1),
            w + 1.0, b, mask)
    if groups is None:
        yr = O.timestep_norm(*args, acc_dtype=torch.float64)[0]
    else:
        yr = O.group_timestep_norm(*args, groups, acc_dtype=torch.float64)[0]
    (yr * dy.double()).sum().backward()
    xd = x.cuda().requires_grad_(True)
    y = mod(xd, mask.cuda())
    (y.float() * dy.cuda().float()).sum().backward()
    f32 = dtype == torch.float32
    assert rel_l2(y.float(), yr) < (1e-5 if f32 else 1e-2)
    assert rel_l2(xd.grad.float(), xr.grad) < (5e-5 if f32 else 2e-2)
    assert (xd.grad.cpu()[mask] == 0).all()
    for t, r, k in ((mod.prior_mean, pm, "pm"), (mod.prior_logv, plv, "plv"), (mod.weight, w, "w"), (mod.bias, b, "b")):
        assert rel_l2(t.grad, r.grad) < (2e-4 if f32 else 2e-2), k


@pytest.mark.parametrize("name", ["sqn_bwd_bhl", "sqn_bwd_blh", "sqn_bwd_bhl_group", "sqn_bwd_blh_group"])
def test_sqn_golden(name):
    M, _ = _mods()
    g = golden(name)
    ll = bool(g["length_last"])
    groups = g.get("groups")
    mask = g["mask"].bool().cuda()
    y, cnt, mean, rstd = M.ops.sequence_norm_fwd(g["x"].cuda(), g["gamma"].cuda(), g["beta"].cuda(), mask, 1e-5, ll,
                                                 groups)
    dx, dgamma, dbeta = M.ops.sequence_norm_bwd(g["dy"].cuda(), g["x"].cuda(), cnt, mean, rstd, g["gamma"].cuda(),
                                                mask, ll, groups)
    assert rel_l2(dx, g["dx"]) < 2e-5
    assert rel_l2(dgamma, g["dgamma"]) < 1e-4 and rel_l2(dbeta, g["dbeta"]) < 1e-4


@pytest.mark.parametrize("bsz,feat,length,groups", [(1, 1, 1, None), (2, 5, 300, None), (3, 64, 1000, None),
                                                     (2, 7, 4100, None), (2, 48, 500, 4), (3, 30, 77, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sqn_module_grid(bsz, feat, length, groups, dtype):
    M, O = _mods()
    gen = torch.Generator().manual_seed(length + feat)
    x = (torch.randn(bsz, feat, length, generator=gen) * 2 - 0.5).to(dtype)
    dy = torch.randn(bsz, feat, length, generator=gen).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.5)
    if length > 4:
        mask[0, 1] = True
    mod = M.SequenceNorm(feat, groups).cuda().train()
    with torch.no_grad():
        mod.weight.copy_(torch.randn(feat, generator=gen) * 0.1)
        mod.bias.copy_(torch.randn(feat, generator=gen) * 0.1)
    w, b = _leaf(mod.weight.detach().cpu()), _leaf(mod.bias.detach().cpu())
    xr = _leaf(x.float())
    yr = O.sequence_norm(xr, w + 1.0, b, mask, groups, 1e-5, True, acc_dtype=torch.float64)[0]
    (yr * dy.double()).sum().backward()
    xd = x.cuda().requires_grad_(True)
    y = mod(xd, mask.cuda())
    (y.float() * dy.cuda().float()).sum().backward()
    f32 = dtype == torch.float32
    assert rel_l2(xd.grad.float(), xr.grad) < (5e-5 if f32 else 2e-2)
    assert rel_l2(mod.weight.grad, w.grad) < (2e-4 if f32 else 2e-2)
    assert rel_l2(mod.bias.grad, b.grad) < (2e-4 if f32 else 2e-2)


def test_block_training_step():
    """TimestepNorm -> EMA (+ SiLU) through the fused helper with autograd on: gradients of every
    parameter against the oracle chain."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(11)
    bsz, length, dim, ndim = 2, 70, 24, 16
    params = make_ema_params(gen, dim, ndim)
    x = torch.randn(bsz, length, dim, generator=gen)
    dy = torch.randn(bsz, length, dim, generator=gen)
    mask = right_pad_mask(gen, bsz, length, 0.3)
    norm = M.TimestepNorm(dim, prior_count=2).cuda().train()
    move = _ema_module(M, dim, ndim, params)
    xd = x.cuda().requires_grad_(True)
    y = M.timestep_norm_ema(norm, move, xd, mask.cuda(), None, 'silu')
    (y * dy.cuda()).sum().backward()
    leaves = [_leaf(t) for t in params]
    xr = _leaf(x)
    w, b = _leaf(torch.zeros(dim)), _leaf(torch.zeros(dim))
    xn = O.timestep_norm(xr, torch.full((bsz,), 2, dtype=torch.int64), torch.zeros(bsz, dim, dtype=torch.float64),
                         torch.ones(bsz, dim, dtype=torch.float64), w + 1.0, b, mask, acc_dtype=torch.float64)[0]
    yr = O.ema_forward_recurrence(xn.transpose(1, 2), *leaves, mask, silu=True).transpose(1, 2)
    (yr * dy.double()).sum().backward()
    assert rel_l2(y, yr) < 1e-5
    assert rel_l2(xd.grad, xr.grad) < 5e-5
    assert rel_l2(norm.weight.grad, w.grad) < 2e-4 and rel_l2(norm.bias.grad, b.grad) < 2e-4
    for t, r in zip((move.alpha, move.delta, move.beta, move.gamma, move.omega), leaves):
        assert rel_l2(t.grad, r.grad) < 2e-4


@pytest.mark.parametrize("name", ["cema_bwd_uni", "cema_bwd_uni_n3", "cema_bwd_bidir_shift", "cema_bwd_bidir_noshift",
                                  "cema_bwd_bidir_trunc", "cema_bwd_bidir_trunc_noshift"])
def test_complex_ema_golden(name):
    """MultiHeadComplexEMA under autograd against the gradients of the reference module."""
    M, _ = _mods()
    g = golden(name)
    m = M.MultiHeadComplexEMA(g["x"].shape[1], ndim=g["alpha"].shape[1], bidirectional=bool(g["bidirectional"]),
                              shift=bool(g["shift"]), truncation=g.get("truncation")).cuda().train()
    with torch.no_grad():
        for k in ("alpha", "delta", "theta", "gamma", "omega"):
            getattr(m, k).copy_(g[k])
    x = g["x"].cuda().requires_grad_(True)
    mask = opt_mask(g["mask"])
    y = m(x, None if mask is None else mask.cuda())
    assert rel_l2(y, g["y"]) < 1e-5
    (y * g["dy"].cuda()).sum().backward()
    assert rel_l2(x.grad, g["dx"]) < 2e-5
    for k in ("alpha", "delta", "theta", "gamma", "omega"):
        assert rel_l2(getattr(m, k).grad, g["d" + k]) < 1e-4, k


@pytest.mark.parametrize("bsz,dim,length,ndim,bidir,shift", [(2, 7, 33, 16, False, True), (3, 5, 130, 2, False, True),
                                                             (2, 9, 65, 32, False, True), (2, 6, 40, 16, True, True),
                                                             (2, 3, 31, 5, True, False), (2, 16, 70, 16, False, True),
                                                             (3, 72, 257, 3, False, True), (2, 136, 33, 11, False, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_complex_ema_grid(bsz, dim, length, ndim, bidir, shift, dtype):
    M, O = _mods()
    gen = torch.Generator().manual_seed(dim * 100 + length)
    torch.manual_seed(dim * 100 + length)
    m = M.MultiHeadComplexEMA(dim, ndim=ndim, bidirectional=bidir, shift=shift).cuda().train()
    with torch.no_grad():
        m.gamma[:, :, 1].normal_(0, 1)
    x0 = torch.randn(bsz, length, dim, generator=gen).to(dtype)
    dy = torch.randn(bsz, dim, length, generator=gen).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.4)
    if length > 4:
        mask[0, 2] = True
    names = ("alpha", "delta", "theta", "gamma", "omega")
    leaves = [_leaf(getattr(m, k).detach().cpu()) for k in names]
    xr = _leaf(x0.float().transpose(1, 2))
    yr = O.cema_forward_recurrence(xr, *leaves, mask, bidirectional=bidir, shift=shift)
    (yr * dy.double()).sum().backward()
    xd = x0.cuda().requires_grad_(True)
    y = m(xd.transpose(1, 2), mask.cuda())
    (y.float() * dy.cuda().float()).sum().backward()
    tol_x, tol_p = (2e-5, 1e-4) if dtype == torch.float32 else (2e-2, 2e-2)
    assert rel_l2(xd.grad.float().transpose(1, 2), xr.grad) < tol_x
    for k, r in zip(names, leaves):
        assert rel_l2(getattr(m, k).grad, r.grad) < tol_p, k
