"""GPU parity of the EMA kernels (through the C ABI) against the oracle and the golden
vectors produced by the reference.  Tolerances: relative L2 <= 1e-5 for fp32 and <= 1e-2 for
bf16 against the fp32/fp64 reference (fp16: 2e-3)."""
import pytest
import torch

from _util import golden, make_ema_params, opt_mask, rel_l2, right_pad_mask

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 2e-3}


def _mods():
    import fairseq_apollo_b200 as M
    from oracle import mega_oracle as O
    return M, O


def _coeffs(M, prm):
    return M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])


@pytest.mark.parametrize("name", ["ema_uni_n16", "ema_uni_n2", "ema_uni_pow2", "ema_bidir_shift",
                                  "ema_bidir_noshift", "ema_bidir_trunc"])
@pytest.mark.parametrize("layout", ["bdl", "bld_view"])
def test_golden(name, layout):
    M, _ = _mods()
    g = golden(name)
    prm = [g[k] for k in ("alpha", "delta", "beta", "gamma", "omega")]
    p, q, gam = _coeffs(M, prm)
    x = g["x"].cuda()
    if layout == "bld_view":
        x = x.transpose(1, 2).contiguous().transpose(1, 2)
    mask = opt_mask(g["mask"])
    trunc = None if g["truncation"] < 0 else g["truncation"]
    y = M.ops.ema_forward(x, p, q, gam, prm[4].cuda(), None if mask is None else mask.cuda(),
                          bidirectional=bool(g["bidirectional"]), shift=bool(g["shift"]), truncation=trunc)
    assert y.shape == x.shape
    assert rel_l2(y, g["y"]) < 1e-5


def test_coeffs_and_kernel_golden():
    M, O = _mods()
    g = golden("ema_uni_n16")
    prm = [g[k] for k in ("alpha", "delta", "beta", "gamma", "omega")]
    p, q, gam = _coeffs(M, prm)
    po, qo, go = O.ema_coeffs(*prm[:4])
    assert rel_l2(p, po) < 1e-6 and rel_l2(q, qo) < 1e-6 and rel_l2(gam, go) < 1e-6
    k = M.ops.ema_kernel(p, q, gam, 50)
    assert rel_l2(k, O.ema_kernel(po, qo, go, 50)) < 1e-5
    h = torch.randn(3, 8, 16, generator=torch.Generator().manual_seed(3))
    b = M.ops.ema_bias(q, gam, h.cuda(), 50)
    assert rel_l2(b, O.ema_bias(qo, go, h, 50)) < 1e-5


@pytest.mark.parametrize("bsz,dim,length,ndim", [(1, 1, 1, 16), (2, 7, 5, 16), (9, 33, 31, 16), (2, 128, 32, 16),
                                                 (3, 40, 33, 3), (2, 130, 257, 16), (1, 16, 100, 1), (2, 8, 64, 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("layout", ["bdl", "bld_view", "time_major"])
def test_grid_causal(bsz, dim, length, ndim, dtype, layout):
    M, O = _mods()
    gen = torch.Generator().manual_seed(bsz * 1000 + dim * 10 + length + ndim)
    prm = make_ema_params(gen, dim, ndim)
    x = torch.randn(bsz, dim, length, generator=gen).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.3)
    if bsz > 1:
        mask[bsz - 1] = True  # a fully padded sequence
    ref = O.ema_forward_recurrence(x.float(), *prm, mask)
    p, q, gam = _coeffs(M, prm)
    xc = x.cuda()
    if layout == "bld_view":
        xc = xc.transpose(1, 2).contiguous().transpose(1, 2)
    elif layout == "time_major":
        xc = xc.permute(2, 0, 1).contiguous().permute(1, 2, 0)
    y = M.ops.ema_forward(xc, p, q, gam, prm[4].cuda(), mask.cuda())
    assert y.stride() == xc.stride()
    assert rel_l2(y.float(), ref) < TOL[dtype]


@pytest.mark.parametrize("shift", [True, False])
@pytest.mark.parametrize("trunc", [None, 5, 1000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["bdl", "bld_view"])
def test_grid_bidirectional(shift, trunc, dtype, layout):
    M, O = _mods()
    gen = torch.Generator().manual_seed(11)
    bsz, dim, length, ndim = 3, 37, 70, 16
    prm = make_ema_params(gen, dim, ndim, bidirectional=True)
    x = torch.randn(bsz, dim, length, generator=gen).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.5)
    ref = O.ema_forward_recurrence(x.float(), *prm, mask, bidirectional=True, shift=shift, truncation=trunc)
    p, q, gam = _coeffs(M, prm)
    xc = x.cuda()
    if layout == "bld_view":
        xc = xc.transpose(1, 2).contiguous().transpose(1, 2)
    y = M.ops.ema_forward(xc, p, q, gam, prm[4].cuda(), mask.cuda(), bidirectional=True, shift=shift, truncation=trunc)
    assert rel_l2(y.float(), ref) < TOL[dtype]


def test_silu_epilogue():
    M, O = _mods()
    gen = torch.Generator().manual_seed(5)
    prm = make_ema_params(gen, 24, 16)
    x = torch.randn(2, 24, 90, generator=gen)
    ref = O.ema_forward_recurrence(x, *prm, silu=True)
    p, q, gam = _coeffs(M, prm)
    y = M.ops.ema_forward(x.cuda(), p, q, gam, prm[4].cuda(), silu=True)
    assert rel_l2(y, ref) < 1e-5


def test_incremental_golden_and_chunked():
    """Chunked calls with a carried state reproduce the reference ops chunk by chunk, and the
    full-length call; L calls of length 1 reproduce one call of length L."""
    M, O = _mods()
    g = golden("ema_incremental")
    prm = [g[k] for k in ("alpha", "delta", "beta", "gamma", "omega")]
    p, q, gam = _coeffs(M, prm)
    om = prm[4].cuda()
    x = g["x"].cuda()
    chunk = g["chunk"]
    beta = g["beta"].squeeze(-1)
    h, ys = None, []
    for i, c in enumerate(range(0, x.shape[-1], chunk)):
        y, h = M.ops.ema_forward(x[..., c:c + chunk], p, q, gam, om, None, h, want_state=True)
        ys.append(y)
        assert rel_l2(h, g["states"][i] * beta) < 1e-5
    assert rel_l2(torch.cat(ys, -1), g["y"]) < 1e-5
    full = M.ops.ema_forward(x, p, q, gam, om)
    assert rel_l2(full, g["y"]) < 1e-5
    h, ys = None, []
    for t in range(x.shape[-1]):
        y, h = M.ops.ema_step(x[..., t:t + 1], p, q, gam, om, h)
        ys.append(y)
    assert rel_l2(torch.cat(ys, -1), g["y"]) < 1e-5
    assert rel_l2(h, g["states"][-1] * beta) < 1e-5
    # closed-form one_step of the reference (no residual): compare through a zero omega
    y1, h1 = M.ops.ema_step(x[..., :1], p, q, gam, torch.zeros_like(om), None)
    assert rel_l2(y1, g["step_y1"]) < 1e-5
    y2, h2 = M.ops.ema_step(x[..., 1:2], p, q, gam, torch.zeros_like(om), h1)
    assert rel_l2(y2, g["step_y2"]) < 1e-5 and rel_l2(h2, g["step_h2"] * beta) < 1e-5


def test_impulse_known_answer():
    """Impulse input: y[l] = sum_n p gamma_hat q^l + omega * delta(l)."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(9)
    prm = make_ema_params(gen, 4, 16)
    x = torch.zeros(1, 4, 40)
    x[:, :, 0] = 1.0
    p, q, gam = _coeffs(M, prm)
    y = M.ops.ema_forward(x.cuda(), p, q, gam, prm[4].cuda()).cpu()
    po, qo, go = O.ema_coeffs(*[t.double() for t in prm[:4]], dtype=torch.float64)
    k = O.ema_kernel(po, qo, go, 40)
    k[:, 0] += prm[4].double()
    assert rel_l2(y[0], k) < 1e-5


def test_config0_fp32():
    """BASELINE config 0: L=1024, B=8, D=512, ndim=16, fp32, 0-25% right padding, generated
    time-major and viewed as (B, D, L)."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(1234)
    length, bsz, dim = 1024, 8, 512
    x_tm = torch.randn(length, bsz, dim, generator=gen)
    prm = make_ema_params(gen, dim, 16)
    mask = right_pad_mask(gen, bsz, length, 0.25)
    x = x_tm.permute(1, 2, 0)
    ref = O.ema_forward_recurrence(x, *prm, mask)
    ref_fft = O.ema_forward_fft(x.contiguous(), *prm, mask)
    p, q, gam = _coeffs(M, prm)
    y = M.ops.ema_forward(x_tm.cuda().permute(1, 2, 0), p, q, gam, prm[4].cuda(), mask.cuda())
    assert rel_l2(y, ref) < 1e-5
    assert rel_l2(y, ref_fft) < 1e-5
    # run twice: bit-identical (no races)
    y2 = M.ops.ema_forward(x_tm.cuda().permute(1, 2, 0), p, q, gam, prm[4].cuda(), mask.cuda())
    assert torch.equal(y, y2)


def test_module_dropin():
    M, O = _mods()
    gen = torch.Generator().manual_seed(21)
    m = M.MultiHeadEMA(12, ndim=16).cuda().eval()
    prm = [m.alpha, m.delta, m.beta, m.gamma, m.omega]
    x = torch.randn(3, 12, 45, generator=gen).cuda()
    mask = right_pad_mask(gen, 3, 45, 0.3).cuda()
    with torch.no_grad():
        y = m(x, mask)
        ref = O.ema_forward_recurrence(x.cpu(), *[t.detach().cpu() for t in prm], mask.cpu())
        assert rel_l2(y, ref) < 1e-5
        # time-major adapter
        ytm = m.forward_time_major(x.permute(2, 0, 1).contiguous(), mask)
        assert rel_l2(ytm.permute(1, 2, 0), ref) < 1e-5
        # incremental through the module equals the full call
        st = {}
        outs = [m(x[..., i:i + 15], None, st) for i in range(0, 45, 15)]
        full = m(x)
        assert rel_l2(torch.cat(outs, -1), full) < 1e-5
        st2 = {}
        outs = [m(x[..., i:i + 1], None, st2) for i in range(45)]
        assert rel_l2(torch.cat(outs, -1), full) < 1e-5
        key = m._get_full_incremental_state_key("ema_state")
        assert st[key]["prev_state"].shape == (3, 12, 16)
        m.reorder_incremental_state(st, torch.tensor([2, 0, 1]).cuda())
        assert torch.equal(st[key]["prev_state"], st2[key]["prev_state"][[2, 0, 1]]) or \
            rel_l2(st[key]["prev_state"], st2[key]["prev_state"][[2, 0, 1]]) < 1e-5
        k, b = m.kernel(45, None)
        assert b is None and k.shape == (12, 45)
        out, h = m.step(x, 45)
        assert rel_l2(out + x * m.omega.view(-1, 1), full) < 1e-5


@pytest.mark.parametrize("bsz,dim,length", [(2, 5, 512), (3, 8, 1000), (1, 4, 16384), (2, 3, 4097)])
@pytest.mark.parametrize("bidir,shift", [(False, True), (True, True), (True, False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_resident_length_contiguous(bsz, dim, length, bidir, shift, dtype):
    """Length-contiguous (B, D, L) rows of >= 512 positions take the row-resident kernel (each row in
    shared memory, segment-parallel scan); check it against the oracle and against the generic
    kernels (a test switch disables the fast paths)."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(length + dim)
    prm = make_ema_params(gen, dim, 16, bidirectional=bidir)
    x = torch.randn(bsz, dim, length, generator=gen).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.4)
    mask[0, 7] = True
    ref = O.ema_forward_recurrence(x.float(), *prm, mask, bidirectional=bidir, shift=shift)
    p, q, gam = _coeffs(M, prm)
    y = M.ops.ema_forward(x.cuda(), p, q, gam, prm[4].cuda(), mask.cuda(), bidirectional=bidir, shift=shift)
    _lib.set_option(0, 1)
    try:
        y_gen = M.ops.ema_forward(x.cuda(), p, q, gam, prm[4].cuda(), mask.cuda(), bidirectional=bidir, shift=shift)
    finally:
        _lib.set_option(0, 0)
    assert rel_l2(y.float(), ref) < TOL[dtype]
    assert rel_l2(y.float(), y_gen.float()) < TOL[dtype]


@pytest.mark.parametrize("bidir", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_sequence_norm_ema(bidir, dtype):
    """SequenceNorm -> EMA in one kernel against the oracle and the two modules run in turn;
    short rows fall back to the two modules."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(31)
    bsz, dim = 3, 6
    for length in (2048, 100):
        norm = M.SequenceNorm(dim).cuda().eval()
        move = M.MultiHeadEMA(dim, ndim=16, bidirectional=bidir).cuda().eval()
        x = (torch.randn(bsz, dim, length, generator=gen) * 2 - 0.5).to(dtype)
        mask = right_pad_mask(gen, bsz, length, 0.5)
        mask[bsz - 1] = True
        with torch.no_grad():
            norm.weight.normal_(0, 0.1)
            norm.bias.normal_(0, 0.1)
            y = M.sequence_norm_ema(norm, move, x.cuda(), mask.cuda())
            y2 = move(norm(x.cuda(), mask.cuda()), mask.cuda())
        prm = [t.detach().cpu() for t in (move.alpha, move.delta, move.beta, move.gamma, move.omega)]
        xn = O.sequence_norm(x.float(), norm.weight.detach().cpu() + 1.0, norm.bias.detach().cpu(), mask)[0]
        ref = O.ema_forward_recurrence(xn, *prm, mask, bidirectional=bidir)
        assert rel_l2(y.float(), ref) < TOL[dtype]
        assert rel_l2(y.float(), y2.float()) < TOL[dtype] * 2
