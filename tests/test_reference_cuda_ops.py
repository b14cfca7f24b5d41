"""GPU: this build's kernels against the REFERENCE'S OWN CUDA operators, compiled unmodified from the
reference checkout by ``oracle/build_ref.py --cuda`` (the reference's GPU path: TimestepNorm /
SequenceNorm kernels, ema_parameters + the shared-memory FFT convolution + ema_hidden).  Skipped
when that build is absent.  The Python glue of the reference does not travel with the compiled
operators, so the few lines that call them restate fairseq/modules/fused_ops/fftconv.py:13-27 and
fairseq/modules/base_moving_average.py:137-172."""
import math

import pytest
import torch

from _util import make_ema_params, rel_l2, right_pad_mask

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2}


def _ref():
    from oracle.build_ref import load_ref_cuda
    mod = load_ref_cuda()
    if mod is None:
        pytest.skip("oracle/_ref/mega_ref_cuda.so not built (python oracle/build_ref.py --cuda)")
    return mod.ops


def _ours():
    import fairseq_apollo_b200 as M
    return M


@pytest.mark.parametrize("bsz,length,feat,groups", [(2, 100, 64, None), (3, 255, 96, None), (2, 200, 64, 4),
                                                     (2, 31, 130, None)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_timestep_norm_forward_and_backward(bsz, length, feat, groups, dtype):
    """The reference's column-wise kernels (L < 256), plain and grouped.  Its chunked kernel for
    longer sequences asks for 32 x 32 threads at a register count that sm_100 refuses
    ("too many resources requested for launch"), so longer cases cannot be compared here."""
    R, M = _ref(), _ours()
    gen = torch.Generator().manual_seed(length + feat)
    x = (torch.randn(bsz, length, feat, generator=gen) * 1.5 + 0.2).to(dtype).cuda()
    dy = torch.randn(bsz, length, feat, generator=gen).to(dtype).cuda()
    mask = right_pad_mask(gen, bsz, length, 0.4).cuda()
    ng = feat if groups is None else groups
    pc = torch.full((bsz,), 2, dtype=torch.int64).cuda()
    pm = (torch.randn(bsz, ng, generator=gen) * 0.1).to(dtype).cuda()
    pv = (torch.rand(bsz, ng, generator=gen) + 0.5).to(dtype).cuda()
    gamma = (torch.randn(feat, generator=gen) * 0.1 + 1).to(dtype).cuda()
    beta = (torch.randn(feat, generator=gen) * 0.1).to(dtype).cuda()
    dmean = torch.randn(bsz, ng, generator=gen).to(dtype).cuda()
    dvar = torch.randn(bsz, ng, generator=gen).to(dtype).cuda()
    if groups is None:
        ry, rc, rm, rv, cm, cr = R.timestep_norm_fwd(x, pc, pm, pv, gamma, beta, mask, 1e-5)
        rdx, rdm, rdv, rdg, rdb = R.timestep_norm_bwd(dy, dmean, dvar, x, pm, rc, cm, cr, gamma, mask)
    else:
        ry, rc, rm, rv, gm, cm, cr = R.group_timestep_norm_fwd(x, pc, pm, pv, gamma, beta, mask, groups, 1e-5)
        rdx, rdm, rdv, rdg, rdb = R.group_timestep_norm_bwd(dy, dmean, dvar, x, pm, rc, gm, cm, cr, gamma, mask, groups)
    y, c, m, v, ocm, ocr, ogm = M.ops.timestep_norm_fwd_train(x, pc, pm, pv, gamma, beta, mask, 1e-5, groups)
    dx, dpm, dpv, dg, db = M.ops.timestep_norm_bwd(dy, dmean, dvar, x, pm, c, ocm, ocr, ogm, gamma, mask, groups)
    assert torch.equal(c, rc)
    assert rel_l2(y.float(), ry.float()) < TOL[dtype]
    assert rel_l2(m, rm.float()) < TOL[dtype] and rel_l2(v, rv.float()) < TOL[dtype]
    if dtype == torch.float32:   # the reference keeps its saved statistics in bf16 otherwise
        assert rel_l2(dx, rdx) < 5e-5
        assert rel_l2(dpm, rdm) < 5e-5 and rel_l2(dpv, rdv) < 5e-5
        assert rel_l2(dg, rdg) < 2e-4 and rel_l2(db, rdb) < 2e-4


@pytest.mark.parametrize("length_last", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sequence_norm_forward_and_backward(length_last, dtype):
    R, M = _ref(), _ours()
    gen = torch.Generator().manual_seed(5)
    bsz, feat, length = 3, 48, 1500
    shape = (bsz, feat, length) if length_last else (bsz, length, feat)
    x = (torch.randn(*shape, generator=gen) * 2 - 0.5).to(dtype).cuda()
    dy = torch.randn(*shape, generator=gen).to(dtype).cuda()
    mask = right_pad_mask(gen, bsz, length, 0.5).cuda()
    gamma = (torch.randn(feat, generator=gen) * 0.1 + 1).to(dtype).cuda()
    beta = (torch.randn(feat, generator=gen) * 0.1).to(dtype).cuda()
    ry, rc, rm, rr = R.sequence_norm_fwd(x, gamma, beta, mask, 1e-5, length_last)
    rdx, rdg, rdb = R.sequence_norm_bwd(dy, x, rc, rm, rr, gamma, mask, length_last)
    y, c, m, r = M.ops.sequence_norm_fwd(x, gamma, beta, mask, 1e-5, length_last)
    dx, dg, db = M.ops.sequence_norm_bwd(dy, x, c, m, r, gamma, mask, length_last)
    assert torch.equal(c, rc)
    assert rel_l2(y.float(), ry.float()) < TOL[dtype]
    assert rel_l2(m, rm.float()) < 1e-5 and rel_l2(r, rr.float()) < 1e-5
    assert rel_l2(dx.float(), rdx.float()) < (5e-5 if dtype == torch.float32 else 2e-2)
    assert rel_l2(dg, rdg.float()) < (2e-4 if dtype == torch.float32 else 2e-2)
    assert rel_l2(db, rdb.float()) < (2e-4 if dtype == torch.float32 else 2e-2)


def _reference_ema_gpu(R, x, params, mask, h):
    """The reference's GPU forward of the real EMA (complex layer with the rotation off):
    kernel and bias from ema_parameters_fwd, convolution through its shared-memory FFT kernel
    (32 <= L <= 8192, fused_ops/fftconv.py:17-25), new state from ema_hidden_fwd."""
    alpha, delta, beta, gamma, omega = [t.cuda() for t in params]
    bsz, dim, length = x.shape
    ndim = alpha.shape[1]
    p = torch.sigmoid(alpha.float())                                   # (D, N, 1): cema keeps beta in gamma
    q = torch.polar(1.0 - p * torch.sigmoid(delta.float()), torch.zeros_like(p))
    g = torch.complex(gamma * beta.squeeze(-1), torch.zeros_like(gamma)) * math.sqrt(1.0 / ndim)
    residual = x * omega.view(dim, 1).to(x.dtype)
    xm = x if mask is None else x * (1.0 - mask.unsqueeze(1).to(x))
    w, b, _ = R.ema_parameters_fwd(p, q.log(), g, h, length)
    n = length if (length & (length - 1)) == 0 else (1 << length.bit_length())
    k_f = torch.fft.rfft(w.float(), 2 * n)
    y, _ = R.fftconv_fwd(xm.contiguous(), k_f)
    if b is not None:
        y = y + b
    hn, _ = R.ema_hidden_fwd(xm.contiguous(), p, q.log(), h)
    return y + residual, hn


@pytest.mark.parametrize("bsz,dim,length", [(2, 16, 64), (3, 40, 1000), (2, 24, 4096)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ema_forward_against_reference_fft_kernel(bsz, dim, length, dtype):
    R, M = _ref(), _ours()
    gen = torch.Generator().manual_seed(dim + length)
    ndim = 16
    params = make_ema_params(gen, dim, ndim)
    x = torch.randn(bsz, dim, length, generator=gen).to(dtype).cuda()
    mask = right_pad_mask(gen, bsz, length, 0.25).cuda()
    ref, _ = _reference_ema_gpu(R, x, params, mask, None)
    m = M.MultiHeadEMA(dim, ndim=ndim).cuda().eval()
    with torch.no_grad():
        for dst, src in zip((m.alpha, m.delta, m.beta, m.gamma, m.omega), params):
            dst.copy_(src)
        y = m(x, mask)
    assert rel_l2(y.float(), ref.float()) < TOL[dtype]


def test_ema_incremental_against_reference_ops():
    """Chunked forward with a carried state: outputs and states against the reference's
    ema_parameters (bias) / ema_hidden CUDA kernels.  The reference state is h / beta-free
    (p = sigmoid(alpha)); with the rotation off its real part times beta is this build's state."""
    R, M = _ref(), _ours()
    gen = torch.Generator().manual_seed(9)
    bsz, dim, length, chunk, ndim = 3, 24, 192, 64, 16
    params = make_ema_params(gen, dim, ndim)
    x = torch.randn(bsz, dim, length, generator=gen).cuda()
    m = M.MultiHeadEMA(dim, ndim=ndim).cuda().eval()
    with torch.no_grad():
        for dst, src in zip((m.alpha, m.delta, m.beta, m.gamma, m.omega), params):
            dst.copy_(src)
        st, h = {}, None
        for i in range(0, length, chunk):
            xc = x[..., i:i + chunk].contiguous()
            ref, h = _reference_ema_gpu(R, xc, params, None, h)
            y = m(xc, None, st)
            assert rel_l2(y, ref) < 1e-5
            ours = m._get_input_buffer(st)["prev_state"]
            assert rel_l2(ours, h.real * params[2].squeeze(-1).cuda()) < 1e-5
