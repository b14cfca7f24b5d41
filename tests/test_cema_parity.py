"""GPU parity of the complex EMA layer (through the C ABI) against the reference module's outputs
(golden fixtures) and the float64 oracle.  fp32 <= 1e-5 relative L2, bf16 <= 1e-2."""
import pytest
import torch

from _util import golden, opt_mask, rel_l2, right_pad_mask

pytestmark = pytest.mark.gpu
NAMES = ["cema_uni_n16", "cema_uni_n3", "cema_bidir_shift", "cema_bidir_noshift", "cema_bidir_trunc"]
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2}


def _mods():
    import fairseq_apollo_b200 as M
    from oracle import mega_oracle as O
    return M, O


def _module(M, g, dim, ndim, **kw):
    m = M.MultiHeadComplexEMA(dim, ndim=ndim, **kw).cuda().eval()
    with torch.no_grad():
        for k in ("alpha", "delta", "theta", "gamma", "omega"):
            getattr(m, k).copy_(g[k])
    return m


@pytest.mark.parametrize("name", NAMES)
def test_golden(name):
    M, _ = _mods()
    g = golden(name)
    trunc = None if g["truncation"] < 0 else g["truncation"]
    m = _module(M, g, g["x"].shape[1], g["alpha"].shape[1], bidirectional=bool(g["bidirectional"]),
                shift=bool(g["shift"]), truncation=trunc)
    mask = opt_mask(g["mask"])
    with torch.no_grad():
        y = m(g["x"].cuda(), None if mask is None else mask.cuda())
        k, _ = m.kernel(g["x"].shape[-1])
    assert rel_l2(y, g["y"]) < 1e-5
    assert rel_l2(k, g["kernel"]) < 1e-5
    sd = m.state_dict()
    assert {n: tuple(v.shape) for n, v in sd.items()} == {n: tuple(g[n].shape) for n in
                                                          ("alpha", "delta", "theta", "gamma", "omega")}
    assert [n for n, _ in m.parameters_no_weight_decay()] == ["alpha", "delta", "theta"]


def test_incremental_golden():
    M, _ = _mods()
    g = golden("cema_incremental")
    m = _module(M, g, g["x"].shape[1], g["alpha"].shape[1])
    x = g["x"].cuda()
    chunk = g["chunk"]
    st, ys = {}, []
    with torch.no_grad():
        for i in range(0, x.shape[-1], chunk):
            ys.append(m(x[..., i:i + chunk], None, st))
            h = m._get_input_buffer(st)["prev_state"]
            assert h.dtype == torch.complex64
            assert rel_l2(torch.view_as_real(h), g["states"][i // chunk]) < 1e-5
        assert rel_l2(torch.cat(ys, -1), g["y"]) < 1e-5
        y1, h1 = m.one_step(x[..., :1])
        y2, h2 = m.one_step(x[..., 1:2], h1)
        assert rel_l2(y1, g["step_y1"]) < 1e-5 and rel_l2(y2, g["step_y2"]) < 1e-5
        assert rel_l2(torch.view_as_real(h2), g["step_h2"]) < 1e-5
        # token-by-token decoding equals the full pass; a reorder permutes the batch rows
        st2, outs = {}, []
        for t in range(8):
            outs.append(m(x[..., t:t + 1], None, st2))
        assert rel_l2(torch.cat(outs, -1), g["y_full"][..., :8]) < 1e-5
        order = torch.tensor([2, 0, 1], device="cuda")
        before = m._get_input_buffer(st2)["prev_state"].clone()
        m.reorder_incremental_state(st2, order)
        assert torch.equal(m._get_input_buffer(st2)["prev_state"], before[order])


@pytest.mark.parametrize("bsz,dim,length,ndim,bidir,shift,trunc", [
    (1, 1, 1, 16, False, True, None), (2, 7, 33, 16, False, True, None), (3, 5, 257, 2, False, True, None),
    (2, 9, 65, 32, False, True, None), (2, 6, 40, 16, True, True, None), (2, 3, 31, 5, True, False, None),
    (2, 4, 50, 16, True, True, 9), (9, 33, 17, 1, True, False, 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_grid(bsz, dim, length, ndim, bidir, shift, trunc, dtype):
    """Odd shapes, interior pads, SiLU, and x given as the (B, D, L) view of (B, L, D) memory."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(dim * 100 + length)
    torch.manual_seed(dim * 100 + length)
    m = M.MultiHeadComplexEMA(dim, ndim=ndim, bidirectional=bidir, shift=shift, truncation=trunc).cuda().eval()
    with torch.no_grad():
        m.gamma[:, :, 1].normal_(0, 1)
    x = torch.randn(bsz, length, dim, generator=gen).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.4)
    if length > 4:
        mask[0, 2] = True
    prm = [getattr(m, k).detach().cpu() for k in ("alpha", "delta", "theta", "gamma", "omega")]
    ref = O.cema_forward_recurrence(x.float().transpose(1, 2), *prm, mask, bidir, shift, trunc, silu=True)
    with torch.no_grad():
        y = m(x.cuda().transpose(1, 2), mask.cuda(), None, 'silu')
    assert y.shape == (bsz, dim, length)
    assert rel_l2(y.float(), ref) < TOL[dtype]


def test_chunked_equals_full_with_masks():
    M, O = _mods()
    gen = torch.Generator().manual_seed(3)
    torch.manual_seed(3)
    m = M.MultiHeadComplexEMA(12, ndim=16).cuda().eval()
    x = torch.randn(2, 12, 96, generator=gen).cuda()
    mask = right_pad_mask(gen, 2, 96, 0.3).cuda()
    with torch.no_grad():
        full = m(x, mask)
        st, parts = {}, []
        for i in range(0, 96, 32):
            parts.append(m(x[..., i:i + 32], mask[:, i:i + 32], st))
    assert rel_l2(torch.cat(parts, -1), full) < 1e-5


@pytest.mark.parametrize("bsz,length,dim,ndim", [(2, 70, 24, 16), (3, 257, 72, 3), (2, 64, 8, 16), (2, 40, 20, 32),
                                                 (50, 40, 1024, 16)])   # the last: one thread per channel
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_timestep_norm_complex_ema(bsz, length, dim, ndim, dtype):
    """TimestepNorm -> complex EMA (+ SiLU) through the fused helper: one streamed kernel when
    ndim <= 16, the two operators in turn otherwise; full pass and chunked with both states."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(length + dim)
    torch.manual_seed(length + dim)
    move = M.MultiHeadComplexEMA(dim, ndim=ndim).cuda().eval()
    norm = M.TimestepNorm(dim, prior_count=2).cuda().eval()
    with torch.no_grad():
        move.gamma[:, :, 1].normal_(0, 1)
        norm.weight.normal_(0, 0.1)
        norm.bias.normal_(0, 0.1)
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.3 + 0.2).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.3)
    prm = [getattr(move, k).detach().cpu() for k in ("alpha", "delta", "theta", "gamma", "omega")]
    xn_ref = O.timestep_norm(x.float(), torch.full((bsz,), 2, dtype=torch.int64), torch.zeros(bsz, dim),
                             torch.ones(bsz, dim), norm.weight.detach().cpu() + 1.0, norm.bias.detach().cpu(), mask)[0]
    y_ref = O.cema_forward_recurrence(xn_ref.transpose(1, 2), *prm, mask, silu=True).transpose(1, 2)
    with torch.no_grad():
        y, xn = M.timestep_norm_ema(norm, move, x.cuda(), mask.cuda(), None, 'silu', return_normed=True)
        assert rel_l2(y.float(), y_ref) < TOL[dtype]
        assert rel_l2(xn.float(), xn_ref) < TOL[dtype]
        assert (xn.cpu()[mask] == 0).all()
        st, parts = {}, []
        step = 32
        for i in range(0, length, step):
            parts.append(M.timestep_norm_ema(norm, move, x[:, i:i + step].cuda(), mask[:, i:i + step].cuda(), st, 'silu'))
        assert rel_l2(torch.cat(parts, 1).float(), y_ref) < TOL[dtype]
        assert move._get_input_buffer(st)["prev_state"].dtype == torch.complex64


@pytest.mark.parametrize("bsz,length,dim,ndim", [(4, 32, 64, 16), (8, 96, 64, 16), (9, 100, 72, 16), (16, 257, 200, 5),
                                                 (8, 1024, 136, 16)])
@pytest.mark.parametrize("normed", [False, True])
@pytest.mark.parametrize("silu", [False, True])
def test_complex_tensor_core_path(bsz, length, dim, ndim, normed, silu):
    """bf16, no padding: fused TimestepNorm -> complex EMA on the tensor-core kernel (complex P, G
    and q^16 fragments) against the oracle and against the streamed kernel (a test switch disables
    the tensor-core path); full pass, then 32-step chunks with the carried complex state."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(bsz * 131 + length + dim)
    torch.manual_seed(bsz * 131 + length + dim)
    move = M.MultiHeadComplexEMA(dim, ndim=ndim).cuda().eval()
    norm = M.TimestepNorm(dim, prior_count=2).cuda().eval()
    with torch.no_grad():
        move.gamma[:, :, 1].normal_(0, 1)
        norm.weight.normal_(0, 0.1)
        norm.bias.normal_(0, 0.1)
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.3 + 0.2).to(torch.bfloat16)
    prm = [getattr(move, k).detach().cpu() for k in ("alpha", "delta", "theta", "gamma", "omega")]
    xn_ref = O.timestep_norm(x.float(), torch.full((bsz,), 2, dtype=torch.int64), torch.zeros(bsz, dim),
                             torch.ones(bsz, dim), norm.weight.detach().cpu() + 1.0, norm.bias.detach().cpu(), None)[0]
    y_ref = O.cema_forward_recurrence(xn_ref.transpose(1, 2), *prm, None, silu=silu).transpose(1, 2)
    act = 'silu' if silu else None
    outs = []
    before = M.launch_count()
    with torch.no_grad():
        for disable in (0, 1):
            _lib.set_option(1, disable)
            try:
                res = M.timestep_norm_ema(norm, move, x.cuda(), None, None, act, return_normed=normed)
                st, parts = {}, []
                for i in range(0, length, 32):
                    parts.append(M.timestep_norm_ema(norm, move, x[:, i:i + 32].cuda(), None, st, act))
            finally:
                _lib.set_option(1, 0)
            y = res[0] if normed else res
            assert rel_l2(y.float(), y_ref) < 1e-2, disable
            if normed:
                assert rel_l2(res[1].float(), xn_ref) < 1e-2, disable
            assert rel_l2(torch.cat(parts, 1).float(), y_ref) < 1e-2, disable
            outs.append((y, move._get_input_buffer(st)["prev_state"]))
    assert rel_l2(outs[0][0].float(), outs[1][0].float()) < 1e-2
    assert outs[0][1].dtype == torch.complex64
    if not normed:   # the complex layer alone (no normalisation) on the same kernel
        e_ref = O.cema_forward_recurrence(x.float().transpose(1, 2), *prm, None, silu=silu)
        with torch.no_grad():
            e = move(x.cuda().transpose(1, 2), None, None, act)
            st2, parts2 = {}, []
            for i in range(0, length, 32):
                parts2.append(move(x[:, i:i + 32].cuda().transpose(1, 2), None, st2, act))
        assert rel_l2(e.float(), e_ref) < 1e-2
        assert rel_l2(torch.cat(parts2, -1).float(), e_ref) < 1e-2
    if length % 32 == 0:   # the final carried states of the two implementations
        assert rel_l2(torch.view_as_real(outs[0][1]), torch.view_as_real(outs[1][1])) < 1e-2
    assert _lib.device_error() == 0


@pytest.mark.parametrize("ndim", [16, 3])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_complex_single_token_decode(ndim, dtype):
    """TimestepNorm -> complex EMA token by token with the incremental state (the fused decode
    step for ndim 16, the two operators in turn for ndim 3) equals the full-length call."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(ndim)
    torch.manual_seed(ndim)
    bsz, length, dim = 5, 37, 72
    move = M.MultiHeadComplexEMA(dim, ndim=ndim).cuda().eval()
    norm = M.TimestepNorm(dim, prior_count=2).cuda().eval()
    with torch.no_grad():
        move.gamma[:, :, 1].normal_(0, 1)
        norm.weight.normal_(0, 0.1)
        norm.bias.normal_(0, 0.1)
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.3 + 0.2).to(dtype).cuda()
    with torch.no_grad():
        full, xn_full = M.timestep_norm_ema(norm, move, x, None, None, 'silu', return_normed=True)
        st, ys, xns = {}, [], []
        for t in range(length):
            y, xn = M.timestep_norm_ema(norm, move, x[:, t:t + 1].contiguous(), None, st, 'silu', return_normed=True)
            ys.append(y)
            xns.append(xn)
    assert rel_l2(torch.cat(ys, 1).float(), full.float()) < TOL[dtype]
    assert rel_l2(torch.cat(xns, 1).float(), xn_full.float()) < TOL[dtype]
    assert move._get_input_buffer(st)["prev_state"].dtype == torch.complex64
    assert int(norm._get_input_buffer(st)["prev_count"][0]) == 2 + length
