"""GPU parity of the fused TimestepNorm -> EMA entry point against the oracle (TimestepNorm
restated from the reference CPU op, then the fp64 recurrence)."""
import pytest
import torch

from _util import make_ema_params, rel_l2, right_pad_mask

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2}


def _mods():
    import fairseq_apollo_b200 as M
    from oracle import mega_oracle as O
    return M, O


def _reference(O, x, pc, pm, pv, gamma, beta, prm, mask, silu=False):
    xn, cnt, mean, var = O.timestep_norm(x.float(), pc, pm, pv, gamma, beta, mask, acc_dtype=torch.float64)
    y = O.ema_forward_recurrence(xn.transpose(1, 2), *prm, mask, silu=silu).transpose(1, 2)
    return xn, y, cnt, mean, var


@pytest.mark.parametrize("bsz,length,dim", [(1, 1, 1), (2, 77, 33), (3, 300, 128), (2, 1024, 72), (9, 40, 256)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("masked", [False, True])
def test_fused_grid(bsz, length, dim, dtype, masked):
    M, O = _mods()
    gen = torch.Generator().manual_seed(length + dim)
    prm = make_ema_params(gen, dim, 16)
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.3 + 0.1).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.3) if masked else None
    pc = torch.full((bsz,), 2, dtype=torch.int64)
    pm = torch.randn(bsz, dim, generator=gen) * 0.1
    pv = torch.rand(bsz, dim, generator=gen) + 0.5
    gamma = torch.randn(dim, generator=gen) * 0.1 + 1
    beta = torch.randn(dim, generator=gen) * 0.1
    xn, y, cnt, mean, var = _reference(O, x, pc, pm, pv, gamma, beta, prm, mask)
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    res = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                p, q, g, prm[4].cuda(), None if mask is None else mask.cuda(), want_normed=True)
    assert torch.equal(res["count"].cpu(), cnt)
    assert rel_l2(res["y"].float(), y) < TOL[dtype]
    assert rel_l2(res["xn"].float(), xn) < TOL[dtype]
    # bf16 without a mask runs on the tensor-core kernel, whose second moment goes through tf32 products
    assert rel_l2(res["mean"], mean) < 1e-5 and rel_l2(res["var"], var) < (1e-5 if dtype == torch.float32 else 1e-3)
    if mask is not None:
        assert (res["xn"].cpu()[mask] == 0).all()


def test_fused_equals_unfused_modules_and_incremental():
    M, O = _mods()
    gen = torch.Generator().manual_seed(4)
    dim, bsz, length = 48, 3, 96
    norm = M.TimestepNorm(dim, prior_count=2).cuda().eval()
    move = M.MultiHeadEMA(dim, ndim=16).cuda().eval()
    x = torch.randn(bsz, length, dim, generator=gen).cuda()
    mask = right_pad_mask(gen, bsz, length, 0.25).cuda()
    with torch.no_grad():
        norm.weight.normal_(0, 0.1)
        norm.bias.normal_(0, 0.1)
        xn = norm(x, mask)
        ref = torch.nn.functional.silu(move(xn.transpose(1, 2), mask).transpose(1, 2))
        mx, xn2 = M.timestep_norm_ema(norm, move, x, mask, None, activation='silu', return_normed=True)
        assert rel_l2(mx, ref) < 1e-5 and rel_l2(xn2, xn) < 1e-6
        # chunked with both modules' incremental buffers
        st = {}
        outs = [M.timestep_norm_ema(norm, move, x[:, i:i + 32], None, st) for i in range(0, length, 32)]
        full = M.timestep_norm_ema(norm, move, x)
        assert rel_l2(torch.cat(outs, 1), full) < 1e-5
        st1 = {}
        outs = [M.timestep_norm_ema(norm, move, x[:, i:i + 1], None, st1) for i in range(length)]
        assert rel_l2(torch.cat(outs, 1), full) < 1e-5


def test_config1_reduced_bf16():
    """BASELINE config 1 at reduced batch (B=2 of 16): L=4096, D=1024, bf16 activations, fp32
    parameters, TimestepNorm weight=1 bias=0 eps=1e-5, no padding."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(1235)
    bsz, length, dim = 2, 4096, 1024
    prm = make_ema_params(gen, dim, 16)
    x = torch.randn(bsz, length, dim, generator=gen).to(torch.bfloat16)
    pc = torch.zeros(bsz, dtype=torch.int64)
    pm = torch.zeros(bsz, dim)
    pv = torch.ones(bsz, dim)
    xn, y, cnt, mean, var = _reference(O, x, pc, pm, pv, torch.ones(dim), torch.zeros(dim), prm, None)
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    res = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), torch.ones(dim).cuda(),
                                torch.zeros(dim).cuda(), 1e-5, p, q, g, prm[4].cuda())
    assert rel_l2(res["y"].float(), y) < 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("bsz,length,dim", [(2, 1, 8), (3, 31, 72), (2, 32, 64), (2, 33, 136), (1, 1000, 200), (5, 257, 8),
                                            (50, 40, 1024)])   # the last: enough rows for one thread per channel
def test_streamed_path_matches_generic(dtype, bsz, length, dim):
    """The TMA-streamed kernels and the generic kernels are two implementations of the same
    entry points: run both (a test switch disables the streamed one) on shapes inside the
    streamed envelope and compare them with each other and with the oracle."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(bsz * 31 + length + dim)
    prm = make_ema_params(gen, dim, 16)
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.3 + 0.1).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.4)
    if length > 3:
        mask[0, 1] = True
    pc = torch.full((bsz,), 3, dtype=torch.int64)
    pm = torch.randn(bsz, dim, generator=gen) * 0.1
    pv = torch.rand(bsz, dim, generator=gen) + 0.5
    gamma = torch.randn(dim, generator=gen) * 0.1 + 1
    beta = torch.randn(dim, generator=gen) * 0.1
    h0 = torch.randn(bsz, dim, 16, generator=gen) * 0.3
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    tol = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 2e-3}[dtype]
    outs = []
    for disable in (0, 1):
        _lib.set_option(0, disable)
        try:
            fused = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                          p, q, g, prm[4].cuda(), mask.cuda(), h_in=h0.cuda(), want_state=True,
                                          want_normed=True, silu=True)
            plain = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                          p, q, g, prm[4].cuda(), None)
            tsn = M.ops.timestep_norm_fwd(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), mask.cuda())
            ema, hs = M.ops.ema_forward(x.cuda().transpose(1, 2), p, q, g, prm[4].cuda(), mask.cuda(), h0.cuda(),
                                        want_state=True)
            ema2 = M.ops.ema_forward(x.cuda().transpose(1, 2), p, q, g, prm[4].cuda())
        finally:
            _lib.set_option(0, 0)
        outs.append((fused, plain, tsn, ema, hs, ema2))
    (f0, p0, t0, e0, h0s, e20), (f1, p1, t1, e1, h1s, e21) = outs
    assert rel_l2(f0["y"].float(), f1["y"].float()) < tol and rel_l2(f0["xn"].float(), f1["xn"].float()) < tol
    assert rel_l2(f0["h"], f1["h"]) < 1e-5 and rel_l2(f0["mean"], f1["mean"]) < 1e-5 and rel_l2(f0["var"], f1["var"]) < 1e-5
    assert torch.equal(f0["count"], f1["count"])
    assert rel_l2(p0["y"].float(), p1["y"].float()) < tol
    assert rel_l2(t0[0].float(), t1[0].float()) < tol and torch.equal(t0[1], t1[1])
    assert rel_l2(e0.float(), e1.float()) < tol and rel_l2(h0s, h1s) < 1e-5 and rel_l2(e20.float(), e21.float()) < tol
    # against the oracle
    xn, cnt, mean, var = O.timestep_norm(x.float(), pc, pm, pv, gamma, beta, mask, acc_dtype=torch.float64)[:4]
    yref, href = O.ema_forward_recurrence(xn.transpose(1, 2), *prm, mask, h=h0, return_state=True, silu=True)
    assert rel_l2(f0["y"].float(), yref.transpose(1, 2)) < tol
    assert rel_l2(f0["h"], href) < max(tol, 1e-5) * (1 if dtype == torch.float32 else 3)
    assert torch.equal(f0["count"].cpu(), cnt)
    assert (f0["xn"].cpu()[mask] == 0).all()
    eref = O.ema_forward_recurrence(x.float().transpose(1, 2), *prm, mask, h=h0)
    assert rel_l2(e0.float(), eref) < tol
    assert _lib.device_error() == 0


@pytest.mark.parametrize("bsz,length,dim,ndim", [(4, 32, 64, 16), (9, 100, 72, 16), (8, 1024, 128, 16),
                                                  (16, 257, 200, 16), (5, 64, 8, 2), (8, 96, 136, 5)])
@pytest.mark.parametrize("with_state", [False, True])
@pytest.mark.parametrize("tile", [8, 7, 4, 2, 22, 222, 224, 422, 124])
def test_tensor_core_path(bsz, length, dim, ndim, with_state, tile):
    """bf16, no padding: the tensor-core kernels (fused TimestepNorm -> EMA and EMA alone) against
    the oracle, and against the streamed SIMT kernels (a test switch disables the MMA path)."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(bsz * 131 + length + dim)
    prm = make_ema_params(gen, dim, ndim)
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.3 + 0.2).to(torch.bfloat16)
    pc = torch.full((bsz,), 2, dtype=torch.int64)
    pc[0] = 5
    pm = torch.randn(bsz, dim, generator=gen) * 0.1
    pv = torch.rand(bsz, dim, generator=gen) + 0.5
    gamma = torch.randn(dim, generator=gen) * 0.1 + 1
    beta = torch.randn(dim, generator=gen) * 0.1
    h0 = torch.randn(bsz, dim, ndim, generator=gen) * 0.3 if with_state else None
    want_state = with_state and length % 32 == 0
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    outs = []
    before = M.launch_count()
    xn_ref = O.timestep_norm(x.float(), pc, pm, pv, gamma, beta, None, acc_dtype=torch.float64)[0]
    ysilu_ref = O.ema_forward_recurrence(xn_ref.transpose(1, 2), *prm, None, h=h0, silu=True).transpose(1, 2)
    for disable in (0, 1):
        _lib.set_option(1, disable)
        # 64-, 56-, 32- or 16-channel tiles; 22: 16 channels with two warps per 16-byte column;
        # 222, 224, 422, 124: the forms pipelined along the sequence (tile, warps per column, depth)
        _lib.set_option(2, tile)
        try:
            fused = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                          p, q, g, prm[4].cuda(), None, h_in=None if h0 is None else h0.cuda(),
                                          want_state=want_state)
            ema = M.ops.ema_forward(x.cuda().transpose(1, 2), p, q, g, prm[4].cuda(), None,
                                    None if h0 is None else h0.cuda(), want_state=want_state, silu=True)
            # the same call with the normalised activations as a second output (the form the Mega
            # block uses: the tensor-core kernel writes both tiles)
            both = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                         p, q, g, prm[4].cuda(), None, h_in=None if h0 is None else h0.cuda(),
                                         want_state=want_state, want_normed=True, silu=True)
            # TimestepNorm alone (the same kernel without the pole matrices)
            tsn_only = M.ops.timestep_norm_fwd(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda())
        finally:
            _lib.set_option(1, 0)
            _lib.set_option(2, 0)
        outs.append((fused, ema))
        assert rel_l2(tsn_only[0].float(), xn_ref) < 1e-2, disable
        assert torch.equal(tsn_only[1].cpu(), fused["count"].cpu())
        assert rel_l2(tsn_only[2], fused["mean"]) < 1e-5 and rel_l2(tsn_only[3], fused["var"]) < 1e-3
        assert rel_l2(both["xn"].float(), xn_ref) < 1e-2, disable
        assert rel_l2(both["y"].float(), ysilu_ref) < 1e-2, disable
        assert torch.equal(both["count"].cpu(), fused["count"].cpu())
        # (the pipelined forms have no second output: `both` then runs the un-pipelined kernel, whose
        # sums of squares are centred differently)
        same_kernel = tile < 100 or disable == 1
        assert rel_l2(both["mean"], fused["mean"]) < 1e-6 and rel_l2(both["var"], fused["var"]) < (1e-6 if same_kernel else 1e-4)
        if want_state:
            assert rel_l2(both["h"], fused["h"]) < (1e-6 if same_kernel else 1e-2)
    xn, cnt, mean, var = O.timestep_norm(x.float(), pc, pm, pv, gamma, beta, None, acc_dtype=torch.float64)[:4]
    yref, href = O.ema_forward_recurrence(xn.transpose(1, 2), *prm, None, h=h0, return_state=True)
    eref, ehref = O.ema_forward_recurrence(x.float().transpose(1, 2), *prm, None, h=h0, return_state=True, silu=True)
    for k, (fused, ema) in enumerate(outs):
        assert rel_l2(fused["y"].float(), yref.transpose(1, 2)) < 1e-2, k
        assert torch.equal(fused["count"].cpu(), cnt)
        assert rel_l2(fused["mean"], mean) < 1e-4 and rel_l2(fused["var"], var) < 1e-3, k
        e = ema[0] if want_state else ema
        assert rel_l2(e.float(), eref) < 1e-2, k
        if want_state:
            assert rel_l2(fused["h"], href) < 1e-2 and rel_l2(ema[1], ehref) < 1e-2, k
    # the two implementations agree with each other well inside the bf16 tolerance
    assert rel_l2(outs[0][0]["y"].float(), outs[1][0]["y"].float()) < 1e-2
    assert _lib.device_error() == 0


@pytest.mark.parametrize("offset,scale", [(5.0, 0.3), (-20.0, 2.0), (0.0, 30.0)])
def test_tensor_core_path_offset_data(offset, scale):
    """Channels whose mean is large against their spread: the tensor-core TimestepNorm keeps its
    sums centred on the running mean, so the normalised output and the statistics stay accurate."""
    M, O = _mods()
    gen = torch.Generator().manual_seed(77)
    bsz, length, dim = 8, 512, 64
    prm = make_ema_params(gen, dim, 16)
    x = (torch.randn(bsz, length, dim, generator=gen) * scale + offset).to(torch.bfloat16)
    pc = torch.full((bsz,), 2, dtype=torch.int64)
    pm = torch.full((bsz, dim), offset)
    pv = torch.full((bsz, dim), scale * scale)
    gamma, beta = torch.ones(dim), torch.zeros(dim)
    xn, cnt, mean, var = O.timestep_norm(x.float(), pc, pm, pv, gamma, beta, None, acc_dtype=torch.float64)[:4]
    yref = O.ema_forward_recurrence(xn.transpose(1, 2), *prm).transpose(1, 2)
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    before = M.launch_count()
    res = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                p, q, g, prm[4].cuda())
    assert rel_l2(res["y"].float(), yref) < 1e-2
    assert rel_l2(res["mean"], mean) < 1e-4 and rel_l2(res["var"], var) < 2e-3


def test_config4_full_size_properties():
    """The bench workload at full size (B=64, L=32768, D=2048, bf16; 8 GiB in, 8 GiB out), checked
    through properties that do not need an oracle pass over 4e9 elements:
    (1) half of the batch run alone (same tile shape) gives bit for bit the rows of the full-batch call;
    (2) two half-length calls with the carried statistics and EMA state give the full call
        within the bf16 tolerance;
    (3) 3 sequences x 8 channels over the whole length against the float64 oracle."""
    M, O = _mods()
    free, _ = torch.cuda.mem_get_info()
    if free < 40 * 2 ** 30:
        pytest.skip("needs ~26 GiB of device memory")
    bsz, length, dim, ndim = 64, 32768, 2048, 16
    gen = torch.Generator().manual_seed(1238)
    params = make_ema_params(gen, dim, ndim)
    norm = M.TimestepNorm(dim, prior_count=2).cuda().eval()
    move = M.MultiHeadEMA(dim, ndim=ndim).cuda().eval()
    with torch.no_grad():
        for dst, src in zip((move.alpha, move.delta, move.beta, move.gamma, move.omega), params):
            dst.copy_(src)
        torch.manual_seed(1238)
        x = torch.empty(bsz, length, dim, device="cuda", dtype=torch.bfloat16)
        for b in range(bsz):
            x[b] = (torch.randn(length, dim, device="cuda") * 1.2 + 0.1).to(torch.bfloat16)
        y = M.timestep_norm_ema(norm, move, x)
        assert torch.isfinite(y[::7, ::101]).all()
        # (1) batch shards are independent and deterministic
        ys = M.timestep_norm_ema(norm, move, x[16:48])
        assert torch.equal(ys, y[16:48])
        del ys
        # (2) chunked == full
        st = {}
        half = length // 2
        y0 = M.timestep_norm_ema(norm, move, x[:, :half], None, st)
        y1 = M.timestep_norm_ema(norm, move, x[:, half:], None, st)
        assert rel_l2(y0[:8].float(), y[:8, :half].float()) < 1e-2
        assert rel_l2(y1[:8].float(), y[:8, half:].float()) < 1e-2
        assert rel_l2(y1[-8:, -4096:].float(), y[-8:, -4096:].float()) < 1e-2
        del y0, y1
        # (3) a sample of rows against the oracle over the whole length
        bs, ds = [0, 31, 63], [0, 1, 777, 1024, 1531, 2045, 2046, 2047]
        xs = x[bs][:, :, ds].float().cpu()
        ysam = y[bs][:, :, ds].float().cpu()
    pc = torch.full((len(bs),), 2, dtype=torch.int64)
    xn, _, _, _ = O.timestep_norm(xs, pc, torch.zeros(len(bs), len(ds)), torch.ones(len(bs), len(ds)),
                                  torch.ones(len(ds)), torch.zeros(len(ds)), None, acc_dtype=torch.float64)
    sub = [p[ds] for p in params]
    ref = O.ema_forward_recurrence(xn.transpose(1, 2), *sub).transpose(1, 2)
    assert rel_l2(ysam, ref) < 1e-2


@pytest.mark.parametrize("tile", [222, 224, 422, 124])
@pytest.mark.parametrize("bsz,length,dim", [(8, 8192, 64), (3, 4100, 40), (1, 2048, 16), (16, 96, 2048)])
def test_pipelined_tensor_core_forms(tile, bsz, length, dim):
    """The forms of the tensor-core kernel that are pipelined along the sequence (groups of warps
    on consecutive steps, running statistics and pole states handed over in shared memory) against
    the oracle and against the un-pipelined form of the same kernel, over many steps, with a carried state, a length that is not a multiple of the step, and fewer than 8
    sequences; the launch is checked to be the pipelined form."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(tile + length)
    prm = make_ema_params(gen, dim, 16)
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.1 - 0.3).to(torch.bfloat16)
    pc = torch.full((bsz,), 2, dtype=torch.int64)
    pc[0] = 0 if length > 1000 else 1
    pm = torch.randn(bsz, dim, generator=gen) * 0.1 - 0.3
    pv = torch.rand(bsz, dim, generator=gen) + 0.5
    gamma = torch.randn(dim, generator=gen) * 0.1 + 1
    beta = torch.randn(dim, generator=gen) * 0.1
    h0 = torch.randn(bsz, dim, 16, generator=gen) * 0.3
    want_state = length % 32 == 0
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    xn, cnt, mean, var = O.timestep_norm(x.float(), pc, pm, pv, gamma, beta, None, acc_dtype=torch.float64)[:4]
    yref, href = O.ema_forward_recurrence(xn.transpose(1, 2), *prm, None, h=h0, return_state=True)
    eref = O.ema_forward_recurrence(x.float().transpose(1, 2), *prm, None, h=h0, silu=True)
    res = {}
    for t in (tile, 22):
        _lib.set_option(2, t)
        try:
            fused = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                          p, q, g, prm[4].cuda(), None, h_in=h0.cuda(), want_state=want_state)
            name = _lib.last_kernel()
            ema = M.ops.ema_forward(x.cuda().transpose(1, 2), p, q, g, prm[4].cuda(), None, h0.cuda(), silu=True)
            name2 = _lib.last_kernel()
        finally:
            _lib.set_option(2, 0)
        res[t] = (fused, ema)
        if t == tile:
            want = "tile=%d warps_per_column=%d pipe=%d" % (tile // 100, (tile // 10) % 10, tile % 10)
            assert want in name and want in name2, (name, name2)
    fused, ema = res[tile]
    assert rel_l2(fused["y"].float(), yref.transpose(1, 2)) < 1e-2
    assert rel_l2(ema.float(), eref) < 1e-2
    assert torch.equal(fused["count"].cpu(), cnt)
    assert rel_l2(fused["mean"], mean) < 1e-4 and rel_l2(fused["var"], var) < 1e-3
    if want_state:
        assert rel_l2(fused["h"], href) < 1e-2
        assert rel_l2(fused["h"], res[22][0]["h"]) < 1e-2
    # two bf16 evaluations of the same function, each within a few 1e-3 of the oracle
    assert rel_l2(fused["y"].float(), res[22][0]["y"].float()) < 1e-2
    assert rel_l2(fused["mean"], res[22][0]["mean"]) < 1e-5 and rel_l2(fused["var"], res[22][0]["var"]) < 1e-3
    assert _lib.device_error() == 0


@pytest.mark.parametrize("runs", [2, 4, 8])
@pytest.mark.parametrize("bsz,length,dim,state", [(8, 2048, 192, True), (20, 1024, 72, False), (4, 4096, 64, True)])
def test_segmented_tensor_core_form(runs, bsz, length, dim, state):
    """The segmented form of the tensor-core kernel (the sequence cut into runs, one CTA per run and
    tile, the running sums and pole states handed from a run to the next through global memory
    behind a flag) against the oracle and, bit for bit, against the unsegmented 64-channel form:
    with and without an exported state (the pole states then travel through h_out or through the
    library's hand-off buffer), with carried-in statistics and states, the EMA alone with SiLU, a
    channel count that leaves a partial tile and a batch that leaves a partial group of sequences;
    two calls in a row reuse the counter and flags."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(runs * 1000 + length)
    prm = make_ema_params(gen, dim, 16)
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.1 - 0.3).to(torch.bfloat16)
    pc = torch.full((bsz,), 3, dtype=torch.int64)
    pc[0] = 0
    pm = torch.randn(bsz, dim, generator=gen) * 0.1 - 0.3
    pv = torch.rand(bsz, dim, generator=gen) + 0.5
    gamma = torch.randn(dim, generator=gen) * 0.1 + 1
    beta = torch.randn(dim, generator=gen) * 0.1
    h0 = torch.randn(bsz, dim, 16, generator=gen) * 0.3
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    xn, cnt, mean, var = O.timestep_norm(x.float(), pc, pm, pv, gamma, beta, None, acc_dtype=torch.float64)[:4]
    yref, href = O.ema_forward_recurrence(xn.transpose(1, 2), *prm, None, h=h0, return_state=True)
    eref = O.ema_forward_recurrence(x.float().transpose(1, 2), *prm, None, h=h0, silu=True)
    res = {}
    for t in (80 + runs, 80 + runs, 8):
        _lib.set_option(2, t)
        try:
            fused = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                          p, q, g, prm[4].cuda(), None, h_in=h0.cuda(), want_state=state)
            name = _lib.last_kernel()
            ema = M.ops.ema_forward(x.cuda().transpose(1, 2), p, q, g, prm[4].cuda(), None, h0.cuda(), silu=True)
            name2 = _lib.last_kernel()
        finally:
            _lib.set_option(2, 0)
        if t != 8:
            assert "segmented runs=%d" % runs in name and "segmented runs=%d" % runs in name2, (name, name2)
        else:
            assert "tile=8" in name and "segmented" not in name, name
        res[t] = (fused, ema)
    fused, ema = res[80 + runs]
    assert rel_l2(fused["y"].float(), yref.transpose(1, 2)) < 1e-2
    assert rel_l2(ema.float(), eref) < 1e-2
    assert torch.equal(fused["count"].cpu(), cnt)
    assert rel_l2(fused["mean"], mean) < 1e-4 and rel_l2(fused["var"], var) < 1e-3
    if state:
        assert rel_l2(fused["h"], href) < 1e-2
        assert torch.equal(fused["h"], res[8][0]["h"])
    # the hand-off is exact: the same bits as the unsegmented form
    assert torch.equal(fused["y"], res[8][0]["y"])
    assert torch.equal(ema, res[8][1])
    assert torch.equal(fused["mean"], res[8][0]["mean"]) and torch.equal(fused["var"], res[8][0]["var"])
    assert _lib.device_error() == 0


def test_segmented_form_silu_and_fewer_poles():
    """The segmented form with the SiLU epilogue, 8 poles instead of 16, a partial last tile of
    channels and a partial group of sequences: the bits of the unsegmented form."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(77)
    bsz, length, dim, ndim = 12, 1024, 136, 8
    prm = make_ema_params(gen, dim, ndim)
    x = (torch.randn(bsz, length, dim, generator=gen) * 0.9 + 0.2).to(torch.bfloat16).cuda()
    pc = torch.full((bsz,), 2, dtype=torch.int64).cuda()
    pm = (torch.randn(bsz, dim, generator=gen) * 0.1).cuda()
    pv = (torch.rand(bsz, dim, generator=gen) + 0.5).cuda()
    gamma = (torch.randn(dim, generator=gen) * 0.1 + 1).cuda()
    beta = (torch.randn(dim, generator=gen) * 0.1).cuda()
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    res = {}
    for t in (84, 8):
        _lib.set_option(2, t)
        try:
            res[t] = M.ops.tsn_ema_forward(x, pc, pm, pv, gamma, beta, 1e-5, p, q, g, prm[4].cuda(), None,
                                           want_state=True, silu=True)
            name = _lib.last_kernel()
        finally:
            _lib.set_option(2, 0)
        assert ("segmented runs=4" in name) == (t == 84), name
    xn = O.timestep_norm(x.float().cpu(), pc.cpu(), pm.cpu(), pv.cpu(), gamma.cpu(), beta.cpu(), None,
                         acc_dtype=torch.float64)[0]
    yref, href = O.ema_forward_recurrence(xn.transpose(1, 2), *prm, None, silu=True, return_state=True)
    assert rel_l2(res[84]["y"].float(), yref.transpose(1, 2)) < 1e-2
    assert rel_l2(res[84]["h"], href) < 1e-2
    for k in ("y", "h", "mean", "var", "count"):
        assert torch.equal(res[84][k], res[8][k]), k
    assert _lib.device_error() == 0


def test_segmented_form_timestep_norm_alone():
    """TimestepNorm alone (bf16, no mask) in the segmented form: the bits of the unsegmented form and the
    oracle's values."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(78)
    bsz, length, dim = 9, 2048, 200
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.4 - 0.3).to(torch.bfloat16).cuda()
    pc = torch.full((bsz,), 4, dtype=torch.int64).cuda()
    pm = (torch.randn(bsz, dim, generator=gen) * 0.1).cuda()
    pv = (torch.rand(bsz, dim, generator=gen) + 0.5).cuda()
    gamma = (torch.randn(dim, generator=gen) * 0.1 + 1).cuda()
    beta = (torch.randn(dim, generator=gen) * 0.1).cuda()
    res = {}
    for t in (84, 8):
        _lib.set_option(2, t)
        try:
            res[t] = M.ops.timestep_norm_fwd(x, pc, pm, pv, gamma, beta, None, 1e-5, None)
            name = _lib.last_kernel()
        finally:
            _lib.set_option(2, 0)
        assert "tsn_ema_mma" in name and ("segmented runs=4" in name) == (t == 84), name
    ref = O.timestep_norm(x.float().cpu(), pc.cpu(), pm.cpu(), pv.cpu(), gamma.cpu(), beta.cpu(), None,
                          acc_dtype=torch.float64)
    assert rel_l2(res[84][0].float(), ref[0]) < 1e-2
    assert torch.equal(res[84][1].cpu(), ref[1])
    assert rel_l2(res[84][2], ref[2]) < 1e-5 and rel_l2(res[84][3], ref[3]) < 1e-3
    for a, b in zip(res[84], res[8]):
        assert torch.equal(a, b)
    assert _lib.device_error() == 0


def test_segmented_form_calls_on_two_streams():
    """Two calls that take the segmented form by themselves (more than 148 wide tiles) on two streams
    without any synchronisation between them: the library orders the second behind the first on the
    device (they share its scratch), and each gives the bits it gives alone."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    free, _ = torch.cuda.mem_get_info()
    if free < 12 * 2 ** 30:
        pytest.skip("needs ~6 GiB of device memory")
    gen = torch.Generator().manual_seed(79)
    bsz, length, dim = 16, 8192, 5120
    prm = [t.cuda() for t in make_ema_params(gen, dim, 16)]
    p, q, g = M.ops.ema_coeffs(*prm[:4])
    pc = torch.full((bsz,), 2, dtype=torch.int64).cuda()
    pm, pv = torch.zeros(bsz, dim).cuda(), torch.ones(bsz, dim).cuda()
    gamma, beta = torch.ones(dim).cuda(), torch.zeros(dim).cuda()
    xs = [torch.randn(bsz, length, dim, device="cuda", dtype=torch.bfloat16) * (1.0 + 0.5 * k) for k in range(2)]
    alone = []
    for x in xs:
        alone.append(M.ops.tsn_ema_forward(x, pc, pm, pv, gamma, beta, 1e-5, p, q, g, prm[4])["y"])
        assert "segmented" in _lib.last_kernel(), _lib.last_kernel()
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = []
    for x, st in zip(xs, streams):
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            outs.append(M.ops.tsn_ema_forward(x, pc, pm, pv, gamma, beta, 1e-5, p, q, g, prm[4])["y"])
    for st in streams:
        st.synchronize()
    for y, y0 in zip(outs, alone):
        assert torch.equal(y, y0)
    assert _lib.device_error() == 0


def test_segmented_form_falls_back():
    """A number of steps that the runs do not divide takes the unsegmented kernel."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(9)
    prm = make_ema_params(gen, 64, 16)
    x = torch.randn(8, 32 * 7, 64, generator=gen).to(torch.bfloat16).cuda()
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    _lib.set_option(2, 84)
    try:
        y = M.ops.ema_forward(x.transpose(1, 2), p, q, g, prm[4].cuda(), None, None)
        name = _lib.last_kernel()
    finally:
        _lib.set_option(2, 0)
    assert "tsn_ema_mma" in name and "segmented" not in name, name
    assert torch.isfinite(y.float()).all()


@pytest.mark.parametrize("tile", [7, 22, 224, 84])
def test_bounded_wait_runs_out(tile):
    """A device-side wait that can never complete must give up, not hang: a test switch makes the
    kernel skip the TMA load of one step while its barrier keeps expecting the bytes, and shortens
    the wait limit to about a millisecond.  Every waiter of that stage gives up, all warps of the CTA
    leave the loop, the kernel returns without its final stores and the error word reads non-zero;
    after a reset the next launch is clean and correct.  Tile 84 is the segmented form: the run of the
    withheld step gives up, and the run after it, which waits for that one's flag, leaves as well."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(5)
    bsz, length, dim = 8, 1024, 64
    prm = make_ema_params(gen, dim, 16)
    x = torch.randn(bsz, length, dim, generator=gen).to(torch.bfloat16).cuda()
    pc = torch.full((bsz,), 2, dtype=torch.int64).cuda()
    pm, pv = torch.zeros(bsz, dim).cuda(), torch.ones(bsz, dim).cuda()
    gamma, beta = torch.ones(dim).cuda(), torch.zeros(dim).cuda()
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    assert _lib.device_error(reset=True) == 0
    import time
    _lib.set_option(2, tile)
    _lib.set_option(3, 2_000_000)   # wait limit in SM cycles (~1 ms)
    _lib.set_option(4, 20)          # the tile of step 20 never arrives
    try:
        t0 = time.time()
        M.ops.tsn_ema_forward(x, pc, pm, pv, gamma, beta, 1e-5, p, q, g, prm[4].cuda())
        assert "tsn_ema_mma" in _lib.last_kernel()
        torch.cuda.synchronize()
        assert time.time() - t0 < 5.0
        assert _lib.device_error(reset=True) != 0
    finally:
        _lib.set_option(3, 0)
        _lib.set_option(4, 0)
        _lib.set_option(2, 0)
    assert _lib.device_error() == 0
    res = M.ops.tsn_ema_forward(x, pc, pm, pv, gamma, beta, 1e-5, p, q, g, prm[4].cuda())
    xn = O.timestep_norm(x.float().cpu(), pc.cpu(), pm.cpu(), pv.cpu(), gamma.cpu(), beta.cpu(), None,
                         acc_dtype=torch.float64)[0]
    yref = O.ema_forward_recurrence(xn.transpose(1, 2), *prm).transpose(1, 2)
    assert rel_l2(res["y"].float(), yref) < 1e-2
    assert _lib.device_error() == 0


@pytest.mark.parametrize("tile", [7, 22])
@pytest.mark.parametrize("bsz,length,dim", [(8, 1024, 128), (9, 300, 72), (16, 4096, 64), (5, 96, 200)])
@pytest.mark.parametrize("interior", [False, True])
def test_tensor_core_path_with_padding_mask(tile, bsz, length, dim, interior):
    """bf16 with a padding mask on the tensor-core kernel (fused pair, with and without the
    normalised activations as a second output, and TimestepNorm alone): right padding of up to 40 %,
    one fully padded sequence, optionally pads in the interior, a length that is not a multiple of
    the step; against the oracle and the streamed SIMT kernel.  Padded positions of the normalised
    output are exactly zero, counts are exact, and the launch is checked to be the masked form."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(bsz * 7 + length + dim + tile)
    prm = make_ema_params(gen, dim, 16)
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.2 + 0.3).to(torch.bfloat16)
    mask = right_pad_mask(gen, bsz, length, 0.4)
    mask[bsz - 1] = True
    if interior:
        mask[0, 3] = True
        mask[1, 40:75] = True
        mask[2, 0] = True
    pc = torch.full((bsz,), 2, dtype=torch.int64)
    pc[1] = 1
    pm = torch.randn(bsz, dim, generator=gen) * 0.1 + 0.3
    pv = torch.rand(bsz, dim, generator=gen) + 0.5
    gamma = torch.randn(dim, generator=gen) * 0.1 + 1
    beta = torch.randn(dim, generator=gen) * 0.1
    h0 = torch.randn(bsz, dim, 16, generator=gen) * 0.3
    want_state = length % 32 == 0
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    xn, cnt, mean, var = O.timestep_norm(x.float(), pc, pm, pv, gamma, beta, mask, acc_dtype=torch.float64)[:4]
    yref, href = O.ema_forward_recurrence(xn.transpose(1, 2), *prm, mask, h=h0, return_state=True, silu=True)
    outs = []
    for disable in (0, 1):
        _lib.set_option(1, disable)
        _lib.set_option(2, tile)
        try:
            both = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                         p, q, g, prm[4].cuda(), mask.cuda(), h_in=h0.cuda(), want_state=want_state,
                                         want_normed=True, silu=True)
            name_both = _lib.last_kernel()
            plain = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                          p, q, g, prm[4].cuda(), mask.cuda(), h_in=h0.cuda(), silu=True)
            name_plain = _lib.last_kernel()
            tsn = M.ops.timestep_norm_fwd(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), mask.cuda())
            name_tsn = _lib.last_kernel()
            # the EMA alone: omega times the UNMASKED input stays at padded positions
            ema = M.ops.ema_forward(x.cuda().transpose(1, 2), p, q, g, prm[4].cuda(), mask.cuda(), h0.cuda(),
                                    want_state=want_state, silu=True)
            name_ema = _lib.last_kernel()
        finally:
            _lib.set_option(1, 0)
            _lib.set_option(2, 0)
        if disable == 0:
            for n in (name_both, name_plain, name_tsn, name_ema):
                assert "tsn_ema_mma" in n and "mask" in n, n
        eref, ehref = O.ema_forward_recurrence(x.float().transpose(1, 2), *prm, mask, h=h0, return_state=True, silu=True)
        assert rel_l2((ema[0] if want_state else ema).float(), eref) < 1e-2, disable
        if want_state:
            assert rel_l2(ema[1], ehref) < 1e-2, disable
        outs.append((both, plain, tsn))
        assert rel_l2(both["y"].float(), yref.transpose(1, 2)) < 1e-2, disable
        assert rel_l2(plain["y"].float(), yref.transpose(1, 2)) < 1e-2, disable
        assert rel_l2(both["xn"].float(), xn) < 1e-2 and rel_l2(tsn[0].float(), xn) < 1e-2, disable
        assert (both["xn"].cpu()[mask] == 0).all() and (tsn[0].cpu()[mask] == 0).all()
        assert torch.equal(both["count"].cpu(), cnt) and torch.equal(tsn[1].cpu(), cnt)
        assert rel_l2(both["mean"], mean) < 1e-4 and rel_l2(both["var"], var) < 2e-3, disable
        assert rel_l2(tsn[2], mean) < 1e-4 and rel_l2(tsn[3], var) < 2e-3, disable
        if want_state:
            assert rel_l2(both["h"], href) < 1e-2, disable
    # the fully padded sequence hands its incoming statistics back unchanged
    assert torch.allclose(outs[0][0]["mean"][bsz - 1].cpu(), pm[bsz - 1], atol=1e-6)
    assert torch.allclose(outs[0][0]["var"][bsz - 1].cpu(), pv[bsz - 1], rtol=1e-5)
    assert rel_l2(outs[0][0]["y"].float(), outs[1][0]["y"].float()) < 1e-2
    assert _lib.device_error() == 0


@pytest.mark.parametrize("length", [1000, 33, 4100])
def test_ragged_length_with_exported_state(length):
    """A state is exported and the length is not a multiple of the tensor-core kernel's step: the
    head runs on the tensor-core kernel and the ragged tail on the streamed kernel, continuing in
    place from the head's statistics and pole states (two launches); outputs, states, statistics and
    counts against the oracle, for the fused pair and for the EMA alone."""
    M, O = _mods()
    from fairseq_apollo_b200 import _lib
    gen = torch.Generator().manual_seed(length)
    bsz, dim = 8, 128
    prm = make_ema_params(gen, dim, 16)
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.1 + 0.2).to(torch.bfloat16)
    pc = torch.full((bsz,), 3, dtype=torch.int64)
    pm = torch.randn(bsz, dim, generator=gen) * 0.1 + 0.2
    pv = torch.rand(bsz, dim, generator=gen) + 0.5
    gamma = torch.randn(dim, generator=gen) * 0.1 + 1
    beta = torch.randn(dim, generator=gen) * 0.1
    h0 = torch.randn(bsz, dim, 16, generator=gen) * 0.3
    p, q, g = M.ops.ema_coeffs(*[t.cuda() for t in prm[:4]])
    before = M.launch_count()
    res = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                p, q, g, prm[4].cuda(), None, h_in=h0.cuda(), want_state=True, want_normed=True)
    assert M.launch_count() - before == 2 and "stream_cl" in _lib.last_kernel()
    xn, cnt, mean, var = O.timestep_norm(x.float(), pc, pm, pv, gamma, beta, None, acc_dtype=torch.float64)[:4]
    yref, href = O.ema_forward_recurrence(xn.transpose(1, 2), *prm, None, h=h0, return_state=True)
    assert rel_l2(res["y"].float(), yref.transpose(1, 2)) < 1e-2 and rel_l2(res["xn"].float(), xn) < 1e-2
    assert rel_l2(res["h"], href) < 1e-2
    assert torch.equal(res["count"].cpu(), cnt)
    assert rel_l2(res["mean"], mean) < 1e-4 and rel_l2(res["var"], var) < 1e-3
    before = M.launch_count()
    y, h = M.ops.ema_forward(x.cuda().transpose(1, 2), p, q, g, prm[4].cuda(), None, h0.cuda(), want_state=True)
    assert M.launch_count() - before == 2
    eref, ehref = O.ema_forward_recurrence(x.float().transpose(1, 2), *prm, None, h=h0, return_state=True)
    assert rel_l2(y.float(), eref) < 1e-2 and rel_l2(h, ehref) < 1e-2
    # against the whole call on the streamed kernel
    _lib.set_option(1, 1)
    try:
        ref2 = M.ops.tsn_ema_forward(x.cuda(), pc.cuda(), pm.cuda(), pv.cuda(), gamma.cuda(), beta.cuda(), 1e-5,
                                     p, q, g, prm[4].cuda(), None, h_in=h0.cuda(), want_state=True)
    finally:
        _lib.set_option(1, 0)
    assert rel_l2(res["y"].float(), ref2["y"].float()) < 1e-2 and rel_l2(res["h"], ref2["h"]) < 1e-2
    assert _lib.device_error() == 0
