"""GPU parity at the shapes of the benchmark configurations, on the kernels the benchmark times.

Config 1 at its full batch on the tensor-core kernel, config 2's SequenceNorm -> bidirectional EMA
at its full length with right padding, config 4's decode half (1024 single-token steps after a
4096-token prefix) against the float64 recurrence, many-chunk incremental calls on the tensor-core
kernel, and the single-token fast path at batch size 1.
"""
import pytest
import torch

from _util import make_ema_params, rel_l2, right_pad_mask

pytestmark = pytest.mark.gpu


def _mods():
    import fairseq_apollo_b200 as M
    from fairseq_apollo_b200 import _lib
    from oracle import mega_oracle as O
    return M, O, _lib


def _modules(M, dim, params, prior_count=2, complex_poles=False):
    norm = M.TimestepNorm(dim, prior_count=prior_count).cuda().eval()
    move = M.MultiHeadEMA(dim, ndim=16).cuda().eval()
    with torch.no_grad():
        for dst, src in zip((move.alpha, move.delta, move.beta, move.gamma, move.omega), params):
            dst.copy_(src)
    return norm, move


def _oracle_rows(O, xs, params, ds, pc_value, prior_mean=None, prior_var=None, h=None, return_state=False):
    """float64 TimestepNorm + recurrence on the sampled rows xs (b, L, len(ds))."""
    nb, nd = xs.shape[0], len(ds)
    pc = torch.full((nb,), pc_value, dtype=torch.int64)
    pm = torch.zeros(nb, nd) if prior_mean is None else prior_mean
    pv = torch.ones(nb, nd) if prior_var is None else prior_var
    xn, cnt, mean, var = O.timestep_norm(xs, pc, pm, pv, torch.ones(nd), torch.zeros(nd), None,
                                         acc_dtype=torch.float64)
    sub = [p[ds] for p in params]
    out = O.ema_forward_recurrence(xn.transpose(1, 2), *sub, None, h=h, return_state=return_state)
    return xn, out, cnt, mean, var


def test_config1_full_batch_on_tensor_core_kernel():
    """BASELINE config 1 as benchmarked: B=16, L=4096, D=1024, bf16 activations, fp32 parameters,
    TimestepNorm weight 1 / bias 0 / eps 1e-5, no padding.  The launch must be the tensor-core kernel;
    sampled (sequence, channel) rows are compared with the float64 oracle over the whole length and
    the whole output with the streamed SIMT kernel."""
    M, O, _lib = _mods()
    gen = torch.Generator().manual_seed(1235)
    bsz, length, dim = 16, 4096, 1024
    params = make_ema_params(gen, dim, 16)
    x = torch.randn(bsz, length, dim, generator=gen).to(torch.bfloat16).cuda()
    norm, move = _modules(M, dim, params)
    with torch.no_grad():
        y = M.timestep_norm_ema(norm, move, x)
        assert "tsn_ema_mma" in _lib.last_kernel(), _lib.last_kernel()
        _lib.set_option(1, 1)
        try:
            y_simt = M.timestep_norm_ema(norm, move, x)
            assert "stream_cl" in _lib.last_kernel(), _lib.last_kernel()
        finally:
            _lib.set_option(1, 0)
    assert rel_l2(y.float(), y_simt.float()) < 1e-2
    bs, ds = [0, 7, 8, 15], [0, 1, 511, 512, 1000, 1022, 1023]
    xs = x[bs][:, :, ds].float().cpu()
    _, ref, _, _, _ = _oracle_rows(O, xs, params, ds, 2)
    assert rel_l2(y[bs][:, :, ds].float().cpu(), ref.transpose(1, 2)) < 1e-2
    assert _lib.device_error() == 0


@pytest.mark.parametrize("shift", [True, False])
def test_config2_bidirectional_sequence_norm_full_length(shift):
    """BASELINE config 2's shape at reduced batch: fp32, L=16384, D=256, bidirectional ndim=16 EMA after
    SequenceNorm, right padding of 0-50 % per sequence and one fully padded sequence; through the
    fused row-resident kernel (checked by name) and through the two modules in turn.  Tolerance
    1e-5 relative L2 against the float64 oracle; padded positions of the normalised activations
    are exactly zero."""
    M, O, _lib = _mods()
    gen = torch.Generator().manual_seed(1236)
    bsz, dim, length = 4, 256, 16384
    x = torch.randn(bsz, dim, length, generator=gen)
    mask = right_pad_mask(gen, bsz, length, 0.5)
    mask[1, length // 2:] = True
    mask[bsz - 1] = True
    norm = M.SequenceNorm(dim).cuda().eval()
    move = M.MultiHeadEMA(dim, ndim=16, bidirectional=True, shift=shift).cuda().eval()
    params = make_ema_params(gen, dim, 16, bidirectional=True)
    with torch.no_grad():
        for dst, src in zip((move.alpha, move.delta, move.beta, move.gamma, move.omega), params):
            dst.copy_(src)
        y = M.sequence_norm_ema(norm, move, x.cuda(), mask.cuda())
        assert "rowres" in _lib.last_kernel(), _lib.last_kernel()
        xn_gpu = norm(x.cuda(), mask.cuda())
        y2 = move(xn_gpu, mask.cuda())
    assert (xn_gpu.cpu()[mask.unsqueeze(1).expand(-1, dim, -1)] == 0).all()
    xn = O.sequence_norm(x, torch.ones(dim), torch.zeros(dim), mask)[0]
    assert rel_l2(xn_gpu, xn) < 1e-5
    ds = list(range(0, dim, 37)) + [dim - 1]
    sub = [p[ds + [d + dim for d in ds]] if p.shape[0] == 2 * dim else p[ds] for p in params]
    ref = O.ema_forward_recurrence(xn[:, ds], *sub, mask, bidirectional=True, shift=shift)
    assert rel_l2(y[:, ds].cpu(), ref) < 1e-5
    assert rel_l2(y2[:, ds].cpu(), ref) < 1e-5
    assert torch.isfinite(y).all()


def test_config4_decode_1024_steps():
    """BASELINE config 4's decode half: the states are seeded by a 4096-token prefix (tensor-core
    kernel), then 1024 single-token steps run through the module fast path (in-place fused step
    kernel) and, separately, through the C entry point mega_tsn_ema_step directly.  Sampled
    (sequence, channel) rows are compared with the float64 recurrence over all 5120 positions, and so
    are the pole states and running statistics after the last step."""
    M, O, _lib = _mods()
    gen = torch.Generator().manual_seed(1238)
    bsz, dim, prefix, steps = 64, 2048, 4096, 1024
    params = make_ema_params(gen, dim, 16)
    norm, move = _modules(M, dim, params)
    xp = (torch.randn(bsz, prefix, dim, generator=gen) * 1.1 + 0.05).to(torch.bfloat16).cuda()
    xs = (torch.randn(steps, bsz, 1, dim, generator=gen) * 1.1 + 0.05).to(torch.bfloat16).cuda()
    st = {}
    with torch.no_grad():
        y0 = M.timestep_norm_ema(norm, move, xp, None, st)
        assert "tsn_ema_mma" in _lib.last_kernel()
        # a second state for the direct C-ABI loop, cloned before the module loop updates it in place
        nst, est = norm._get_input_buffer(st), move._get_input_buffer(st)
        cnt = nst['prev_count'].clone()
        mean, var = nst['prev_mean'].float().clone().contiguous(), nst['prev_var'].float().clone().contiguous()
        h = est['prev_state'].clone().contiguous()
        before = M.launch_count()
        ys = [M.timestep_norm_ema(norm, move, xs[t], None, st) for t in range(steps)]
        # the fast path: fused single-token kernel(s), not the general forward kernels
        assert M.launch_count() - before <= 2 * steps + 32   # (+ the one-off coefficient kernels)
        y_mod = torch.cat(ys, 1)
        p, q, g = M.ops.ema_coeffs(move.alpha, move.delta, move.beta, move.gamma)
        gamma, beta = torch.ones(dim, device="cuda"), torch.zeros(dim, device="cuda")
        y_abi = torch.empty(bsz, steps, dim, dtype=torch.bfloat16, device="cuda")
        yt = torch.empty(bsz, dim, dtype=torch.bfloat16, device="cuda")
        for t in range(steps):
            M.ops.tsn_ema_step_(xs[t].view(bsz, dim), yt, cnt, mean, var, gamma, beta, 1e-5, p, q, g,
                                move.omega.detach().float(), h)
            y_abi[:, t] = yt
    assert torch.equal(y_abi, y_mod)
    nst, est = norm._get_input_buffer(st), move._get_input_buffer(st)
    assert torch.equal(nst['prev_count'].cpu(), torch.full((bsz,), 2 + prefix + steps, dtype=torch.int64))
    assert torch.equal(cnt, nst['prev_count'])
    bs, ds = [0, 13, 63], [0, 5, 1024, 2047]
    xall = torch.cat([xp[bs][:, :, ds], xs[:, bs, 0][:, :, ds].transpose(0, 1)], 1).float().cpu()
    _, (ref, href), _, mref, vref = _oracle_rows(O, xall, params, ds, 2, return_state=True)
    ref = ref.transpose(1, 2)
    got = torch.cat([y0[bs][:, :, ds], y_mod[bs][:, :, ds]], 1).float().cpu()
    assert rel_l2(got[:, :prefix], ref[:, :prefix]) < 1e-2
    assert rel_l2(got[:, prefix:], ref[:, prefix:]) < 1e-2
    # drift check on the last 64 steps alone
    assert rel_l2(got[:, -64:], ref[:, -64:]) < 1e-2
    assert rel_l2(est['prev_state'][bs][:, ds].cpu(), href) < 1e-2
    assert rel_l2(nst['prev_mean'][bs][:, ds].cpu(), mref) < 1e-3
    assert rel_l2(nst['prev_var'][bs][:, ds].cpu(), vref) < 2e-3
    assert rel_l2(h[bs][:, ds].cpu(), href) < 1e-2


@pytest.mark.parametrize("chunks", [8, 16])
def test_many_chunks_equal_full_on_tensor_core_kernel(chunks):
    """Incremental calls in bf16 on the tensor-core kernel: the statistics carried from chunk to
    chunk come out of tf32 products, so 8 and 16 chunks are compared with the single full call and
    with the float64 oracle (the error must not build up from chunk to chunk)."""
    M, O, _lib = _mods()
    gen = torch.Generator().manual_seed(chunks)
    bsz, length, dim = 8, 8192, 128
    params = make_ema_params(gen, dim, 16)
    norm, move = _modules(M, dim, params)
    x = (torch.randn(bsz, length, dim, generator=gen) * 0.9 + 0.3).to(torch.bfloat16).cuda()
    step = length // chunks
    st = {}
    with torch.no_grad():
        full = M.timestep_norm_ema(norm, move, x)
        outs = []
        for c in range(chunks):
            outs.append(M.timestep_norm_ema(norm, move, x[:, c * step:(c + 1) * step], None, st))
            assert "tsn_ema_mma" in _lib.last_kernel(), _lib.last_kernel()
    got = torch.cat(outs, 1)
    assert rel_l2(got.float(), full.float()) < 5e-3
    assert rel_l2(got[:, -step:].float(), full[:, -step:].float()) < 5e-3
    ds = [0, 17, 127]
    _, ref, _, mref, vref = _oracle_rows(O, x[:, :, ds].float().cpu(), params, ds, 2)
    assert rel_l2(got[:, :, ds].float().cpu(), ref.transpose(1, 2)) < 1e-2
    nst = norm._get_input_buffer(st)
    assert rel_l2(nst['prev_mean'][:, ds].cpu(), mref) < 1e-4
    assert rel_l2(nst['prev_var'][:, ds].cpu(), vref) < 2e-3


@pytest.mark.parametrize("bsz", [1, 3])
@pytest.mark.parametrize("complex_poles", [False, True])
def test_single_token_fast_path_small_batch(bsz, complex_poles):
    """The in-place single-token step through the module at batch size 1 and 3, from an empty
    incremental state: contiguous (B, 1, D) slices, so the fast path is the one that runs (checked
    by its launch count); the outputs equal the full-length call, and the module's prior statistics
    (parameters) are bit-identical afterwards: the step must update copies, never the parameters."""
    M, O, _lib = _mods()
    gen = torch.Generator().manual_seed(11 + bsz)
    dim, length = 48, 40
    norm = M.TimestepNorm(dim, prior_count=2).cuda().eval()
    move = (M.MultiHeadComplexEMA(dim, ndim=16) if complex_poles else M.MultiHeadEMA(dim, ndim=16)).cuda().eval()
    with torch.no_grad():
        norm.prior_mean.normal_(0, 0.2)
        norm.prior_logv.normal_(0, 0.2)
    x = torch.randn(bsz, length, dim, generator=gen).cuda()
    keep = [t.detach().clone() for t in (norm.prior_mean, norm.prior_logv, norm.prior_count)]
    with torch.no_grad():
        full = M.timestep_norm_ema(norm, move, x)
        st = {}
        before = M.launch_count()
        outs = [M.timestep_norm_ema(norm, move, x[:, i:i + 1].contiguous(), None, st) for i in range(length)]
        launches = M.launch_count() - before
    # one or two launches of the step kernel per token, plus the coefficient kernels of the first call
    assert launches <= 2 * length + 4, launches
    assert rel_l2(torch.cat(outs, 1), full) < 1e-5
    for a, b in zip(keep, (norm.prior_mean, norm.prior_logv, norm.prior_count)):
        assert torch.equal(a, b.detach())
    # a second generation from a fresh state reproduces the first (the priors were not corrupted)
    with torch.no_grad():
        st2 = {}
        outs2 = [M.timestep_norm_ema(norm, move, x[:, i:i + 1].contiguous(), None, st2) for i in range(length)]
    assert torch.equal(torch.cat(outs2, 1), torch.cat(outs, 1))
