"""The segmented form of the fused TimestepNorm -> EMA on request (mega_tsn_ema_fwd_runs), which works
out of fixed device arrays of the library and allocates nothing, against the regular entry point
(mega_tsn_ema_fwd): the same bits, on two calls in a row (the second reuses the counter, the flags
and the hand-off arrays the first left behind), with and without an exported state, and a refusal
beyond the arrays' sizes.  Collected last: it shares the library's scratch with the regular path."""
import pytest
import torch

from _util import make_ema_params, rel_l2

pytestmark = pytest.mark.gpu


def _call(M, _lib, entry, x, pc, pm, pv, gamma, beta, p, q, g, omega, h_in, want_state, runs=None):
    bsz, length, dim = x.shape
    y = torch.empty_like(x)
    count = torch.empty(bsz, device=x.device, dtype=torch.int64)
    mean = torch.empty(bsz, dim, device=x.device, dtype=torch.float32)
    var = torch.empty_like(mean)
    h_out = torch.empty(bsz, dim, p.shape[1], device=x.device, dtype=torch.float32) if want_state else None
    stream = torch.cuda.current_stream().cuda_stream
    hp = None if h_out is None else h_out.data_ptr()
    head = (x.data_ptr(), y.data_ptr())
    mid = (1, bsz, length, dim, *x.stride(), *y.stride(), pc.data_ptr(), pm.data_ptr(), pv.data_ptr(),
           gamma.data_ptr(), beta.data_ptr(), 1e-5, count.data_ptr(), mean.data_ptr(), var.data_ptr(),
           p.data_ptr(), q.data_ptr(), g.data_ptr(), omega.data_ptr(), p.shape[1])
    if runs is None:
        rc = entry(*head, None, *mid, None, h_in.data_ptr(), hp, 0, stream)
    else:
        rc = entry(*head, *mid, h_in.data_ptr(), hp, 0, runs, stream)
    return rc, y, count, mean, var, h_out


@pytest.mark.parametrize("runs,want_state", [(4, False), (2, True), (8, False)])
def test_runs_entry_point_matches_the_regular_one(runs, want_state):
    import fairseq_apollo_b200 as M
    from fairseq_apollo_b200 import _lib
    lib = _lib.lib()
    bsz, length, dim = 12, 2048, 200
    gen = torch.Generator().manual_seed(31 + runs)
    prm = [t.cuda() for t in make_ema_params(gen, dim, 16)]
    p, q, g = M.ops.ema_coeffs(*prm[:4])
    omega = prm[4].float().contiguous()
    x = (torch.randn(bsz, length, dim, generator=gen) * 1.3 + 0.2).to(torch.bfloat16).cuda()
    pc = torch.full((bsz,), 5, dtype=torch.int64).cuda()
    pm = (torch.randn(bsz, dim, generator=gen) * 0.1).cuda()
    pv = (torch.rand(bsz, dim, generator=gen) + 0.5).cuda()
    gamma = (torch.randn(dim, generator=gen) * 0.1 + 1).cuda()
    beta = (torch.randn(dim, generator=gen) * 0.1).cuda()
    h0 = (torch.randn(bsz, dim, 16, generator=gen) * 0.3).cuda()
    args = (x, pc, pm, pv, gamma, beta, p, q, g, omega, h0, want_state)
    # the regular entry point: as it dispatches by itself (here a form pipelined along the sequence), and
    # held to the unsegmented 64-channel form of the same kernel, which the runs reproduce bit for bit
    rc, yd = _call(M, _lib, lib.mega_tsn_ema_fwd, *args)[:2]
    assert rc == 0
    _lib.set_option(2, 8)
    try:
        rc, y0, c0, m0, v0, hs0 = _call(M, _lib, lib.mega_tsn_ema_fwd, *args)
        assert rc == 0 and "tile=8" in _lib.last_kernel() and "segmented" not in _lib.last_kernel()
    finally:
        _lib.set_option(2, 0)
    for _ in range(2):   # two calls in a row
        rc, y1, c1, m1, v1, hs1 = _call(M, _lib, lib.mega_tsn_ema_fwd_runs, *args, runs=runs)
        assert rc == 0, _lib.lib().mega_status_string(rc)
        assert "segmented runs=%d" % runs in _lib.last_kernel()
        torch.cuda.synchronize()
        assert torch.equal(y1, y0) and torch.equal(c1, c0) and torch.equal(m1, m0) and torch.equal(v1, v0)
        if want_state:
            assert torch.equal(hs1, hs0)
        assert rel_l2(y1.float(), yd.float()) < 1e-2
    assert _lib.device_error() == 0


def test_runs_entry_point_refuses_what_its_arrays_cannot_hold():
    """B x D beyond the running-sum array (256 Ki channels) and a length the runs do not divide:
    MEGA_ERR_UNSUPPORTED (7); a number of runs other than 2, 4, 8: MEGA_ERR_SHAPE (3); nothing launched."""
    import fairseq_apollo_b200 as M
    from fairseq_apollo_b200 import _lib
    lib = _lib.lib()
    gen = torch.Generator().manual_seed(3)

    def attempt(bsz, length, dim, runs=4):
        prm = [t.cuda() for t in make_ema_params(gen, dim, 16)]
        p, q, g = M.ops.ema_coeffs(*prm[:4])
        x = torch.zeros(bsz, length, dim, dtype=torch.bfloat16, device="cuda")
        pc = torch.zeros(bsz, dtype=torch.int64, device="cuda")
        pm = torch.zeros(bsz, dim, device="cuda")
        pv = torch.ones(bsz, dim, device="cuda")
        one, zero = torch.ones(dim, device="cuda"), torch.zeros(dim, device="cuda")
        h0 = torch.zeros(bsz, dim, 16, device="cuda")
        before = M.launch_count()
        rc = _call(M, _lib, lib.mega_tsn_ema_fwd_runs, x, pc, pm, pv, one, zero, p, q, g,
                   prm[4].float().contiguous(), h0, False, runs=runs)[0]
        return rc, M.launch_count() - before

    assert attempt(40, 128, 8192) == (7, 0)            # 40 x 8192 = 320 Ki channels
    assert attempt(8, 32 * 6, 64) == (7, 0)            # 6 steps in 4 runs
    rc, launched = attempt(8, 256, 64, runs=3)
    assert rc == 3 and launched == 0                   # MEGA_ERR_SHAPE: runs is 2, 4 or 8
