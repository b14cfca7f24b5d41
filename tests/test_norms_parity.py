"""GPU parity of TimestepNorm / SequenceNorm against the golden vectors of the reference's
CPU C++ ops and the oracle.  fp32 <= 1e-5 relative L2, bf16 <= 1e-2; padded outputs exactly 0."""
import pytest
import torch

from _util import golden, opt_mask, rel_l2, right_pad_mask

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 2e-3}


def _mods():
    import fairseq_apollo_b200 as M
    from oracle import mega_oracle as O
    return M, O


@pytest.mark.parametrize("name", ["tsn_plain", "tsn_plain_nomask", "tsn_group2", "tsn_group_prior"])
def test_tsn_golden(name):
    M, _ = _mods()
    g = golden(name)
    mask = opt_mask(g["mask"])
    groups = None if g["groups"] < 0 else g["groups"]
    y, cnt, mean, var = M.ops.timestep_norm_fwd(g["x"].cuda(), g["prev_count"].cuda(), g["prev_mean"].cuda(),
                                                g["prev_var"].cuda(), g["gamma"].cuda(), g["beta"].cuda(),
                                                None if mask is None else mask.cuda(), 1e-5, groups)
    assert torch.equal(cnt.cpu(), g["count"])
    assert rel_l2(y, g["y"]) < 1e-5
    assert rel_l2(mean, g["mean"]) < 1e-5 and rel_l2(var, g["var"]) < 1e-5
    if mask is not None:
        assert (y.cpu()[mask] == 0).all()


@pytest.mark.parametrize("bsz,length,feat,groups", [(1, 1, 1, None), (2, 300, 33, None), (9, 17, 128, None),
                                                     (2, 50, 64, 4), (3, 33, 96, 3), (2, 20, 70, 1),
                                                     (2, 70, 128, 16), (2, 257, 128, 2), (3, 100, 192, 6)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_tsn_grid(bsz, length, feat, groups, dtype):
    M, O = _mods()
    gen = torch.Generator().manual_seed(length * 7 + feat)
    x = (torch.randn(bsz, length, feat, generator=gen) * 1.5 + 0.2).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.4)
    if length > 4:
        mask[0, 2] = True
    ng = feat if groups is None else groups
    prev_count = torch.full((bsz,), 2, dtype=torch.int64)
    prev_mean = torch.randn(bsz, ng, generator=gen) * 0.1
    prev_var = torch.rand(bsz, ng, generator=gen) + 0.5
    gamma = torch.randn(feat, generator=gen) * 0.1 + 1
    beta = torch.randn(feat, generator=gen) * 0.1
    if groups is None:
        ref = O.timestep_norm(x.float(), prev_count, prev_mean, prev_var, gamma, beta, mask)
    else:
        ref = O.group_timestep_norm(x.float(), prev_count, prev_mean, prev_var, gamma, beta, mask, groups)
    y, cnt, mean, var = M.ops.timestep_norm_fwd(x.cuda(), prev_count.cuda(), prev_mean.cuda(), prev_var.cuda(),
                                                gamma.cuda(), beta.cuda(), mask.cuda(), 1e-5, groups)
    assert torch.equal(cnt.cpu(), ref[1])
    assert rel_l2(y.float(), ref[0]) < TOL[dtype]
    # (bf16 with at least 4 sequences and 8-aligned features runs the tensor-core kernel, whose sums of
    # squares go through tf32 MMAs: ~2^-11 of the variance)
    assert rel_l2(mean, ref[2]) < 1e-5 and rel_l2(var, ref[3]) < (1e-3 if dtype == torch.bfloat16 else 1e-5)
    assert (y.cpu()[mask] == 0).all()


def test_tsn_chunked_equals_full():
    M, _ = _mods()
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(2, 96, 20, generator=gen).cuda()
    pc = torch.full((2,), 2, dtype=torch.int64).cuda()
    pm = torch.zeros(2, 20).cuda()
    pv = torch.ones(2, 20).cuda()
    gam = torch.ones(20).cuda()
    bet = torch.zeros(20).cuda()
    full = M.ops.timestep_norm_fwd(x, pc, pm, pv, gam, bet)
    ys = []
    st = (pc, pm, pv)
    for i in range(0, 96, 32):
        y, c, m, v = M.ops.timestep_norm_fwd(x[:, i:i + 32], st[0], st[1], st[2], gam, bet)
        st = (c, m, v)
        ys.append(y)
    assert rel_l2(torch.cat(ys, 1), full[0]) < 1e-6
    assert torch.equal(st[0], full[1]) and rel_l2(st[1], full[2]) < 1e-6 and rel_l2(st[2], full[3]) < 1e-6


@pytest.mark.parametrize("name", ["sqn_bhl", "sqn_blh", "sqn_bhl_group", "sqn_blh_group"])
def test_sqn_golden(name):
    M, _ = _mods()
    g = golden(name)
    mask = opt_mask(g["mask"])
    groups = None if g["groups"] < 0 else g["groups"]
    y, cnt, mean, rstd = M.ops.sequence_norm_fwd(g["x"].cuda(), g["gamma"].cuda(), g["beta"].cuda(),
                                                 None if mask is None else mask.cuda(), 1e-5,
                                                 bool(g["length_last"]), groups)
    assert torch.equal(cnt.cpu(), g["count"])
    assert rel_l2(y, g["y"]) < 1e-5
    assert rel_l2(mean, g["mean"]) < 1e-5 and rel_l2(rstd, g["rstd"]) < 1e-5
    if mask is not None:
        yy = y.cpu() if g["length_last"] else y.cpu().transpose(1, 2)
        assert (yy.transpose(1, 2)[mask] == 0).all()


@pytest.mark.parametrize("bsz,feat,length,groups", [(1, 1, 1, None), (2, 33, 300, None), (3, 8, 20000, None),
                                                     (2, 64, 50, 4), (2, 12, 11000, 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["bdl", "bld_view", "blh_op"])
def test_sqn_grid(bsz, feat, length, groups, dtype, layout):
    M, O = _mods()
    gen = torch.Generator().manual_seed(length + feat)
    x = (torch.randn(bsz, feat, length, generator=gen) * 2 - 0.5).to(dtype)
    mask = right_pad_mask(gen, bsz, length, 0.5)
    if bsz > 1:
        mask[bsz - 1] = True
    gamma = torch.randn(feat, generator=gen) * 0.1 + 1
    beta = torch.randn(feat, generator=gen) * 0.1
    ref = O.sequence_norm(x.float(), gamma, beta, mask, groups, 1e-5, True)
    xc = x.cuda()
    if layout == "bld_view":
        xc = xc.transpose(1, 2).contiguous().transpose(1, 2)
    if layout == "blh_op":
        y, cnt, mean, rstd = M.ops.sequence_norm_fwd(xc.transpose(1, 2).contiguous(), gamma.cuda(), beta.cuda(),
                                                     mask.cuda(), 1e-5, False, groups)
        y = y.transpose(1, 2)
    else:
        y, cnt, mean, rstd = M.ops.sequence_norm_fwd(xc, gamma.cuda(), beta.cuda(), mask.cuda(), 1e-5, True, groups)
    assert torch.equal(cnt.cpu(), ref[1])
    assert rel_l2(y.float(), ref[0]) < TOL[dtype]
    assert rel_l2(mean, ref[2]) < 1e-4 and rel_l2(rstd, ref[3]) < 1e-4
    assert (y.cpu().transpose(1, 2)[mask] == 0).all()


def test_modules_golden():
    M, _ = _mods()
    g = golden("tsn_module")
    t = M.TimestepNorm(10, num_groups=None, prior_count=2)
    t.load_state_dict({k[3:]: torch.as_tensor(v) for k, v in g.items() if k.startswith("sd_")}, strict=True)
    t = t.cuda().eval()
    with torch.no_grad():
        x = g["x"].cuda()
        assert rel_l2(t(x), g["y_full"]) < 1e-5
        st = {}
        y = torch.cat([t(x[:, :16], None, st), t(x[:, 16:], None, st)], 1)
        assert rel_l2(y, g["y_chunked"]) < 1e-5
        key = t._get_full_incremental_state_key("norm_state")
        assert set(st[key]) == {"prev_mean", "prev_var", "prev_count"}
        t.reorder_incremental_state(st, torch.tensor([1, 0]).cuda())
    g = golden("sqn_module")
    s = M.SequenceNorm(6)
    s.load_state_dict({k[3:]: torch.as_tensor(v) for k, v in g.items() if k.startswith("sd_")}, strict=True)
    s = s.cuda().eval()
    with torch.no_grad():
        assert rel_l2(s(g["x"].cuda(), g["mask"].cuda()), g["y"]) < 1e-5
