"""Drop-in acceptance at operator level: the reference's own wrappers around its native extension
(norm_layer/timestep_norm.py, norm_layer/sequence_norm.py, attention_softmax.py,
efficient_attention.py, staged unmodified under oracle/_ref/py) run with this package's
``mega2_ops`` bound as ``fairseq.mega2_extension.ops``; their forward results and the gradients
through their autograd Functions are compared with the fixtures produced by the reference's CPU
operators."""
import pytest
import torch

from _util import golden, opt_mask, rel_l2

pytestmark = pytest.mark.gpu


def _wrappers():
    import fairseq_apollo_b200.mega2_ops as shim
    from oracle import build_ref
    mods = build_ref.load_reference_wrappers(shim)
    if mods is None:
        pytest.skip("oracle/_ref/py is not staged (python oracle/build_ref.py needs the reference checkout)")
    return mods


def _leaf(t):
    return t.clone().cuda().requires_grad_(True)


@pytest.mark.parametrize("name", ["tsn_bwd_plain", "tsn_bwd_plain_nomask", "tsn_bwd_group", "tsn_bwd_group_prior"])
def test_reference_timestep_norm_function_on_this_library(name):
    tsn, _, _, _ = _wrappers()
    g = golden(name)
    x, pm, pv, gamma, beta = [_leaf(g[k]) for k in ("x", "prev_mean", "prev_var", "gamma", "beta")]
    mask = opt_mask(g["mask"])
    groups = None if g["groups"] < 0 else int(g["groups"])
    y, count, mean, var = tsn.timestep_norm(x, g["prev_count"].cuda(), pm, pv, gamma, beta,
                                            None if mask is None else mask.cuda(), groups, 1e-5)
    loss = (y * g["dy"].cuda()).sum() + (mean * g["dmean"].cuda()).sum() + (var * g["dvar"].cuda()).sum()
    loss.backward()
    for t, k in ((x, "dx"), (pm, "dprev_mean"), (pv, "dprev_var"), (gamma, "dgamma"), (beta, "dbeta")):
        assert rel_l2(t.grad, g[k]) < 1e-4, k


@pytest.mark.parametrize("name", ["tsn_plain", "tsn_plain_nomask", "tsn_group2", "tsn_group_prior"])
def test_reference_timestep_norm_forward_on_this_library(name):
    tsn, _, _, _ = _wrappers()
    g = golden(name)
    mask = opt_mask(g["mask"])
    groups = None if g["groups"] < 0 else int(g["groups"])
    with torch.no_grad():
        y, count, mean, var = tsn.timestep_norm(g["x"].cuda(), g["prev_count"].cuda(), g["prev_mean"].cuda(),
                                                g["prev_var"].cuda(), g["gamma"].cuda(), g["beta"].cuda(),
                                                None if mask is None else mask.cuda(), groups, 1e-5)
    assert rel_l2(y, g["y"]) < 1e-5 and torch.equal(count.cpu(), g["count"])
    assert rel_l2(mean, g["mean"]) < 1e-5 and rel_l2(var, g["var"]) < 1e-5
    if mask is not None:
        assert (y.cpu()[mask] == 0).all()


@pytest.mark.parametrize("name", ["sqn_bwd_bhl", "sqn_bwd_blh", "sqn_bwd_bhl_group", "sqn_bwd_blh_group"])
def test_reference_sequence_norm_function_on_this_library(name):
    _, sqn, _, _ = _wrappers()
    g = golden(name)
    x, gamma, beta = [_leaf(g[k]) for k in ("x", "gamma", "beta")]
    groups = g.get("groups")
    y = sqn.sequence_norm(x, gamma, beta, g["mask"].bool().cuda(), None if groups is None else int(groups), 1e-5,
                          bool(g["length_last"]))
    (y * g["dy"].cuda()).sum().backward()
    for t, k in ((x, "dx"), (gamma, "dgamma"), (beta, "dbeta")):
        assert rel_l2(t.grad, g[k]) < 1e-4, k


def test_reference_attention_wrappers_on_this_library():
    """The reference's AttentionSoftmax and EfficientAttention modules on the shim against a plain
    float64 evaluation of causal softmax attention, forward and backward."""
    _, _, asm, eff = _wrappers()
    gen = torch.Generator().manual_seed(3)
    bsz, length, zdim, vdim = 3, 48, 16, 40
    q, k, v = [torch.randn(bsz, length, d, generator=gen).cuda().requires_grad_(True) for d in (zdim, zdim, vdim)]
    att = eff.EfficientAttention(scale=0.25, dropout=0.0, use_causal_mask=True).eval()
    y = att(q, k, v)
    dy = torch.randn(bsz, length, vdim, generator=gen).cuda()
    (y * dy).sum().backward()
    qd, kd, vd = [t.detach().double().requires_grad_(True) for t in (q, k, v)]
    s = torch.bmm(qd, kd.transpose(1, 2)) * 0.25
    s = s.masked_fill(torch.triu(torch.ones(length, length, device="cuda", dtype=torch.bool), 1), float("-inf"))
    ref = torch.bmm(torch.softmax(s, -1), vd)
    (ref * dy.double()).sum().backward()
    assert rel_l2(y, ref) < 1e-5
    for a, b in ((q, qd), (k, kd), (v, vd)):
        assert rel_l2(a.grad, b.grad) < 1e-4
    sm = asm.AttentionSoftmax(dropout=0.0, use_causal_mask=True).eval()
    x = torch.randn(4, 32, 32, generator=gen).cuda()
    w = sm(x)
    wref = torch.softmax(x.double().masked_fill(torch.triu(torch.ones(32, 32, device="cuda", dtype=torch.bool), 1),
                                                float("-inf")), -1)
    assert rel_l2(w, wref) < 1e-5


def test_ema_operator_names_explain_themselves():
    import fairseq_apollo_b200.mega2_ops as shim
    with pytest.raises(NotImplementedError, match="MultiHeadEMA"):
        shim.ema_parameters_fwd(None, None, None, None, 8)
