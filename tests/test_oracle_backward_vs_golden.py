"""Pins the oracle's gradients (torch autograd through the CPU restatement, float64) against
gradients produced by the reference itself: its CPU backward ops for TimestepNorm / SequenceNorm
and autograd through its EMA module (tests/golden/make_golden.py backward)."""
import pytest
import torch

from _util import golden, opt_mask, rel_l2
from oracle import mega_oracle as O


def _leaf(t):
    return t.double().clone().requires_grad_(True)


@pytest.mark.parametrize("name", ["ema_bwd_uni", "ema_bwd_uni_n3", "ema_bwd_bidir_shift", "ema_bwd_bidir_noshift",
                                  "ema_bwd_bidir_trunc", "ema_bwd_bidir_trunc_noshift"])
def test_ema_gradients(name):
    g = golden(name)
    x, alpha, delta, beta, gamma, omega = [_leaf(g[k]) for k in ("x", "alpha", "delta", "beta", "gamma", "omega")]
    y = O.ema_forward_recurrence(x, alpha, delta, beta, gamma, omega, opt_mask(g["mask"]),
                                 bidirectional=bool(g["bidirectional"]), shift=bool(g["shift"]),
                                 truncation=g.get("truncation"))
    assert rel_l2(y, g["y"]) < 2e-6
    (y * g["dy"].double()).sum().backward()
    for t, k in ((x, "dx"), (alpha, "dalpha"), (delta, "ddelta"), (beta, "dbeta"), (gamma, "dgamma"),
                 (omega, "domega")):
        assert rel_l2(t.grad, g[k]) < 2e-5, k


@pytest.mark.parametrize("name", ["tsn_bwd_plain", "tsn_bwd_plain_nomask", "tsn_bwd_group", "tsn_bwd_group_prior"])
def test_timestep_norm_gradients(name):
    g = golden(name)
    x, pm, pv, gamma, beta = [_leaf(g[k]) for k in ("x", "prev_mean", "prev_var", "gamma", "beta")]
    mask = opt_mask(g["mask"])
    if g["groups"] < 0:
        y, _, mean, var = O.timestep_norm(x, g["prev_count"], pm, pv, gamma, beta, mask, acc_dtype=torch.float64)
    else:
        y, _, mean, var = O.group_timestep_norm(x, g["prev_count"], pm, pv, gamma, beta, mask, g["groups"],
                                                acc_dtype=torch.float64)
    loss = (y * g["dy"].double()).sum() + (mean * g["dmean"].double()).sum() + (var * g["dvar"].double()).sum()
    loss.backward()
    for t, k in ((x, "dx"), (pm, "dprev_mean"), (pv, "dprev_var"), (gamma, "dgamma"), (beta, "dbeta")):
        assert rel_l2(t.grad, g[k]) < 2e-5, k


@pytest.mark.parametrize("name", ["sqn_bwd_bhl", "sqn_bwd_blh", "sqn_bwd_bhl_group", "sqn_bwd_blh_group"])
def test_sequence_norm_gradients(name):
    g = golden(name)
    x, gamma, beta = [_leaf(g[k]) for k in ("x", "gamma", "beta")]
    y = O.sequence_norm(x, gamma, beta, g["mask"].bool(), g.get("groups"), 1e-5, bool(g["length_last"]),
                        acc_dtype=torch.float64)[0]
    (y * g["dy"].double()).sum().backward()
    for t, k in ((x, "dx"), (gamma, "dgamma"), (beta, "dbeta")):
        assert rel_l2(t.grad, g[k]) < 2e-5, k


@pytest.mark.parametrize("name", ["cema_bwd_uni", "cema_bwd_uni_n3", "cema_bwd_bidir_shift", "cema_bwd_bidir_noshift",
                                  "cema_bwd_bidir_trunc", "cema_bwd_bidir_trunc_noshift"])
def test_complex_ema_gradients(name):
    g = golden(name)
    leaves = [_leaf(g[k]) for k in ("x", "alpha", "delta", "theta", "gamma", "omega")]
    y = O.cema_forward_recurrence(*leaves, opt_mask(g["mask"]), bidirectional=bool(g["bidirectional"]),
                                  shift=bool(g["shift"]), truncation=g.get("truncation"))
    assert rel_l2(y, g["y"]) < 2e-6
    (y * g["dy"].double()).sum().backward()
    for t, k in zip(leaves, ("dx", "dalpha", "ddelta", "dtheta", "dgamma", "domega")):
        assert rel_l2(t.grad, g[k]) < 2e-5, k
