"""Pins the oracle's complex-EMA restatement against outputs of the reference's own
MultiHeadComplexEMA module and CPU ops (tests/golden/make_golden.py cema)."""
import pytest
import torch

from _util import golden, opt_mask, rel_l2
from oracle import mega_oracle as O

NAMES = ["cema_uni_n16", "cema_uni_n3", "cema_bidir_shift", "cema_bidir_noshift", "cema_bidir_trunc"]


@pytest.mark.parametrize("name", NAMES)
def test_forward(name):
    g = golden(name)
    trunc = None if g["truncation"] < 0 else g["truncation"]
    y = O.cema_forward_recurrence(g["x"], g["alpha"], g["delta"], g["theta"], g["gamma"], g["omega"],
                                  opt_mask(g["mask"]), bool(g["bidirectional"]), bool(g["shift"]), trunc)
    assert rel_l2(y, g["y"]) < 2e-6


def test_incremental():
    g = golden("cema_incremental")
    args = [g[k] for k in ("alpha", "delta", "theta", "gamma", "omega")]
    chunk = g["chunk"]
    h, ys = None, []
    for i in range(0, g["x"].shape[-1], chunk):
        y, h = O.cema_forward_recurrence(g["x"][..., i:i + chunk], *args, h=h, return_state=True)
        ys.append(y)
        assert rel_l2(torch.view_as_real(h), g["states"][i // chunk]) < 2e-6
    assert rel_l2(torch.cat(ys, -1), g["y"]) < 2e-6
    assert rel_l2(torch.cat(ys, -1), g["y_full"]) < 2e-6
    # closed-form single steps (the reference's one_step omits the omega residual)
    zero = torch.zeros_like(g["omega"])
    y1, h1 = O.cema_forward_recurrence(g["x"][..., :1], *args[:4], zero, return_state=True)
    y2, h2 = O.cema_forward_recurrence(g["x"][..., 1:2], *args[:4], zero, h=h1, return_state=True)
    assert rel_l2(y1, g["step_y1"]) < 2e-6 and rel_l2(y2, g["step_y2"]) < 2e-6
    assert rel_l2(torch.view_as_real(h2), g["step_h2"]) < 2e-6
