"""CPU: the oracle restatement against outputs of the reference itself
(tests/golden/*.npz, produced by tests/golden/make_golden.py)."""
import pytest
import torch

from oracle import mega_oracle as O
from _util import golden, opt_mask, rel_l2

EMA_CASES = ["ema_uni_n16", "ema_uni_n2", "ema_uni_pow2", "ema_bidir_shift", "ema_bidir_noshift", "ema_bidir_trunc"]


@pytest.mark.parametrize("name", EMA_CASES)
def test_ema_fft_restatement(name):
    g = golden(name)
    trunc = None if g["truncation"] < 0 else g["truncation"]
    y = O.ema_forward_fft(g["x"], g["alpha"], g["delta"], g["beta"], g["gamma"], g["omega"],
                          opt_mask(g["mask"]), bool(g["bidirectional"]), bool(g["shift"]), trunc)
    assert rel_l2(y, g["y"]) < 2e-6


@pytest.mark.parametrize("name", EMA_CASES)
def test_ema_recurrence_ground_truth(name):
    g = golden(name)
    trunc = None if g["truncation"] < 0 else g["truncation"]
    y = O.ema_forward_recurrence(g["x"], g["alpha"], g["delta"], g["beta"], g["gamma"], g["omega"],
                                 opt_mask(g["mask"]), bool(g["bidirectional"]), bool(g["shift"]), trunc)
    assert rel_l2(y, g["y"]) < 2e-6


def test_ema_incremental_ops():
    g = golden("ema_incremental")
    assert g["imag_max"] < 1e-6
    p, q, gam = O.ema_coeffs(g["alpha"], g["delta"], g["beta"], g["gamma"])
    chunk = g["chunk"]
    x = g["x"]
    h = None
    ys = []
    for i, c in enumerate(range(0, x.shape[-1], chunk)):
        xc = x[..., c:c + chunk]
        y, h = O.ema_forward_fft(xc, g["alpha"], g["delta"], g["beta"], g["gamma"], g["omega"], h=h, return_state=True)
        ys.append(y)
        # the reference's complex class keeps p = sigmoid(alpha) in the state and folds beta into
        # gamma; the real class keeps p = sigmoid(alpha) * beta.  Compare in the real convention.
        beta = g["beta"].squeeze(-1)
        assert rel_l2(h, g["states"][i] * beta) < 2e-6
    assert rel_l2(torch.cat(ys, -1), g["y"]) < 2e-6
    # recurrence ground truth agrees with the chunked reference ops as well
    y64, h64 = O.ema_forward_recurrence(x, g["alpha"], g["delta"], g["beta"], g["gamma"], g["omega"], return_state=True)
    assert rel_l2(y64, g["y"]) < 2e-6
    assert rel_l2(h64, g["states"][-1] * g["beta"].squeeze(-1)) < 2e-6
    # closed-form single step (base_moving_average.one_step)
    y1, h1 = O.ema_one_step(x[..., 0], p, q, gam, None)
    assert rel_l2(y1, g["step_y1"].squeeze(-1)) < 2e-6
    y2, h2 = O.ema_one_step(x[..., 1], p, q, gam, h1)
    assert rel_l2(y2, g["step_y2"].squeeze(-1)) < 2e-6
    assert rel_l2(h2, g["step_h2"] * g["beta"].squeeze(-1)) < 2e-6


@pytest.mark.parametrize("name", ["tsn_plain", "tsn_plain_nomask", "tsn_group2", "tsn_group_prior"])
def test_timestep_norm(name):
    g = golden(name)
    mask = opt_mask(g["mask"])
    if g["groups"] < 0:
        y, cnt, mean, var = O.timestep_norm(g["x"], g["prev_count"], g["prev_mean"], g["prev_var"], g["gamma"], g["beta"], mask)
    else:
        y, cnt, mean, var = O.group_timestep_norm(g["x"], g["prev_count"], g["prev_mean"], g["prev_var"], g["gamma"],
                                                  g["beta"], mask, g["groups"])
    assert torch.equal(cnt, g["count"])
    assert rel_l2(y, g["y"]) < 2e-6
    assert rel_l2(mean, g["mean"]) < 2e-6 and rel_l2(var, g["var"]) < 2e-6
    if mask is not None:
        assert (y[mask] == 0).all() and (g["y"][mask] == 0).all()


@pytest.mark.parametrize("name", ["sqn_bhl", "sqn_blh", "sqn_bhl_group", "sqn_blh_group"])
def test_sequence_norm(name):
    g = golden(name)
    mask = opt_mask(g["mask"])
    groups = None if g["groups"] < 0 else g["groups"]
    y, cnt, mean, rstd = O.sequence_norm(g["x"], g["gamma"], g["beta"], mask, groups, 1e-5, bool(g["length_last"]))
    assert torch.equal(cnt, g["count"])
    assert rel_l2(y, g["y"]) < 2e-6
    assert rel_l2(mean, g["mean"]) < 2e-6 and rel_l2(rstd, g["rstd"]) < 2e-6


def test_fft_path_vs_recurrence_long():
    """The reference's FFT formulation and the plain recurrence agree at a longer length."""
    gen = torch.Generator().manual_seed(7)
    from _util import make_ema_params
    prm = make_ema_params(gen, 16, 16)
    x = torch.randn(2, 16, 1000, generator=gen)
    a = O.ema_forward_fft(x, *prm)
    b = O.ema_forward_recurrence(x, *prm)
    assert rel_l2(a, b) < 2e-6


def test_philox_known_answers():
    """Philox4x32-10 known-answer vectors published with the generator (Random123 kat_vectors):
    the DropKey mask of the attention softmax is built on it."""
    from oracle import mega_oracle as O
    ones = 0xFFFFFFFF
    assert [int(v) for v in O.philox4x32_10(0, 0, 0, 0, 0, 0)] == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert [int(v) for v in O.philox4x32_10(ones, ones, ones, ones, ones, ones)] == [0x408f276d, 0x41c83b0e,
                                                                                      0xa20bc7c6, 0x6d5451fd]
    assert [int(v) for v in O.philox4x32_10(0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344, 0xa4093822,
                                            0x299f31d0)] == [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    m = O.dropkey_mask(64, 1000, 0.3, 99, 1)
    assert m.shape == (64, 1000) and abs(m.float().mean().item() - 0.3) < 0.01
