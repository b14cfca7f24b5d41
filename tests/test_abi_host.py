"""CPU: the C-ABI library loads, exports every symbol the header declares, and rejects bad
arguments with status codes before touching CUDA.  Also the host logic of the modules."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    import fairseq_apollo_b200 as M
    from fairseq_apollo_b200 import _lib
    if not os.path.exists(M.LIB_PATH):
        import __graft_entry__
        __graft_entry__.build()
    return _lib.lib(), _lib


def test_header_symbols_exported():
    lib, mod = _lib()
    hdr = open(os.path.join(ROOT, "include", "mega_b200.h")).read()
    names = set(re.findall(r"MEGA_API[^;(]*?\b(mega_\w+)\s*\(", hdr))
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    assert names == set(mod.SIGNATURES) | set(mod.OTHER)
    assert lib.mega_abi_version() == 1
    assert lib.mega_status_string(0) == b"ok"


def test_argument_rejection_without_gpu():
    lib, _ = _lib()
    one = ctypes.c_void_p(16)
    # null pointers
    assert lib.mega_ema_fwd(None, None, 0, 1, 1, 1, 0, 0, 0, 0, 0, 0, None, None, None, None, 16, None, None, None, 0, 0, None) == 1
    # bad dtype
    assert lib.mega_ema_fwd(one, one, 9, 1, 1, 1, 1, 1, 1, 1, 1, 1, one, one, one, one, 16, None, None, None, 0, 0, None) == 2
    # bad shape
    assert lib.mega_ema_fwd(one, one, 0, 0, 1, 1, 1, 1, 1, 1, 1, 1, one, one, one, one, 16, None, None, None, 0, 0, None) == 3
    # ndim out of range
    assert lib.mega_ema_fwd(one, one, 0, 1, 1, 1, 1, 1, 1, 1, 1, 1, one, one, one, one, 33, None, None, None, 0, 0, None) == 6
    # misaligned activation pointer
    assert lib.mega_ema_fwd(ctypes.c_void_p(18), one, 0, 1, 1, 1, 1, 1, 1, 1, 1, 1, one, one, one, one, 16, None, None, None, 0, 0, None) == 5
    # state with bidirectional / truncation on a causal layer
    assert lib.mega_ema_fwd(one, one, 0, 1, 1, 8, 1, 1, 1, 1, 1, 1, one, one, one, one, 16, None, one, None, 1, 0, None) == 7
    assert lib.mega_ema_fwd(one, one, 0, 1, 1, 8, 1, 1, 1, 1, 1, 1, one, one, one, one, 16, None, None, None, 0, 4, None) == 7
    # groups must divide features
    two = ctypes.c_void_p(32)
    assert lib.mega_timestep_norm_fwd(one, one, 0, 1, 1, 10, 1, 1, 1, 1, 1, 1, one, one, one, one, one, None, 3, 1e-5, two, one, one, None) == 3
    # the new counts must not be written over the incoming ones (every thread block of a sequence reads them)
    assert lib.mega_timestep_norm_fwd(one, one, 0, 1, 1, 8, 1, 1, 1, 1, 1, 1, one, one, one, one, one, None, 8, 1e-5, one, one, one, None) == 7
    assert lib.mega_tsn_ema_fwd(one, one, None, 1, 8, 64, 8, 1, 1, 1, 1, 1, 1, one, one, one, one, one, 1e-5, one, one, one,
                                one, one, one, one, 16, None, None, None, 0, None) == 7
    assert lib.mega_sequence_norm_fwd(one, one, 0, 1, 10, 1, 1, 1, 1, 1, 1, 1, one, one, None, 3, 1e-5, one, one, one, None) == 3
    assert lib.mega_ema_step(one, one, 0, 1, 1, one, one, one, one, 16, None, None, 0, None) == 1


def test_argument_rejection_training_and_complex_entry_points():
    lib, _ = _lib()
    one = ctypes.c_void_p(16)
    st9 = [1] * 9
    # mega_ema_bwd: null, SiLU flag, truncation, state with bidirectional, ndim
    ema = lambda dy, N, flags, trunc, h: lib.mega_ema_bwd(dy, one, one, 0, 1, 1, 8, *st9, one, one, one, one, N, None, h,
                                                          None, flags, trunc, one, one, one, one, None, None)
    assert ema(None, 16, 0, 0, None) == 1
    assert ema(one, 16, 4, 0, None) == 7
    assert ema(one, 16, 0, 3, None) == 7
    assert ema(one, 16, 1, 0, one) == 7
    assert ema(one, 40, 0, 0, None) == 6
    # mega_timestep_norm_bwd: grouped form needs group_mean; groups must divide features; group size cap
    tsn = lambda D, G, gm: lib.mega_timestep_norm_bwd(one, one, one, 0, 1, 1, D, *st9, None, None, one, one, one, one, gm,
                                                      one, None, G, one, one, one, one, None)
    assert tsn(12, 3, None) == 1
    assert tsn(10, 3, one) == 3
    assert tsn(1024, 2, one) == 7
    # mega_timestep_norm_fwd_train: the saves are required
    assert lib.mega_timestep_norm_fwd_train(one, one, 0, 1, 1, 8, 1, 1, 1, 1, 1, 1, one, one, one, one, one, None, 8,
                                            1e-5, one, one, one, None, None, None, None) == 1
    assert lib.mega_timestep_norm_fwd_train(one, one, 0, 1, 1, 8, 1, 1, 1, 1, 1, 1, one, one, one, one, one, None, 2,
                                            1e-5, one, one, one, one, one, None, None) == 1
    # mega_sequence_norm_bwd: groups must divide the channels
    assert lib.mega_sequence_norm_bwd(one, one, one, 0, 1, 8, 4, *st9, one, one, one, one, None, 3, one, one, None) == 3
    assert lib.mega_sequence_norm_bwd(one, one, one, 5, 1, 8, 4, *st9, one, one, one, one, None, 8, one, one, None) == 2
    # complex EMA: same envelope rules as the real layer
    cema = lambda x, N, flags, trunc, h: lib.mega_cema_fwd(x, one, 0, 1, 1, 8, 1, 1, 1, 1, 1, 1, one, one, one, one, N,
                                                           None, h, None, flags, trunc, None)
    assert cema(None, 16, 0, 0, None) == 1
    assert cema(one, 0, 0, 0, None) == 6
    assert cema(one, 16, 1, 0, one) == 7
    assert cema(one, 16, 0, 4, None) == 7
    assert lib.mega_cema_step(one, one, 0, 1, 1, one, one, one, one, 16, None, None, 0, None) == 1
    assert lib.mega_cema_coeffs(one, one, one, one, 7, 4, 16, one, one, one, None) == 2
    assert lib.mega_gate_qk(one, 4, one, one, one, 8, one, 8, 0, 2, 8, 1e-5, None) == 4  # pitch below the row length
    assert lib.mega_ema_coeffs_bwd(one, one, one, one, one, one, 0, 16, one, one, one, one, None) == 3
    # DropKey softmax: probability in [0, 1)
    assert lib.mega_attention_dropkey_softmax_fwd(one, one, 0, 1, 1, 8, 1, 1.0, 1, 0, None) == 7
    assert lib.mega_attention_dropkey_softmax_fwd(None, one, 0, 1, 1, 8, 1, 0.1, 1, 0, None) == 1


def test_ops_refuse_cpu_tensors():
    import fairseq_apollo_b200 as M
    m = M.MultiHeadEMA(4, ndim=16).eval()
    with torch.no_grad(), pytest.raises(RuntimeError, match="CUDA"):
        m(torch.randn(1, 4, 8))
    with pytest.raises(RuntimeError, match="CUDA"):  # the differentiable path has no CPU fallback either
        m(torch.randn(1, 4, 8))


def test_module_state_dict_contract():
    import fairseq_apollo_b200 as M
    from _util import golden
    e = M.MultiHeadEMA(8, ndim=16, bidirectional=True, truncation=5, shift=False)
    sd = e.state_dict()
    assert {k: tuple(v.shape) for k, v in sd.items()} == {
        "alpha": (16, 16, 1), "delta": (16, 16, 1), "beta": (16, 16, 1), "gamma": (16, 16), "omega": (8,)}
    assert [n for n, _ in e.parameters_no_weight_decay()] == ["alpha", "delta"]
    assert "bidirectional=True" in e.extra_repr()
    with pytest.raises(AssertionError):
        M.MultiHeadEMA(8, ndim=16, bidirectional=False, truncation=5)
    # beta alternates in sign along ndim
    b = e.beta.detach().squeeze(-1)
    assert (b[:, 0::2] > 0.8).all() and (b[:, 1::2] < -0.8).all()
    # TimestepNorm: keys, dtypes and the prior_count rules of the reference
    t = M.TimestepNorm(10, prior_count=2)
    g = golden("tsn_module")
    ref_keys = {k[3:]: torch.as_tensor(v) for k, v in g.items() if k.startswith("sd_")}
    assert set(t.state_dict()) == set(ref_keys)
    for k, v in t.state_dict().items():
        assert tuple(v.shape) == tuple(ref_keys[k].shape) and v.dtype == ref_keys[k].dtype
    with pytest.raises(AssertionError):
        M.TimestepNorm(10)  # per-feature statistics need prior_count > 1
    tg = M.TimestepNorm(12, num_groups=3)
    assert "prior_mean" in dict(tg.named_buffers()) and tg.prior_mean.shape == (3,)
    with pytest.raises(AssertionError):
        M.TimestepNorm(10, num_groups=3)
    s = M.SequenceNorm(6, num_groups=2)
    assert set(s.state_dict()) == {"weight", "bias"}
    with pytest.raises(AssertionError):
        M.SequenceNorm(7, num_groups=2)
