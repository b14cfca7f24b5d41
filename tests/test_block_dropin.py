"""Drop-in acceptance at the level of the Mega block.

The reference's own, unmodified ``MovingAverageGatedAttention`` (staged from the reference checkout
into oracle/_ref/py by ``oracle/build_ref.py``; test infrastructure) is imported with this package's
classes standing in for its EMA / norm / attention imports, loaded with the state dict of a block
that the reference built from its own modules, and run on the GPU.  The expected outputs come from
the reference running on CPU on top of its own modules and operators (tests/golden/make_golden.py
block).  This checks what a maintainer does when swapping the imports: constructor arguments,
state-dict keys and shapes, the (B, D, L) transposed views the block hands to the EMA, half-precision
parameters as the trainer casts them, and the incremental-state plumbing.
"""
import pytest
import torch

from _util import golden, rel_l2

pytestmark = pytest.mark.gpu


def _block_module():
    import fairseq_apollo_b200 as M
    from oracle import build_ref
    swap = {"MultiHeadEMA": M.MultiHeadEMA, "MultiHeadComplexEMA": M.MultiHeadComplexEMA,
            "TimestepNorm": M.TimestepNorm, "SequenceNorm": M.SequenceNorm,
            "EfficientAttention": M.EfficientAttention, "AttentionSoftmax": M.AttentionSoftmax}
    mod = build_ref.load_reference_block(swap)
    if mod is None:
        pytest.skip("oracle/_ref/py is not staged (python oracle/build_ref.py needs the reference checkout)")
    return M, mod


def _build(mod, g, **kw):
    dim, zdim, hdim, ndim, chunk, groups = [int(v) for v in g["dims"]]
    args = dict(chunk_size=chunk, moving_layer='cema', moving_act='silu', norm_num_groups=groups,
                rel_pos_bias='rotary', efficient_attn=False)
    args.update(kw)
    blk = mod.MovingAverageGatedAttention(dim, zdim, hdim, ndim, **args).eval()
    blk.load_state_dict(_state_dict(g), strict=True)
    return blk, chunk


def _state_dict(g):
    # (the fixture loader returns 0-d arrays, e.g. prior_count, as Python scalars)
    return {k[3:]: torch.as_tensor(v) for k, v in g.items() if k.startswith("sd.")}


def _causal_mask(chunk, device, dtype):
    causal = torch.tril(torch.ones(chunk, chunk, device=device))
    return torch.zeros(chunk, chunk, device=device, dtype=dtype).masked_fill(causal == 0, float("-inf"))


@pytest.mark.parametrize("name", ["mega_block_causal", "mega_block_causal_padded"])
def test_reference_block_runs_on_these_modules_fp32(name):
    """fp32: the block on this package's modules reproduces the reference block's output (through
    three GEMMs, the attention softmax and the gates) to 1e-4; the state dict loads with strict keys."""
    M, mod = _block_module()
    from fairseq_apollo_b200 import _lib
    g = golden(name)
    blk, chunk = _build(mod, g)
    assert isinstance(blk.move, M.MultiHeadComplexEMA) and isinstance(blk.norm, M.TimestepNorm)
    blk = blk.cuda()
    x = g["x"].cuda()
    mask = g["mask"].bool().cuda() if g["mask"].numel() else None
    before = M.launch_count()
    with torch.no_grad():
        y, _ = blk(x, padding_mask=mask, attn_mask=_causal_mask(chunk, x.device, x.dtype))
    assert M.launch_count() > before          # this library's kernels ran
    if mask is not None:   # the reference leaves garbage-free but unspecified values at padded rows
        keep = ~mask
        assert rel_l2(y[keep], g["y"].cuda()[keep]) < 1e-4
    else:
        assert rel_l2(y, g["y"]) < 1e-4
    assert _lib.device_error() == 0


def test_reference_block_efficient_attention_and_bf16():
    """The block's efficient_attn=True branch (EfficientAttention, this package's fused causal
    attention path) gives the same result as its softmax branch with an explicit causal mask; the whole
    block cast to bf16 (parameters included, as the trainer casts a model) stays within 2e-2."""
    M, mod = _block_module()
    g = golden("mega_block_causal")
    blk_e, chunk = _build(mod, g, efficient_attn=True)
    blk_e = blk_e.cuda()
    x = g["x"].cuda()
    with torch.no_grad():
        y_e, _ = blk_e(x)
    assert rel_l2(y_e, g["y"]) < 1e-4
    blk_h = _build(mod, g, efficient_attn=True)[0].cuda().bfloat16()
    assert blk_h.move.alpha.dtype == torch.bfloat16 and blk_h.norm.weight.dtype == torch.bfloat16
    with torch.no_grad():
        y_h, _ = blk_h(x.bfloat16())
    assert y_h.dtype == torch.bfloat16
    assert rel_l2(y_h.float(), g["y"]) < 2e-2


def test_reference_block_incremental_chunks():
    """Chunk-by-chunk decoding through the block's incremental_state (one chunk of 32 positions per
    call, then single tokens): the modules' buffers live under the reference's key names and the
    outputs equal the full-length call."""
    M, mod = _block_module()
    g = golden("mega_block_causal")
    blk, chunk = _build(mod, g, efficient_attn=True)
    blk = blk.cuda()
    x = g["x"].cuda()
    with torch.no_grad():
        full, _ = blk(x)
        st = {}
        outs = [blk(x[:, i:i + chunk], incremental_state=st)[0] for i in range(0, 2 * chunk, chunk)]
        # then token by token through the third chunk
        outs += [blk(x[:, i:i + 1], incremental_state=st)[0] for i in range(2 * chunk, x.size(1))]
    assert rel_l2(torch.cat(outs, 1), full) < 1e-4
    keys = sorted(k.split(".")[-1] for k in st)
    assert keys == ["attn_state", "ema_state", "norm_state"], keys
    norm_state = [v for k, v in st.items() if k.endswith("norm_state")][0]
    assert sorted(norm_state) == ["prev_count", "prev_mean", "prev_var"]
    ema_state = [v for k, v in st.items() if k.endswith("ema_state")][0]
    assert list(ema_state) == ["prev_state"] and ema_state["prev_state"].shape == (x.size(0), x.size(2), 16)
    assert bool((norm_state["prev_count"] == x.size(1)).all())


def test_reference_nffn_on_gpu():
    """The layer's second half (NormalizedFeedForwardNetwork: layer norm, SiLU MLP, residual) is
    caller-side code that needs nothing from this library; it is run here from the staged reference
    source so that a whole Mega layer = block + NFFN is covered by reference outputs."""
    M, mod = _block_module()
    import sys
    nffn = sys.modules["fairseq.modules.normalized_feedforward_network"]
    g = golden("mega_nffn")
    ff = nffn.NormalizedFeedForwardNetwork(64, 96, norm_type='layernorm').eval()
    ff.load_state_dict(_state_dict(g), strict=True)
    with torch.no_grad():
        y = ff.cuda()(g["x"].cuda())
    assert rel_l2(y, g["y"]) < 1e-5


def _own_block(g, **kw):
    """This package's own block class, built with the fixture's arguments and loaded (strict) with the state
    dict of the block the reference built."""
    import fairseq_apollo_b200 as M
    dim, zdim, hdim, ndim, chunk, groups = [int(v) for v in g["dims"]]
    args = dict(chunk_size=chunk, moving_layer='cema', moving_act='silu', norm_num_groups=groups,
                rel_pos_bias='rotary', efficient_attn=False)
    args.update(kw)
    blk = M.MovingAverageGatedAttention(dim, zdim, hdim, ndim, **args).eval()
    blk.load_state_dict(_state_dict(g), strict=True)
    return blk.cuda(), chunk


@pytest.mark.parametrize("efficient", [False, True])
def test_own_block_class_matches_reference_outputs(efficient):
    """The package's MovingAverageGatedAttention (fused norm -> EMA -> SiLU, gates, and for the efficient
    branch the rotary embedding inside the query / key kernel) against the outputs of the reference block
    on CPU: fp32 to 1e-4, the block cast to bf16 to 2e-2; token-by-token continuation equals the full call."""
    M, _ = _block_module()   # (skips when the reference sources are not staged, like the tests above)
    g = golden("mega_block_causal")
    blk, chunk = _own_block(g, efficient_attn=efficient)
    x = g["x"].cuda()
    with torch.no_grad():
        if efficient:
            y, _ = blk(x)
        else:
            y, _ = blk(x, attn_mask=_causal_mask(chunk, x.device, x.dtype))
    assert rel_l2(y, g["y"]) < 1e-4
    blk_h = _own_block(g, efficient_attn=True)[0].bfloat16()
    with torch.no_grad():
        y_h, _ = blk_h(x.bfloat16())
    assert rel_l2(y_h.float(), g["y"]) < 2e-2
    if efficient:
        with torch.no_grad():
            st = {}
            outs = [blk(x[:, i:i + chunk], incremental_state=st)[0] for i in range(0, 2 * chunk, chunk)]
            outs += [blk(x[:, i:i + 1].contiguous(), incremental_state=st)[0] for i in range(2 * chunk, x.size(1))]
        assert rel_l2(torch.cat(outs, 1), y) < 1e-4


def test_own_block_class_with_padding():
    M, _ = _block_module()
    g = golden("mega_block_causal_padded")
    blk, chunk = _own_block(g)
    x, mask = g["x"].cuda(), g["mask"].bool().cuda()
    with torch.no_grad():
        y, _ = blk(x, padding_mask=mask, attn_mask=_causal_mask(chunk, x.device, x.dtype))
    keep = ~mask
    assert rel_l2(y[keep], g["y"].cuda()[keep]) < 1e-4
