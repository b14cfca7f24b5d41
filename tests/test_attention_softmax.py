"""GPU parity of the attention-weight softmax (forward and backward) against the oracle, and —
when the reference's CUDA operators are built — against the reference's own kernel."""
import pytest
import torch

from _util import rel_l2

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2}


def _mods():
    import fairseq_apollo_b200 as M
    from oracle import mega_oracle as O
    return M, O


@pytest.mark.parametrize("batch,outer,inner", [(1, 1, 1), (3, 5, 5), (2, 33, 70), (4, 128, 128), (2, 1, 1024),
                                                (2, 64, 1024), (1, 3, 4100), (1, 2, 8192)])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_forward_backward(batch, outer, inner, causal, dtype):
    M, O = _mods()
    if causal and outer > inner:
        pytest.skip("more query rows than keys")
    gen = torch.Generator().manual_seed(outer * 7 + inner)
    x = (torch.randn(batch, outer, inner, generator=gen) * 3).to(dtype)
    if inner > 4:
        x[0, 0, :2] = float("-inf")           # padded keys
    if not causal and outer > 1:
        x[-1, -1, :] = float("-inf")          # a fully masked row gives zeros, not NaN
    dy = torch.randn(batch, outer, inner, generator=gen).to(dtype)
    xr = x.double().clone().requires_grad_(True)
    yr = O.attention_softmax(xr, causal)
    (yr * dy.double()).sum().backward()
    xd = x.cuda().requires_grad_(True)
    mod = M.AttentionSoftmax(0.0, causal).cuda()
    y = mod(xd)
    assert torch.isfinite(y).all()
    assert rel_l2(y.float(), yr) < TOL[dtype]
    (y.float() * dy.cuda().float()).sum().backward()
    assert torch.isfinite(xd.grad).all()
    assert rel_l2(xd.grad.float(), torch.nan_to_num(xr.grad)) < (2e-5 if dtype == torch.float32 else 2e-2)
    if causal:  # masked scores get exactly zero weight and zero gradient
        cols = torch.arange(inner).view(1, inner)
        dead = cols >= (inner - outer + torch.arange(outer).view(outer, 1) + 1)
        assert (y.cpu()[:, dead] == 0).all() and (xd.grad.cpu()[:, dead] == 0).all()


def test_against_reference_cuda_kernel():
    from oracle.build_ref import load_ref_cuda
    ref = load_ref_cuda()
    if ref is None:
        pytest.skip("oracle/_ref/mega_ref_cuda.so not built")
    M, _ = _mods()
    gen = torch.Generator().manual_seed(3)
    for dtype in (torch.float32, torch.bfloat16):
        for causal in (True, False):
            x = (torch.randn(6, 1024, 1024, generator=gen) * 2).to(dtype).cuda()
            dy = torch.randn(6, 1024, 1024, generator=gen).to(dtype).cuda()
            ry = ref.ops.attention_softmax_fwd(x, 0.0, causal)
            rdx = ref.ops.attention_softmax_bwd(dy, ry, causal)
            y = M.ops.attention_softmax_fwd(x, causal)
            dx = M.ops.attention_softmax_bwd(dy, y, causal)
            assert rel_l2(y.float(), ry.float()) < TOL[dtype]
            assert rel_l2(dx.float(), rdx.float()) < (2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("batch,outer,inner", [(3, 5, 5), (2, 33, 70), (2, 64, 1024), (1, 3, 4100), (2, 16, 2048)])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dropkey_forward_backward(batch, outer, inner, causal, dtype):
    """DropKey: the dropped columns are exactly those of the oracle's restatement of the mask
    (Philox4x32-10 keyed by seed, offset, row, column), the kept ones are the softmax of the
    remaining scores, and the backward is the softmax backward on that result."""
    M, O = _mods()
    if causal and outer > inner:
        pytest.skip("more query rows than keys")
    gen = torch.Generator().manual_seed(outer * 11 + inner)
    x = (torch.randn(batch, outer, inner, generator=gen) * 3).to(dtype)
    dy = torch.randn(batch, outer, inner, generator=gen).to(dtype)
    dropout, seed, offset = 0.3, 0x1234567887654321, 5
    xr = x.double().clone().requires_grad_(True)
    yr = O.attention_dropkey_softmax(xr, dropout, causal, seed, offset)
    (yr * dy.double()).sum().backward()
    y = M.ops.attention_dropkey_softmax_fwd(x.cuda(), dropout, causal, seed, offset)
    assert torch.equal(y.cpu() == 0, yr == 0)          # the same columns are dropped (or masked)
    assert rel_l2(y.float(), yr) < TOL[dtype]
    dx = M.ops.attention_softmax_bwd(dy.cuda(), y, causal)
    assert rel_l2(dx.float(), torch.nan_to_num(xr.grad)) < (2e-5 if dtype == torch.float32 else 2e-2)
    drop = O.dropkey_mask(batch * outer, inner, dropout, seed, offset)
    if drop.numel() > 10000:
        assert abs(drop.float().mean().item() - dropout) < 0.02
    # another offset gives another mask; dropout 0 is the plain softmax
    if inner >= 64:
        y2 = M.ops.attention_dropkey_softmax_fwd(x.cuda(), dropout, causal, seed, offset + 1)
        assert not torch.equal(y2 == 0, y == 0)
    y0 = M.ops.attention_dropkey_softmax_fwd(x.cuda(), 0.0, causal, seed, offset)
    assert torch.equal(y0, M.ops.attention_softmax_fwd(x.cuda(), causal))


def test_dropkey_module():
    """Training mode draws a fresh mask per call from torch's CPU generator (repeatable under
    manual_seed); evaluation mode applies no dropout; rows always sum to 1 (or 0)."""
    M, _ = _mods()
    mod = M.AttentionSoftmax(0.25, True).cuda()
    x = torch.randn(2, 128, 128, device="cuda", requires_grad=True)
    torch.manual_seed(7)
    a = mod(x)
    b = mod(x)
    torch.manual_seed(7)
    c = mod(x)
    assert torch.equal(a, c) and not torch.equal(a, b)
    sums = a.sum(-1)
    assert torch.all(((sums - 1).abs() < 1e-5) | (sums == 0))
    frac = 1.0 - (a[:, -1, :] > 0).float().mean().item()   # the last row keeps every column
    assert abs(frac - 0.25) < 0.1
    a.sum().backward()
    assert torch.isfinite(x.grad).all()
    mod.eval()
    assert torch.equal(mod(x), M.ops.attention_softmax_fwd(x.detach(), True))


@pytest.mark.parametrize("bsz,length,heads,h1,h2", [(2, 64, 1, 32, 48), (1, 256, 2, 16, 64), (2, 33, 3, 8, 8)])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_efficient_attention(bsz, length, heads, h1, h2, causal, dtype):
    """attention(q, k, v, scale, dropout, causal, training) against float64 autograd through
    softmax(scale q k^T + mask) v; q, k (B, L, N, H1), v (B, L, N, H2) as the reference operator takes them."""
    M, O = _mods()
    from fairseq_apollo_b200.modules.efficient_attention import attention
    gen = torch.Generator().manual_seed(length + h2)
    q, k = [torch.randn(bsz, length, heads, h1, generator=gen).to(dtype) for _ in range(2)]
    v = torch.randn(bsz, length, heads, h2, generator=gen).to(dtype)
    dy = torch.randn(bsz, length, heads, h2, generator=gen).to(dtype)
    scale = h1 ** -0.5
    ref = [t.double().clone().requires_grad_(True) for t in (q, k, v)]
    s = torch.einsum("blnh,bmnh->bnlm", ref[0], ref[1]) * scale
    yr = torch.einsum("bnlm,bmnh->blnh", O.attention_softmax(s, causal), ref[2])
    (yr * dy.double()).sum().backward()
    dev = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    y = attention(*dev, scale, 0.0, causal, True)
    assert y.shape == (bsz, length, heads, h2)
    (y.float() * dy.cuda().float()).sum().backward()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert rel_l2(y.float(), yr) < tol
    for a, r in zip(dev, ref):
        assert rel_l2(a.grad.float(), r.grad) < (1e-4 if dtype == torch.float32 else 3e-2)
    if heads == 1:
        mod = M.EfficientAttention(scale, 0.0, causal).cuda()
        y1 = mod(dev[0].detach()[:, :, 0], dev[1].detach()[:, :, 0], dev[2].detach()[:, :, 0])
        assert rel_l2(y1.float(), yr[:, :, 0]) < tol
    # DropKey in training mode: rows of the weights still sum to one, result finite and different
    torch.manual_seed(1)
    yd = attention(*[t.detach() for t in dev], scale, 0.5, causal, True)
    assert torch.isfinite(yd).all() and not torch.equal(yd, y.detach())
    assert torch.equal(attention(*[t.detach() for t in dev], scale, 0.5, causal, False), y.detach())


def test_efficient_attention_against_reference_cuda_op():
    from oracle.build_ref import load_ref_cuda
    ref = load_ref_cuda()
    if ref is None:
        pytest.skip("oracle/_ref/mega_ref_cuda.so not built")
    from fairseq_apollo_b200.modules.efficient_attention import attention
    gen = torch.Generator().manual_seed(11)
    for dtype in (torch.float32, torch.bfloat16):
        q, k = [torch.randn(2, 512, 1, 64, generator=gen).to(dtype).cuda() for _ in range(2)]
        v = torch.randn(2, 512, 1, 128, generator=gen).to(dtype).cuda()
        dy = torch.randn(2, 512, 1, 128, generator=gen).to(dtype).cuda()
        ry, rw = ref.ops.attention_fwd(q, k, v, 0.125, 0.0, True)
        rq, rk, rv = ref.ops.attention_bwd(dy, q, k, v, rw, 0.125, True)
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
        y = attention(*leaves, 0.125, 0.0, True, True)
        y.backward(dy)
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert rel_l2(y.float(), ry.float()) < tol
        for a, r in zip(leaves, (rq, rk, rv)):
            assert rel_l2(a.grad.float(), r.float()) < (1e-4 if dtype == torch.float32 else 3e-2)
