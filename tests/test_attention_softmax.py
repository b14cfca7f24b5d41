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
