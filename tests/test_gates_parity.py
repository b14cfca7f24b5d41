"""GPU parity of the Mega gate elementwise ops against the oracle's restatement of
fairseq/modules/moving_average_gated_attention.py:319-330,407-412.  The inputs are column slices
of one wide projection output, as in the reference's torch.split of mx_proj's result."""
import pytest
import torch

from _util import rel_l2

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2}


def _mods():
    import fairseq_apollo_b200 as M
    from oracle import mega_oracle as O
    return M, O


def _block(gen, bsz, length, embed, zdim, hdim, dtype):
    base = (torch.randn(bsz, length, 2 * embed + zdim + hdim, generator=gen) * 1.3).to(dtype)
    z_gamma = torch.randn(2, zdim, generator=gen) * 0.3
    z_beta = torch.randn(2, zdim, generator=gen) * 0.3
    return base, z_gamma, z_beta


@pytest.mark.parametrize("bsz,length,embed,zdim,hdim", [(1, 1, 8, 4, 8), (2, 37, 64, 33, 96), (3, 128, 256, 64, 512)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_split(bsz, length, embed, zdim, hdim, dtype):
    M, O = _mods()
    gen = torch.Generator().manual_seed(embed + zdim)
    base, zg, zb = _block(gen, bsz, length, embed, zdim, hdim, dtype)
    u_ref, q_ref, k_ref, r_ref, hx_ref = O.mega_gate_split(base.float(), zdim, hdim, embed, zg, zb)
    dev = base.cuda()
    u, z, r, hx = torch.split(dev, [embed, zdim, hdim, embed], dim=-1)
    q, k = M.ops.gate_qk(z, zg.cuda(), zb.cuda(), 1e-5)
    assert q.shape == z.shape and k.shape == z.shape
    assert rel_l2(q.float(), q_ref) < TOL[dtype]
    assert rel_l2(k.float(), k_ref) < TOL[dtype]
    rs = M.ops.gate_silu(r)
    assert rel_l2(rs.float(), r_ref) < TOL[dtype]
    # attn * silu(r): any tensor of r's shape stands in for the attention output
    attn = (torch.randn(bsz, length, hdim, generator=gen)).to(dtype)
    ar = M.ops.gate_mul_silu(attn.cuda(), r)
    assert rel_l2(ar.float(), attn.float() * r_ref) < TOL[dtype]


@pytest.mark.parametrize("bsz,length,embed", [(1, 1, 5), (2, 50, 96), (4, 64, 1024)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_output(bsz, length, embed, dtype):
    M, O = _mods()
    gen = torch.Generator().manual_seed(embed)
    base = torch.randn(bsz, length, 2 * embed + 7, generator=gen).to(dtype)
    residual = torch.randn(bsz, length, embed, generator=gen).to(dtype)
    h_lin = torch.randn(bsz, length, embed, generator=gen).to(dtype)
    u_pre, _, hx = torch.split(base, [embed, 7, embed], dim=-1)
    ref = O.mega_gate_output(residual.float(), torch.sigmoid(u_pre.float()), hx.float(), h_lin.float())
    dev = base.cuda()
    u_d, _, hx_d = torch.split(dev, [embed, 7, embed], dim=-1)
    out = M.ops.gate_output(residual.cuda(), u_d, hx_d, h_lin.cuda())
    assert rel_l2(out.float(), ref) < TOL[dtype]
    # silu(a + b)
    s = M.ops.gate_silu(hx_d, h_lin.cuda())
    assert rel_l2(s.float(), torch.nn.functional.silu(hx.float() + h_lin.float())) < TOL[dtype]


def test_gate_qk_zero_row():
    """A zero row divides by eps, not by zero: outputs are exactly beta."""
    M, _ = _mods()
    z = torch.zeros(3, 16, device="cuda")
    g = torch.full((2, 16), 0.5, device="cuda")
    b = torch.arange(32, dtype=torch.float32, device="cuda").view(2, 16)
    q, k = M.ops.gate_qk(z, g, b)
    assert torch.equal(q, b[0].expand(3, 16)) and torch.equal(k, b[1].expand(3, 16))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_qk_rotary(dtype):
    """gate_qk with the rotary embedding in the same kernel against gate_qk's definition followed by the
    complex multiplication the reference's RotaryEmbedding performs, on a column slice, with chunks of 16
    positions and a query offset."""
    import fairseq_apollo_b200 as M
    gen = torch.Generator().manual_seed(11)
    bsz, length, S, period = 3, 48, 64, 16
    base = torch.randn(bsz, length, S + 40, generator=gen).to(dtype).cuda()
    z = base[..., 8:8 + S]
    gamma = (torch.randn(2, S, generator=gen) * 0.2).cuda()
    beta = (torch.randn(2, S, generator=gen) * 0.2).cuda()
    t = torch.arange(40, dtype=torch.float32)
    freqs = 1.0 / torch.tensor([10000 ** (j / S) for j in range(0, S, 2)], dtype=torch.float32)
    ang = torch.outer(t, freqs)
    table = torch.polar(torch.ones_like(ang), ang).cuda()
    for q_offset in (0, 5):
        q, k = M.ops.gate_qk_rotary(z, gamma, beta, table, period, q_offset)
        zn = torch.nn.functional.normalize(z.float(), p=2, dim=-1, eps=1e-5)
        q0 = zn * (gamma[0] + 1) + beta[0]
        k0 = zn * (gamma[1] + 1) + beta[1]
        pos = torch.arange(length, device="cuda") % period

        def rot(x, p):
            xc = torch.view_as_complex(x.reshape(bsz, length, S // 2, 2).contiguous())
            return torch.view_as_real(xc * table[p]).flatten(2)
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert rel_l2(q.float(), rot(q0, pos + q_offset)) < tol
        assert rel_l2(k.float(), rot(k0, pos)) < tol
