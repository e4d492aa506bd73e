"""Fused edge geometry (vectors + Bessel x polynomial-cutoff basis, and the position gradient) against the
torch expressions the models otherwise use."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-12), (torch.float32, 2e-6)])
def test_edge_geometry_matches_torch(dtype, tol):
    from fasteq_b200.graph import config1_batch
    from fasteq_b200.nn.mace_style import bessel_basis, polynomial_cutoff
    from fasteq_b200.ops.edge_geometry import edge_geometry
    b = config1_batch(2, seed=4)
    pos = torch.from_numpy(b.positions).cuda()
    src, dst = torch.from_numpy(b.edge_src).cuda(), torch.from_numpy(b.edge_dst).cuda()
    shift = torch.from_numpy(b.edge_shift).cuda()
    g = torch.Generator().manual_seed(0)
    E = src.numel()
    rv, rb = torch.randn(E, 3, generator=g, dtype=torch.float64).cuda(), torch.randn(E, 8, generator=g, dtype=torch.float64).cuda()
    # float64 torch reference
    p64 = pos.clone().requires_grad_(True)
    vec = p64[src] + shift - p64[dst]
    r = vec.norm(dim=-1)
    basis = bessel_basis(r, 5.0, 8) * polynomial_cutoff(r, 5.0, 5).unsqueeze(-1)
    (g_ref,) = torch.autograd.grad((vec * rv).sum() + (basis * rb).sum(), p64, retain_graph=True)
    pt = pos.to(dtype).requires_grad_(True)
    v2, b2 = edge_geometry(pt, src, dst, shift.to(dtype), 5.0, 8, 5)
    (g2,) = torch.autograd.grad((v2 * rv.to(dtype)).sum() + (b2 * rb.to(dtype)).sum(), pt)
    rel = lambda a, ref: float((a.double() - ref).abs().max() / ref.abs().max())
    assert rel(v2, vec.detach()) <= tol and rel(b2, basis.detach()) <= tol * 4 and rel(g2, g_ref) <= tol * 8
    # only one of the two cotangents
    (g3,) = torch.autograd.grad((edge_geometry(pt, src.int(), dst.int(), shift.to(dtype), 5.0, 8, 5)[1] * rb.to(dtype)).sum(), pt)
    (g3_ref,) = torch.autograd.grad((basis * rb).sum(), p64)
    assert rel(g3, g3_ref) <= tol * 8
