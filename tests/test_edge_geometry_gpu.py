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


def test_out_of_range_indices_are_skipped_and_reported():
    """An edge whose sender or receiver index lies outside the position array is not followed (no access through
    it), gets zero features and no gradient, and leaves code 2 in the status word; a coincident pair (r = 0) gets the
    finite limit of the basis and a finite (zero) radial gradient."""
    import math
    from fasteq_b200.ops.edge_geometry import edge_geometry, edge_geometry_device_status
    edge_geometry_device_status()                     # clear
    pos = torch.tensor([[0.0, 0.0, 0.0], [1.0, 0.5, 0.2], [0.3, 2.0, 1.0]], device="cuda", requires_grad=True)
    src = torch.tensor([1, 7, 2, -1, 0], dtype=torch.int32, device="cuda")
    dst = torch.tensor([0, 0, 9, 1, 0], dtype=torch.int32, device="cuda")      # edges 1, 2, 3 are bad; edge 4 is a coincident pair
    shift = torch.zeros(5, 3, device="cuda")
    vec, basis = edge_geometry(pos, src, dst, shift, 5.0, 8, 5)
    (g,) = torch.autograd.grad(basis.sum() + vec.sum(), pos)
    assert edge_geometry_device_status() == 2
    assert edge_geometry_device_status() == 0         # reading clears it
    assert torch.count_nonzero(vec[1:4]) == 0 and torch.count_nonzero(basis[1:4]) == 0
    assert torch.isfinite(basis).all() and torch.isfinite(g).all()
    want = torch.tensor([math.sqrt(2.0 / 5.0) * (n + 1) * math.pi / 5.0 for n in range(8)], device="cuda")
    assert torch.allclose(basis[4], want, rtol=1e-6)
    # the good edge alone gives the same result
    p2 = pos.detach().clone().requires_grad_(True)
    v1, b1 = edge_geometry(p2, src[:1], dst[:1], shift[:1], 5.0, 8, 5)
    (g1,) = torch.autograd.grad(b1.sum() + v1.sum(), p2)
    assert torch.equal(v1[0], vec[0]) and torch.equal(b1[0], basis[0])
    assert torch.allclose(g, g1, rtol=1e-6, atol=1e-7)


def test_device_status_helper_reports_and_clears():
    """``fasteq_b200.status.device_status`` names the family whose status word is set and clears it."""
    from fasteq_b200.ops.edge_geometry import edge_geometry
    from fasteq_b200.status import device_status
    device_status()                                   # clear whatever earlier tests left
    pos = torch.zeros(3, 3, device="cuda")
    bad = torch.tensor([5], dtype=torch.int32, device="cuda")
    ok = torch.tensor([0], dtype=torch.int32, device="cuda")
    edge_geometry(pos, bad, ok, torch.zeros(1, 3, device="cuda"), 5.0, 8, 5)
    assert device_status() == {"edge geometry": 2}
    assert device_status() == {}
