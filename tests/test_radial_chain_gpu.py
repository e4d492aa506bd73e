"""GPU parity of the fused radial-MLP hidden layers (one tcgen05 kernel per direction) against a float64
torch evaluation of the same bias-free SiLU MLP, values and the gradient with respect to the basis.
Bound: 1e-5 relative (the FP32 tolerance of the path)."""
import pytest
import torch


def _ref(basis, ws):
    h = basis.double()
    for w in ws:
        h = torch.nn.functional.silu(h @ w.double().t())
    return h


def _rel(a, b):
    return float((a.double() - b).norm() / b.norm().clamp_min(1e-30))


def test_cpu_tensors_and_trainable_weights_take_the_layered_path():
    from fasteq_b200.ops.radial_chain import radial_chain, radial_chain_usable
    b = torch.randn(10, 8)
    ws = [torch.randn(64, 8), torch.randn(64, 64)]
    assert radial_chain(b, ws) is None
    assert not radial_chain_usable(b.double(), ws)


@pytest.mark.gpu
@pytest.mark.parametrize("E", [1, 77, 128, 148 * 128 * 2 + 33, 148 * 128 * 5 + 1])
@pytest.mark.parametrize("n_hidden,nb", [(3, 8), (2, 8), (1, 8), (3, 5), (2, 16)])
def test_chain_forward_and_basis_gradient(E, n_hidden, nb):
    from fasteq_b200.ops.dense import tensorcore_device_status
    from fasteq_b200.ops.radial_chain import radial_chain
    if E > 100000 and (n_hidden, nb) not in ((3, 8), (2, 16)):
        pytest.skip("large case covered by two signatures")
    g = torch.Generator().manual_seed(E % 1000 + 10 * n_hidden + nb)
    basis = torch.randn(E, nb, generator=g)
    dims = [nb] + [64] * n_hidden
    ws = [torch.randn(o, i, generator=g) / i ** 0.5 for i, o in zip(dims[:-1], dims[1:])]
    r = torch.randn(E, 64, generator=g)
    bd = basis.double().requires_grad_(True)
    ref = _ref(bd, ws)
    (ref_g,) = torch.autograd.grad(ref, bd, r.double())
    bc = basis.cuda().requires_grad_(True)
    out = radial_chain(bc, [w.cuda() for w in ws])
    assert out is not None and out.shape == (E, 64)
    err = _rel(out.detach().cpu(), ref.detach())
    (gb,) = torch.autograd.grad(out, bc, r.cuda())
    errg = _rel(gb.cpu(), ref_g)
    assert tensorcore_device_status() == 0
    assert err <= 1e-5 and errg <= 1e-5, (err, errg)
    # row-wise: a misplaced tile or swapped group would hide in a norm over a large batch
    row_err = (out.detach().cpu().double() - ref.detach()).norm(dim=1) / ref.detach().norm(dim=1).clamp_min(1e-6)
    assert float(row_err.max()) <= 1e-4, float(row_err.max())


@pytest.mark.gpu
def test_radial_mlp_module_uses_the_same_values_as_the_layered_path():
    from fasteq_b200.nn.mace_style import RadialMLP
    torch.manual_seed(0)
    mlp = RadialMLP(8, [64, 64, 64], 1280).cuda()
    x = torch.randn(5000, 8, device="cuda")
    with torch.no_grad():
        fused = mlp(x)                                   # weights require grad, but grad mode is off: fused
    layered = mlp(x)                                     # grad mode on + trainable weights: layered
    assert _rel(fused.cpu(), layered.detach().cpu().double()) <= 1e-5
    for p in mlp.parameters():
        p.requires_grad_(False)
    xg = x.clone().requires_grad_(True)
    (g1,) = torch.autograd.grad(mlp(xg).sum(), xg)
    ws = [l.weight.double().cpu() for l in mlp.layers]
    xd = x.cpu().double().requires_grad_(True)
    (g2,) = torch.autograd.grad((_ref(xd, ws[:-1]) @ ws[-1].t()).sum(), xd)
    assert _rel(g1.cpu(), g2) <= 2e-5
