"""Gate against the e3nn golden case; NequIP-style model energy / forces against the CPU oracle model."""
import numpy as np
import pytest
import torch

from fasteq_b200.irreps import Irreps, mul_ir_to_ir_mul, ir_mul_to_mul_ir

pytestmark = pytest.mark.gpu


def _golden_to_ours(x, u):
    """e3nn's sorted Gate input (6x0o + 24x0e + 6x1o + 6x1e + 6x2e, mul_ir) -> scalar 0e, scalar 0o, 3 gates, gated irreps (ir_mul)."""
    odd, even = x[:, :u], x[:, u:5 * u]
    gated = mul_ir_to_ir_mul(x[:, 5 * u:], Irreps(f"{u}x1o+{u}x1e+{u}x2e"))
    return np.concatenate([even[:, :u], odd, even[:, u:], gated], axis=1)


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-12), (torch.float32, 1e-5)])
def test_gate_matches_e3nn(golden, dtype, tol):
    from fasteq_b200.ops.gate import GateSpec, gate
    u = 6
    cs, cg = golden["gate_cst_scalars"], golden["gate_cst_gates"]
    spec = GateSpec(u, ["silu", "tanh"], ["silu"] * 3, [1, 1, 2], scalar_csts=cs, gate_csts=[cg[0]] * 3)
    x = torch.tensor(_golden_to_ours(golden["gate_x"], u), dtype=dtype, device="cuda", requires_grad=True)
    out = gate(x, spec)
    ref = golden["gate_out"]
    ref_ours = np.concatenate([ref[:, :2 * u], mul_ir_to_ir_mul(ref[:, 2 * u:], Irreps(f"{u}x1o+{u}x1e+{u}x2e"))], axis=1)
    assert np.abs(out.detach().cpu().double().numpy() - ref_ours).max() <= tol * np.abs(ref_ours).max()
    r = golden["gate_r"]
    r_ours = np.concatenate([r[:, :2 * u], mul_ir_to_ir_mul(r[:, 2 * u:], Irreps(f"{u}x1o+{u}x1e+{u}x2e"))], axis=1)
    (gx,) = torch.autograd.grad((out * torch.tensor(r_ours, dtype=dtype, device="cuda")).sum(), x)
    gref = _golden_to_ours(golden["gate_gx"], u)
    assert np.abs(gx.cpu().double().numpy() - gref).max() <= tol * np.abs(gref).max()


def test_quadrature_constants_agree_with_e3nn_samples(golden):
    from fasteq_b200.ops.gate import second_moment_constant
    assert abs(second_moment_constant("silu") - golden["gate_cst_scalars"][0]) < 5e-3
    assert abs(second_moment_constant("tanh") - golden["gate_cst_scalars"][1]) < 5e-3


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-11), (torch.float32, 1e-5)])
def test_nequip_style_energy_and_forces(dtype, tol):
    from fasteq_b200.graph import make_boxes
    from fasteq_b200.nn.nequip_style import NequIPStyleModel
    from oracle import mace_style_ref
    torch.manual_seed(0)
    b = make_boxes(1, 40, 8.0, 3.5, 2, seed=3)
    model = NequIPStyleModel(channels=16, num_layers=3, r_max=3.5, avg_num_neighbors=10.0).to(dtype)
    pos, spec = torch.from_numpy(b.positions).to(dtype), torch.from_numpy(b.species)
    src, dst, shift = torch.from_numpy(b.edge_src), torch.from_numpy(b.edge_dst), torch.from_numpy(b.edge_shift).to(dtype)
    e_ref, f_ref = mace_style_ref.nequip_energy_and_forces(model, pos, spec, src, dst, shift)
    m = model.cuda()
    out = m(pos.cuda(), spec.cuda(), src.cuda(), dst.cuda(), shift.cuda())
    from fasteq_b200.status import device_status
    assert device_status() == {}           # no kernel gave up on a wait or skipped an index
    e_err = abs(float(out["energy"].detach()) - float(e_ref.sum())) / max(abs(float(e_ref.sum())), float(e_ref.abs().max()))
    f = out["forces"].cpu().double()
    f_err = float((f - f_ref).abs().max() / f_ref.abs().max())
    assert e_err <= tol and f_err <= tol, (e_err, f_err)


def test_gate_second_order_matches_torch_autograd():
    """d/d(grad_out) and d/d(x) of <r, grad_x> against torch autograd on the dense float64 restatement."""
    from fasteq_b200.ops.gate import GateSpec, gate
    from oracle.mace_style_ref import gate_ref
    u = 8
    spec = GateSpec(u, ["silu", "tanh", "sigmoid"], ["silu", "tanh"], [1, 2])
    g = torch.Generator().manual_seed(4)
    B = 53
    x = torch.randn(B, spec.n_in * u, generator=g, dtype=torch.float64)
    go = torch.randn(B, spec.n_out * u, generator=g, dtype=torch.float64)
    r = torch.randn(B, spec.n_in * u, generator=g, dtype=torch.float64)

    def second(fn, dev):
        xt, gt = x.to(dev).requires_grad_(True), go.to(dev).requires_grad_(True)
        (gx,) = torch.autograd.grad(fn(xt), xt, gt, create_graph=True)
        return [t.detach().cpu() for t in torch.autograd.grad((gx * r.to(dev)).sum(), (gt, xt))]

    ref = second(lambda t: gate_ref(t, spec), "cpu")
    got = second(lambda t: gate(t, spec), "cuda")
    for a, b in zip(got, ref):
        assert float((a - b).abs().max()) <= 1e-12 * max(1.0, float(b.abs().max()))
