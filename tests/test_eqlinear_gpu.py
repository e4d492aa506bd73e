"""GPU parity of SO3Linear against the oracle, with the reference's configurations and bounds
(test/test_eqlinear.py:15-22, :119-171)."""
import numpy as np
import pytest
import torch

from fasteq_b200.descriptors import linear
from oracle import eqlinear_ref
from tests.test_eqlinear_cpu import _FakeDescriptor

pytestmark = pytest.mark.gpu

CONFIGS = {
    "SMALL_P1": (96, [1, 3, 5, 7]),
    "MEDIUM_P1": (128, [1, 3, 5, 7]),
    "MEDIUM_P2": (128, [1, 1, 3, 3, 3, 5, 5, 5, 7, 7]),
    "LARGE_P1": (224, [1, 3, 5, 7]),
    "LARGE_P3": (224, [1, 1, 1, 3, 3, 3, 3, 3, 5, 5, 5, 5, 5, 7, 7, 7, 7]),
}


def _make(shape, batch, dtype, seed=0):
    u, i_dims = CONFIGS[shape]
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(batch, sum(i_dims) * u, generator=g, dtype=torch.float64).to(dtype)
    w = torch.randn(len(i_dims) * u * u, generator=g, dtype=torch.float64).to(dtype)
    cg = [float(0.01 + 0.001 * p) for p in range(len(i_dims))]
    return x, w, cg, i_dims, u


def _rel_fro(a, b):
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _ref(x, w, i_dims, cg, u):
    m = eqlinear_ref.mapping_from_i_dims(i_dims)
    x3 = x.double().numpy().reshape(x.shape[0], -1, u)
    w3 = w.double().numpy().reshape(len(i_dims), u, u)
    return m, x3, w3, eqlinear_ref.eqlinear_forward(x3, w3, m, cg, eqlinear_ref.out_rows(i_dims))


@pytest.mark.parametrize("shape", list(CONFIGS))
@pytest.mark.parametrize("batch", [512, 2944])
def test_fp64_forward_and_grad(shape, batch):
    from fasteq_b200.ops.eqlinear import fast_equi_linear
    x, w, cg, i_dims, u = _make(shape, batch, torch.float64)
    m, x3, w3, ref = _ref(x, w, i_dims, cg, u)
    xd = x.cuda().requires_grad_(True)
    out = fast_equi_linear(_FakeDescriptor(i_dims, u, u, cg), w.cuda(), xd)
    assert out.shape == (batch, eqlinear_ref.out_rows(i_dims) * u)
    assert _rel_fro(out.detach().cpu().numpy().reshape(ref.shape), ref) <= 1e-12
    r = torch.randn(out.shape, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    (gx,) = torch.autograd.grad(out, xd, r.cuda())
    ref_gx = eqlinear_ref.eqlinear_dgrad(r.numpy().reshape(ref.shape), w3, m, cg, sum(i_dims))
    assert _rel_fro(gx.cpu().numpy().reshape(ref_gx.shape), ref_gx) <= 1e-12


@pytest.mark.parametrize("shape", list(CONFIGS))
@pytest.mark.parametrize("precision,bound", [("fp32", None), (None, 1e-5)])
def test_fp32_paths(shape, precision, bound):
    from fasteq_b200.ops.eqlinear import fast_equi_linear
    batch = 1024
    x, w, cg, i_dims, u = _make(shape, batch, torch.float32)
    m, x3, w3, ref = _ref(x, w, i_dims, cg, u)
    # error of a plain float32 evaluation of the same loop: the strict-FP32 yardstick of the reference
    ref32 = np.zeros(ref.shape, dtype=np.float32)
    for (ir, orow, wp, rows), c in zip(m, cg):
        ref32[:, orow:orow + rows, :] += np.float32(c) * (x3[:, ir:ir + rows, :].astype(np.float32) @ w3[wp].astype(np.float32))
    torch_rel = _rel_fro(ref32.astype(np.float64), ref)
    xd = x.cuda().requires_grad_(True)
    out = fast_equi_linear(_FakeDescriptor(i_dims, u, u, cg), w.cuda(), xd, compute_precision=precision)
    err = _rel_fro(out.detach().cpu().double().numpy().reshape(ref.shape), ref)
    assert err <= (bound if bound is not None else 1.05 * torch_rel + 1e-7), (err, torch_rel)
    r = torch.randn(out.shape, generator=torch.Generator().manual_seed(1))
    (gx,) = torch.autograd.grad(out, xd, r.cuda())
    ref_gx = eqlinear_ref.eqlinear_dgrad(r.double().numpy().reshape(ref.shape), w3, m, cg, sum(i_dims))
    errg = _rel_fro(gx.cpu().double().numpy().reshape(ref_gx.shape), ref_gx)
    assert errg <= (bound if bound is not None else 1.05 * torch_rel + 1e-7)


def test_e3nn_style_descriptor_with_shared_outputs_and_odd_sizes():
    """Explicit path indices, several paths into one output block, u != v, batch not a tile multiple."""
    from fasteq_b200.ops.eqlinear import fast_equi_linear, _descriptor_problem
    d = linear("24x0e+24x0e+24x1o+24x2e", "40x0e+40x1o+40x1o+40x2e")
    mapping, coeff, u, v, I, J = _descriptor_problem(d)
    g = torch.Generator().manual_seed(5)
    B = 333
    x = torch.randn(B, I * u, generator=g, dtype=torch.float64)
    w = torch.randn(len(d.paths) * u * v, generator=g, dtype=torch.float64)
    ref = eqlinear_ref.eqlinear_forward(x.numpy().reshape(B, I, u), w.numpy().reshape(-1, u, v), mapping, coeff, J)
    for dt, tol in ((torch.float64, 1e-12), (torch.float32, 1e-5)):
        xd = x.to(dt).cuda().requires_grad_(True)
        out = fast_equi_linear(d, w.to(dt).cuda(), xd)
        assert _rel_fro(out.detach().cpu().double().numpy().reshape(ref.shape), ref) <= tol
        (gx,) = torch.autograd.grad(out.sum(), xd)
        ref_gx = eqlinear_ref.eqlinear_dgrad(np.ones_like(ref), w.numpy().reshape(-1, u, v), mapping, coeff, I)
        assert _rel_fro(gx.cpu().double().numpy().reshape(ref_gx.shape), ref_gx) <= tol


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-12), (torch.float32, 2e-6)])
@pytest.mark.parametrize("shape,batch", [("MEDIUM_P2", 2944), ("SMALL_P1", 77), ("LARGE_P3", 700)])
def test_weight_gradient(shape, batch, dtype, tol):
    """grad_w against the float64 adjoint of the forward formula (two-stage deterministic reduction)."""
    from fasteq_b200.ops.eqlinear import fast_equi_linear
    x, w, cg, i_dims, u = _make(shape, batch, dtype)
    m, x3, w3, ref = _ref(x, w, i_dims, cg, u)
    wd = w.cuda().requires_grad_(True)
    xd = x.cuda().requires_grad_(True)
    out = fast_equi_linear(_FakeDescriptor(i_dims, u, u, cg), wd, xd, compute_precision="fp32" if dtype == torch.float32 else None)
    r = torch.randn(out.shape, generator=torch.Generator().manual_seed(2), dtype=torch.float64).to(dtype)
    gw, gx = torch.autograd.grad(out, (wd, xd), r.cuda())
    ref_gw = eqlinear_ref.eqlinear_wgrad(x3, r.double().numpy().reshape(ref.shape), m, cg, len(i_dims))
    assert gw.shape == w.shape
    assert _rel_fro(gw.cpu().double().numpy().reshape(ref_gw.shape), ref_gw) <= tol
    gw2, = torch.autograd.grad(fast_equi_linear(_FakeDescriptor(i_dims, u, u, cg), wd, xd.detach()), wd, r.cuda())
    assert torch.equal(gw, gw2)          # fixed reduction order: bit-identical across calls


def test_weight_gradient_with_permuted_weight_blocks():
    from fasteq_b200.ops.eqlinear import fast_equi_linear, _descriptor_problem
    d = linear("24x0e+24x0e+24x1o+24x2e", "40x0e+40x1o+40x1o+40x2e")
    mapping, coeff, u, v, I, J = _descriptor_problem(d)
    g = torch.Generator().manual_seed(6)
    B = 201
    x = torch.randn(B, I * u, generator=g, dtype=torch.float64)
    w = torch.randn(len(d.paths) * u * v, generator=g, dtype=torch.float64)
    r = torch.randn(B, J * v, generator=g, dtype=torch.float64)
    wd = w.cuda().requires_grad_(True)
    out = fast_equi_linear(d, wd, x.cuda())
    (gw,) = torch.autograd.grad(out, wd, r.cuda())
    ref = eqlinear_ref.eqlinear_wgrad(x.numpy().reshape(B, I, u), r.numpy().reshape(B, J, v), mapping, coeff, len(d.paths))
    assert _rel_fro(gw.cpu().numpy().reshape(ref.shape), ref) <= 1e-12


def test_second_order_by_composition():
    """The first backward is differentiable (force-loss training): gradients of <r_x, grad_x> + <r_w, grad_w>
    with respect to grad_out, w and x against torch autograd on a float64 restatement."""
    from fasteq_b200.ops.eqlinear import fast_equi_linear, _descriptor_problem
    d = linear("24x0e+24x1o+24x1o+24x2e", "40x0e+40x1o+40x2e")
    mapping, coeff, u, v, I, J = _descriptor_problem(d)
    g = torch.Generator().manual_seed(9)
    B = 130
    x = torch.randn(B, I * u, generator=g, dtype=torch.float64)
    w = torch.randn(len(d.paths) * u * v, generator=g, dtype=torch.float64)
    go = torch.randn(B, J * v, generator=g, dtype=torch.float64)
    rx, rw = torch.randn(B, I * u, generator=g, dtype=torch.float64), torch.randn(w.shape, generator=g, dtype=torch.float64)

    def ref_fn(wt, xt):
        w3, x3 = wt.reshape(len(d.paths), u, v), xt.reshape(B, I, u)
        out = xt.new_zeros(B, J, v)
        for (ir, orow, wp, rows), c in zip(mapping, coeff):
            out[:, orow:orow + rows, :] = out[:, orow:orow + rows, :] + c * (x3[:, ir:ir + rows, :] @ w3[wp])
        return out.reshape(B, J * v)

    def second(fn, dev):
        wt, xt, gt = (t.to(dev).requires_grad_(True) for t in (w, x, go))
        gw, gx = torch.autograd.grad(fn(wt, xt), (wt, xt), gt, create_graph=True)
        L = (gx * rx.to(dev)).sum() + (gw * rw.to(dev)).sum()
        return [t.detach().cpu() for t in torch.autograd.grad(L, (gt, wt, xt))]

    ref = second(ref_fn, "cpu")
    got = second(lambda wt, xt: fast_equi_linear(d, wt, xt), "cuda")
    for a, b in zip(got, ref):
        assert _rel_fro(a.numpy(), b.numpy()) <= 1e-12


@pytest.mark.parametrize("dtype,prec,tol", [(torch.float64, None, 1e-12), (torch.float32, "fp32", 2e-6), (torch.float32, None, 2e-5)])
def test_rows_without_a_path_are_zero(dtype, prec, tol):
    """Input blocks no path reads (their grad_x rows) and output blocks no path writes must come back as exact zeros,
    in the middle and at both ends of the row range: the tensor-product output of all parities mixed down to the
    natural-parity irreps (the benchmark's SO3Linear shape) plus an output irrep nothing feeds."""
    from fasteq_b200.ops.eqlinear import fast_equi_linear, _descriptor_problem
    d = linear("32x1e+32x0e+32x1o+32x2o+32x2e+32x0o", "32x3o+32x0e+32x1o+32x2e+32x4e")
    mapping, coeff, u, v, I, J = _descriptor_problem(d)
    assert len(d.paths) == 3 and I == 18 and J == 25
    g = torch.Generator().manual_seed(12)
    B = 333
    x = torch.randn(B, I * u, generator=g, dtype=torch.float64)
    w = torch.randn(len(d.paths) * u * v, generator=g, dtype=torch.float64)
    r = torch.randn(B, J * v, generator=g, dtype=torch.float64)
    xd = x.to(dtype).cuda().requires_grad_(True)
    out = fast_equi_linear(d, w.to(dtype).cuda(), xd, compute_precision=prec)
    (gx,) = torch.autograd.grad(out, xd, r.to(dtype).cuda())
    ref = eqlinear_ref.eqlinear_forward(x.numpy().reshape(B, I, u), w.numpy().reshape(-1, u, v), mapping, coeff, J)
    ref_gx = eqlinear_ref.eqlinear_dgrad(r.numpy().reshape(B, J, v), w.numpy().reshape(-1, u, v), mapping, coeff, I)
    o3, g3 = out.detach().cpu().double().numpy().reshape(ref.shape), gx.cpu().double().numpy().reshape(ref_gx.shape)
    assert _rel_fro(o3, ref) <= tol and _rel_fro(g3, ref_gx) <= tol
    assert np.count_nonzero(o3[:, :7]) == 0 and np.count_nonzero(o3[:, 16:]) == 0           # 3o (rows 0-6) and 4e (rows 16-24)
    assert np.count_nonzero(g3[:, :3]) == 0 and np.count_nonzero(g3[:, 7:12]) == 0 and np.count_nonzero(g3[:, 17:]) == 0
