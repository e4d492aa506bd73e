"""GPU parity of the symmetric tensor contraction against the path-level oracle."""
import numpy as np
import pytest
import torch

from fasteq_b200.descriptors import symmetric_contraction
from oracle import stc_ref

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.float64: 1e-11}


def _close(got, ref, dtype, what):
    got = got.detach().cpu().double().numpy().reshape(ref.shape)
    err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert err <= TOL[dtype], f"{what}: relative error {err:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("irr_in,irr_out,B,S", [
    ("128x0e+128x1o+128x2e+128x3o", "128x0e+128x1o", 257, 4),     # config 1 product basis
    ("33x0e+33x1o+33x2e", "33x0e+33x1o+33x2e", 19, 10),           # channel tail, every output irrep
])
def test_forward_backward(dtype, irr_in, irr_out, B, S):
    from fasteq_b200.ops import fast_stc_uniform1d_jit
    d = symmetric_contraction(irr_in, irr_out)
    U = d.u_dim
    g = torch.Generator().manual_seed(0)
    x1 = (torch.randn(B, d.x1_segs, U, generator=g, dtype=torch.float64) * 0.3).to(dtype)
    x0 = (torch.randn(S, d.x0_segs, U, generator=g, dtype=torch.float64) * 0.1).to(dtype)
    i0 = torch.randint(0, S, (B,), generator=g)
    r = torch.randn(B, d.out_segs * U, generator=g, dtype=torch.float64).to(dtype)
    coeffs, paths, idx_lists = d.tensors(dtype, "cuda")
    x1d, x0d = x1.cuda().requires_grad_(True), x0.cuda().requires_grad_(True)
    out = fast_stc_uniform1d_jit(x1d, x0d, i0.cuda(), coeffs, paths, idx_lists, d.out_segs)
    assert out.shape == (B, d.out_segs * U)
    x1n, x0n = x1.double().numpy(), x0.double().numpy()
    ref = stc_ref.stc_forward(x1n, x0n, i0.numpy(), d.paths, d.coeffs, d.out_segs)
    _close(out, ref, dtype, "forward")
    gx1, gx0 = torch.autograd.grad((out * r.cuda()).sum(), (x1d, x0d))
    rgx1, rgx0 = stc_ref.stc_backward(r.double().numpy().reshape(ref.shape), x1n, x0n, i0.numpy(), d.paths, d.coeffs)
    _close(gx1, rgx1, dtype, "grad_x1")
    _close(gx0, rgx0, dtype, "grad_x0")
    # forces only need grad_x1: the module without the weight gradient must agree
    (gx1b,) = torch.autograd.grad((fast_stc_uniform1d_jit(x1d, x0d.detach(), i0.cuda(), coeffs, paths, idx_lists, d.out_segs) * r.cuda()).sum(), (x1d,))
    _close(gx1b, rgx1, dtype, "grad_x1 (no weight gradient)")


def test_rejects_cpu_and_mismatched_inputs():
    from fasteq_b200.ops import fast_stc_uniform1d_jit
    d = symmetric_contraction("4x0e+4x1o", "4x0e")
    coeffs, paths, idx_lists = d.tensors(torch.float32, "cuda")
    x1 = torch.zeros(3, d.x1_segs, 4, device="cuda"); x0 = torch.zeros(2, d.x0_segs, 4, device="cuda")
    i0 = torch.zeros(3, dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError, match="no CPU path"):
        fast_stc_uniform1d_jit(x1.cpu(), x0, i0, coeffs, paths, idx_lists, d.out_segs)
    with pytest.raises(ValueError):
        fast_stc_uniform1d_jit(x1, x0.double(), i0, coeffs, paths, idx_lists, d.out_segs)
    out = fast_stc_uniform1d_jit(x1, x0, i0, coeffs, paths, idx_lists, d.out_segs)
    assert out.shape == (3, d.out_segs * 4) and float(out.abs().max()) == 0.0


def _torch_stc(x1, x0, i0, paths, coeffs, out_segs, pad_value=-1):
    """Differentiable float64 restatement of the path formula (for second-order references)."""
    B, _, U = x1.shape
    xg = x0[i0]
    cols = [x1.new_zeros(B, U) for _ in range(out_segs)]
    for row, c in zip(paths, coeffs):
        vals = [int(t) for t in row if int(t) != pad_value]
        a, d, v = vals[:-2], vals[-2], vals[-1]
        term = xg[:, d, :] * float(c)
        for t in a:
            term = term * x1[:, t, :]
        cols[v] = cols[v] + term
    return torch.stack(cols, 1).reshape(B, out_segs * U)


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-11), (torch.float32, 2e-5)])
def test_second_order_matches_torch_autograd(dtype, tol):
    """grad of <r1, grad_x1> + <r0, grad_x0> with respect to grad_out, x1 and x0 (what a force loss needs)."""
    from fasteq_b200.ops import fast_stc_uniform1d_jit
    d = symmetric_contraction("16x0e+16x1o+16x2e", "16x0e+16x1o")
    U, B, S = d.u_dim, 37, 3
    g = torch.Generator().manual_seed(1)
    x1 = (torch.randn(B, d.x1_segs, U, generator=g, dtype=torch.float64) * 0.5)
    x0 = (torch.randn(S, d.x0_segs, U, generator=g, dtype=torch.float64) * 0.3)
    i0 = torch.randint(0, S, (B,), generator=g)
    go = torch.randn(B, d.out_segs * U, generator=g, dtype=torch.float64)
    r1 = torch.randn(B, d.x1_segs, U, generator=g, dtype=torch.float64)
    r0 = torch.randn(S, d.x0_segs, U, generator=g, dtype=torch.float64)

    def second_order(fn, dt, dev):
        a, w, gout = (t.to(dt).to(dev).requires_grad_(True) for t in (x1, x0, go))
        out = fn(a, w)
        gx1, gx0 = torch.autograd.grad(out, (a, w), gout, create_graph=True)
        L = (gx1 * r1.to(dt).to(dev)).sum() + (gx0 * r0.to(dt).to(dev)).sum()
        return [t.detach().cpu().double() for t in torch.autograd.grad(L, (gout, a, w))]

    ref = second_order(lambda a, w: _torch_stc(a, w, i0, d.paths, d.coeffs, d.out_segs), torch.float64, "cpu")
    coeffs, paths, idx_lists = d.tensors(dtype, "cuda")
    got = second_order(lambda a, w: fast_stc_uniform1d_jit(a, w, i0.cuda(), coeffs, paths, idx_lists, d.out_segs), dtype, "cuda")
    for name, a, b in zip(("d grad_out", "d x1", "d x0"), got, ref):
        err = float((a - b).abs().max() / b.abs().max())
        assert err <= tol, f"{name}: relative error {err:.3e}"
