"""SO3Linear oracle, descriptor generator and front-end logic on the CPU."""
import numpy as np
import pytest
import torch

from fasteq_b200.descriptors import linear
from fasteq_b200.irreps import Irreps, mul_ir_to_ir_mul, ir_mul_to_mul_ir
from fasteq_b200.ops import eqlinear as eq
from oracle import eqlinear_ref


def _torch_loop_reference(x, w, i_dims, cg):
    """The loop of test/test_eqlinear.py:38-69, transcribed for float64 numpy."""
    runs = eqlinear_ref.runs_of(i_dims)
    in_prefix = np.concatenate([[0], np.cumsum(i_dims)[:-1]])
    out = np.zeros((x.shape[0], eqlinear_ref.out_rows(i_dims), w.shape[2]))
    j0 = 0
    for i, p0, count in runs:
        for t in range(i):
            for q in range(p0, p0 + count):
                out[:, j0 + t, :] += x[:, in_prefix[q] + t, :] @ w[q] * cg[q]
        j0 += i
    return out


@pytest.mark.parametrize("i_dims", [[1, 3, 5, 7], [1, 1, 3, 3, 3, 5, 5, 5, 7, 7]])
def test_oracle_matches_reference_loop(i_dims):
    rng = np.random.default_rng(0)
    u = 8
    x = rng.normal(size=(5, sum(i_dims), u)); w = rng.normal(size=(len(i_dims), u, u))
    cg = [0.01 + 0.001 * p for p in range(len(i_dims))]
    m = eqlinear_ref.mapping_from_i_dims(i_dims)
    got = eqlinear_ref.eqlinear_forward(x, w, m, cg, eqlinear_ref.out_rows(i_dims))
    np.testing.assert_allclose(got, _torch_loop_reference(x, w, i_dims, cg), rtol=1e-13, atol=1e-13)
    # grad_x is the adjoint of the forward
    r = rng.normal(size=got.shape)
    gx = eqlinear_ref.eqlinear_dgrad(r, w, m, cg, sum(i_dims))
    assert abs((gx * x).sum() - (got * r).sum()) < 1e-9 * abs((got * r).sum())


@pytest.mark.parametrize("name", ["simple", "multi"])
def test_linear_descriptor_matches_e3nn(golden, name):
    irr_in, irr_out = (Irreps(str(s)) for s in golden[f"lin_{name}_irreps"])
    d = linear(irr_in, irr_out)
    ins = golden[f"lin_{name}_ins"]
    assert [(p.indices[1], p.indices[2]) for p in d.paths] == [tuple(t) for t in ins.tolist()]
    np.testing.assert_allclose([p.coefficients for p in d.paths], golden[f"lin_{name}_pw"], rtol=1e-14)
    mapping, coeff, u, v, I, J = eq._descriptor_problem(d)
    x = mul_ir_to_ir_mul(golden[f"lin_{name}_x"], irr_in).reshape(-1, I, u)
    w = golden[f"lin_{name}_w"].reshape(len(d.paths), u, v)
    out = eqlinear_ref.eqlinear_forward(x, w, mapping, coeff, J)
    got = ir_mul_to_mul_ir(out.reshape(out.shape[0], -1), irr_out)
    np.testing.assert_allclose(got, golden[f"lin_{name}_out"], rtol=1e-12, atol=1e-12)


class _FakePath:
    def __init__(self, c):
        self.coefficients = c


class _FakeDescriptor:
    """Index-free descriptor exactly as in the reference's test (test/test_eqlinear.py:72-101)."""

    def __init__(self, i_dims, u, v, cg):
        self.paths = [_FakePath(c) for c in cg]
        runs = [i for i, _, _ in eqlinear_ref.runs_of(i_dims)]
        self.operands = [tuple((u * v,) for _ in i_dims), tuple((i,) for i in i_dims), tuple((i,) for i in runs)]
        self._u, self._v, self._i = u, v, list(i_dims)

    def get_dims(self, name):
        return [self._u] if name == "u" else [self._v]

    def get_dimensions_dict(self):
        return {"i": list(self._i)}


def test_front_end_geometry_and_errors():
    i_dims = [1, 1, 3, 3, 3, 5]
    d = _FakeDescriptor(i_dims, 16, 16, [0.5] * 6)
    mapping, coeff, u, v, I, J = eq._descriptor_problem(d)
    assert mapping == eqlinear_ref.mapping_from_i_dims(i_dims) and (u, v, I, J) == (16, 16, 16, 9)
    x32, w64 = torch.zeros(2, 4), torch.zeros(4, dtype=torch.float64)
    with pytest.raises(ValueError, match="same dtype"):
        eq._resolve_precision(x32, w64, None)
    with pytest.raises(ValueError, match="compute_precision"):
        eq._resolve_precision(x32, x32, "bf16")
    with pytest.raises(ValueError, match="float32 and float64"):
        eq._resolve_precision(x32.half(), x32.half(), None)
    assert eq._resolve_precision(x32, x32, None) == 0 and eq._resolve_precision(x32, x32, "fp32") == 1
    assert eq._resolve_precision(w64, w64, "fp32") == 2
    d2 = linear("4x0e+4x1o", "4x0e+4x1o")
    d2.operands_and_subscripts = tuple(zip(d2.operands, ("uv", "iu", "iw")))
    with pytest.raises(NotImplementedError):
        eq._descriptor_problem(d2)
    with pytest.raises(RuntimeError, match="no CPU path"):
        eq.fast_equi_linear(linear("4x0e", "4x0e"), torch.zeros(16), torch.zeros(3, 4))


def test_oracle_weight_gradient_is_the_adjoint_of_the_forward():
    """<r, forward(x, w + dw) - forward(x, w)> == <wgrad(x, r), dw> exactly (the forward is linear in w)."""
    import numpy as np
    from oracle import eqlinear_ref
    rng = np.random.default_rng(3)
    i_dims, u, v, B = [1, 1, 3, 3, 5], 6, 4, 9
    m = eqlinear_ref.mapping_from_i_dims(i_dims)
    cg = [0.3 + 0.1 * q for q in range(len(i_dims))]
    J = eqlinear_ref.out_rows(i_dims)
    x = rng.standard_normal((B, sum(i_dims), u)); dw = rng.standard_normal((len(i_dims), u, v))
    r = rng.standard_normal((B, J, v))
    lhs = float((r * eqlinear_ref.eqlinear_forward(x, dw, m, cg, J)).sum())
    rhs = float((eqlinear_ref.eqlinear_wgrad(x, r, m, cg, len(i_dims)) * dw).sum())
    assert abs(lhs - rhs) <= 1e-12 * max(1.0, abs(lhs))
