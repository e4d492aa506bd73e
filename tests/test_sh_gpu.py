"""GPU spherical harmonics against the e3nn golden vectors and the torch oracle."""
import numpy as np
import pytest
import torch

from oracle import sh_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-11), (torch.float32, 1e-5)])
@pytest.mark.parametrize("tag,normalize", [("n", True), ("u", False)])
def test_matches_e3nn_golden_values_and_gradient(golden, dtype, tol, tag, normalize):
    from fasteq_b200.ops.spherical_harmonics import spherical_harmonics
    vec = torch.tensor(golden["sh_vec"], dtype=dtype, device="cuda", requires_grad=True)
    sh = spherical_harmonics([0, 1, 2, 3, 4], vec, normalize, "component")
    ref = golden[f"sh_{tag}_val"]
    assert np.abs(sh.detach().cpu().double().numpy() - ref).max() <= tol * np.abs(ref).max()
    r = torch.tensor(golden[f"sh_{tag}_r"], dtype=dtype, device="cuda")
    (g,) = torch.autograd.grad((sh * r).sum(), vec)
    gref = golden[f"sh_{tag}_grad"]
    assert np.abs(g.cpu().double().numpy() - gref).max() <= tol * np.abs(gref).max()


@pytest.mark.parametrize("normalization", ["integral", "norm", "component"])
def test_normalizations_and_degree_subsets(normalization):
    from fasteq_b200.ops.spherical_harmonics import SphericalHarmonics
    g = torch.Generator().manual_seed(3)
    v = torch.randn(1000, 3, generator=g, dtype=torch.float64)
    mod = SphericalHarmonics("1x1o+1x3o", True, normalization)
    out = mod(v.cuda())
    full = sh_ref.spherical_harmonics(3, v, True, normalization)
    ref = torch.cat([full[:, 1:4], full[:, 9:16]], dim=1)
    assert (out.cpu() - ref).abs().max() < 1e-12
    assert str(mod.irreps_out) == "1x1o+1x3o"
    with pytest.raises(ValueError):
        SphericalHarmonics("1x2o", True)          # an even degree cannot be odd
    with pytest.raises(ValueError):
        mod(torch.zeros(4, 2, device="cuda"))


def test_zero_vector_is_finite():
    from fasteq_b200.ops.spherical_harmonics import spherical_harmonics
    v = torch.zeros(3, 3, device="cuda", requires_grad=True)
    sh = spherical_harmonics(3, v, True, "component")
    (g,) = torch.autograd.grad(sh.sum(), v)
    assert torch.isfinite(sh).all() and torch.isfinite(g).all()


@pytest.mark.parametrize("normalize,normalization", [(True, "component"), (False, "integral")])
def test_second_order_matches_torch_autograd(normalize, normalization):
    """The vector gradient is differentiable: d/d(grad_out) and d/d(vec) of <r, grad_vec> against torch autograd on a
    float64 evaluation of the same polynomials."""
    import math
    from fasteq_b200.ops.spherical_harmonics import SphericalHarmonics
    from fasteq_b200.sh import sh_polynomials
    ls = [0, 1, 2, 3]
    table = sh_polynomials(3)

    def ref_sh(v):
        if normalize:
            v = v / v.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        cols = []
        for l in ls:
            scale = {"component": 1.0, "norm": 1.0 / math.sqrt(2 * l + 1), "integral": 1.0 / math.sqrt(4 * math.pi)}[normalization]
            for p in table[l]:
                acc = torch.zeros_like(v[:, 0])
                for (a, b, c), coef in p.items():
                    acc = acc + coef * scale * v[:, 0] ** a * v[:, 1] ** b * v[:, 2] ** c
                cols.append(acc)
        return torch.stack(cols, 1)

    g = torch.Generator().manual_seed(2)
    vec = torch.randn(200, 3, generator=g, dtype=torch.float64) * 1.7
    go = torch.randn(200, 16, generator=g, dtype=torch.float64)
    r = torch.randn(200, 3, generator=g, dtype=torch.float64)

    def second(fn, dev):
        v, gt = vec.to(dev).requires_grad_(True), go.to(dev).requires_grad_(True)
        (gv,) = torch.autograd.grad(fn(v), v, gt, create_graph=True)
        return [t.detach().cpu() for t in torch.autograd.grad((gv * r.to(dev)).sum(), (gt, v))]

    ref = second(ref_sh, "cpu")
    got = second(SphericalHarmonics(ls, normalize, normalization), "cuda")
    for a, b in zip(got, ref):
        assert float((a - b).abs().max()) <= 1e-10 * max(1.0, float(b.abs().max()))
