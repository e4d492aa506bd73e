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
