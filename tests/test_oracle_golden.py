"""Pin the CPU oracle and the descriptor generator against e3nn golden vectors (CPU only)."""
import numpy as np
import torch

from fasteq_b200.descriptors import channelwise_tensor_product
from fasteq_b200.irreps import Irreps, mul_ir_to_ir_mul, ir_mul_to_mul_ir
from fasteq_b200.wigner import wigner_3j
from oracle import e3nn_uvu_ref, sh_ref, uniform1d_ref


def test_wigner_3j_matches_e3nn(golden):
    n = 0
    for key in golden.files:
        if key.startswith("w3j_"):
            l1, l2, l3 = map(int, key.split("_")[1:])
            np.testing.assert_allclose(wigner_3j(l1, l2, l3), golden[key], atol=1e-14, rtol=0)
            n += 1
    assert n > 40


def test_sh_oracle_matches_e3nn(golden):
    for tag, normalize in (("n", True), ("u", False)):
        vec = torch.tensor(golden["sh_vec"], requires_grad=True)
        sh = sh_ref.spherical_harmonics(4, vec, normalize=normalize)
        np.testing.assert_allclose(sh.detach().numpy(), golden[f"sh_{tag}_val"], rtol=1e-12, atol=1e-12)
        (g,) = torch.autograd.grad((sh * torch.tensor(golden[f"sh_{tag}_r"])).sum(), vec)
        np.testing.assert_allclose(g.numpy(), golden[f"sh_{tag}_grad"], rtol=1e-11, atol=1e-11)


def _tp_case(golden, name):
    irr = [str(s) for s in golden[f"tp_{name}_irreps"]]
    ins = [(int(a), int(b), int(c), "uvu", True) for a, b, c in golden[f"tp_{name}_ins"]]
    return irr, ins


def test_e3nn_level_oracle_matches_e3nn(golden):
    for name in ("full", "shared"):
        irr, ins = _tp_case(golden, name)
        tp = e3nn_uvu_ref.TensorProductUVU(*irr, ins)
        x1 = torch.tensor(golden[f"tp_{name}_x1"], requires_grad=True)
        x2 = torch.tensor(golden[f"tp_{name}_x2"], requires_grad=True)
        w = torch.tensor(golden[f"tp_{name}_w"], requires_grad=True)
        o = tp(x1, x2, w)
        np.testing.assert_allclose(o.detach().numpy(), golden[f"tp_{name}_out"], rtol=1e-12, atol=1e-13)
        g1, g2, gw = torch.autograd.grad((o * torch.tensor(golden[f"tp_{name}_r"])).sum(), (x1, x2, w))
        np.testing.assert_allclose(g1.numpy(), golden[f"tp_{name}_g1"], rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(g2.numpy(), golden[f"tp_{name}_g2"], rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(gw.numpy(), golden[f"tp_{name}_gw"], rtol=1e-12, atol=1e-12)


def test_path_table_and_path_oracle_match_e3nn(golden):
    """descriptor (ir_mul path table) + numpy Uniform1D oracle == e3nn TensorProduct, values and grads."""
    for name in ("full", "shared"):
        irr, ins = _tp_case(golden, name)
        d = channelwise_tensor_product(*irr, ins)
        i1, i2, io = Irreps(irr[0]), Irreps(irr[1]), Irreps(irr[2])
        z = golden[f"tp_{name}_x1"].shape[0]
        x = mul_ir_to_ir_mul(golden[f"tp_{name}_x1"], i1).reshape(z, d.x_seg_num, d.u_dim)
        y = golden[f"tp_{name}_x2"].reshape(z, d.y_seg_num, 1)
        w = golden[f"tp_{name}_w"].reshape(z, d.w_seg_num, d.u_dim)
        paths = list(zip(d.i_list, d.j_list, d.k_list, d.v_list))
        out = uniform1d_ref.uniform1d_forward(w, x, y, paths, d.coeff_list, d.out_seg_num)
        got = ir_mul_to_mul_ir(out.reshape(z, -1), io)
        np.testing.assert_allclose(got, golden[f"tp_{name}_out"], rtol=1e-12, atol=1e-13)
        r = mul_ir_to_ir_mul(golden[f"tp_{name}_r"], io).reshape(z, d.out_seg_num, d.u_dim)
        gw, gx, gy = uniform1d_ref.uniform1d_backward(r, w, x, y, paths, d.coeff_list)
        np.testing.assert_allclose(ir_mul_to_mul_ir(gx.reshape(z, -1), i1), golden[f"tp_{name}_g1"], rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(gy.reshape(z, -1), golden[f"tp_{name}_g2"], rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(gw.reshape(z, -1), golden[f"tp_{name}_gw"], rtol=1e-12, atol=1e-12)


def test_path_oracle_reference_fixture():
    """The formula-plus-seed case of the reference's own test
    (tests/adapters/test_uniform1d_hip_forward.py:48-68): N=5, E=11, paths
    [(0,0,0,0),(1,1,1,0),(0,1,0,2)], coeffs [.5,-.25,.75], src=3e%N, dst=2e%N, checked
    against the 4-line loop it uses as reference, including the untouched segment 1."""
    rng = np.random.default_rng(1701)
    N, E, U = 5, 11, 33
    paths = [(0, 0, 0, 0), (1, 1, 1, 0), (0, 1, 0, 2)]
    coeffs = [.5, -.25, .75]
    src, dst = (np.arange(E) * 3) % N, (np.arange(E) * 2) % N
    w, x, y = rng.normal(size=(E, 2, U)), rng.normal(size=(N, 2, U)), rng.normal(size=(E, 2, 1))
    ref = np.zeros((E, 3, U))
    for (i, j, k, v), c in zip(paths, coeffs):
        ref[:, v] += c * w[:, i] * x[src][:, j] * y[:, k]
    exp = np.zeros((N, 3, U)); np.add.at(exp, dst, ref)
    got = uniform1d_ref.uniform1d_forward(w, x, y, paths, coeffs, 3, src_x=src, dst=dst, num_out_rows=N)
    np.testing.assert_allclose(got, exp, rtol=1e-13, atol=1e-13)
    assert np.count_nonzero(got[:, 1]) == 0


def test_radial_basis_matches_the_reference_bundle(golden):
    """Polynomial cutoff (p = 5) and Bessel basis against the reference's NequIP bundle, for the model oracle's own
    restatement and for the product's functions.  The bundle normalises the Bessel functions as ``sinc(n x) n``
    (x = r / r_max); the MACE-style ``sqrt(2 / r_max) sin(n pi r / r_max) / r`` used here is that times the
    constant ``sqrt(2 / r_max) pi / r_max``."""
    import math
    from fasteq_b200.nn import mace_style
    from oracle import mace_style_ref
    r_max = 5.0
    x = torch.tensor(golden["radial_x"])
    r = x * r_max
    k = math.sqrt(2.0 / r_max) * math.pi / r_max
    for mod in (mace_style_ref, mace_style):
        cut = mod.polynomial_cutoff(r, r_max, 5)
        np.testing.assert_allclose(cut.numpy(), golden["radial_cutoff_p5"], rtol=1e-12, atol=1e-14)
        rb = mod.bessel_basis(r, r_max, 8) * cut.unsqueeze(-1)
        np.testing.assert_allclose(rb.numpy(), k * golden["radial_bessel8_times_cutoff"], rtol=1e-11, atol=1e-13)
    assert float(golden["radial_cutoff_p5"][-1]) == 0.0 and float(golden["radial_cutoff_p5"][-3]) == 0.0   # x >= 1


def test_model_oracle_linear_mapping_matches_e3nn(golden):
    """The model oracle's own reading of a uv,iu,iv descriptor reproduces e3nn ``Linear`` on the golden cases
    (independently of the product's descriptor parser)."""
    from fasteq_b200.descriptors import linear
    from oracle import mace_style_ref
    for name in ("simple", "multi"):
        a, b = (str(s) for s in golden[f"lin_{name}_irreps"])
        d = linear(a, b)
        x = torch.tensor(mul_ir_to_ir_mul(golden[f"lin_{name}_x"], Irreps(a)))
        w = torch.tensor(golden[f"lin_{name}_w"])
        out = mace_style_ref.eqlinear(x, w, d)
        np.testing.assert_allclose(ir_mul_to_mul_ir(out.numpy(), Irreps(b)), golden[f"lin_{name}_out"], rtol=1e-12, atol=1e-12)
