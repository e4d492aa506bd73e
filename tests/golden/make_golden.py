"""Generate golden vectors from the e3nn 0.5.6 sources vendored in the reference tree.

Run where the reference tree is available:  python tests/golden/make_golden.py <reference-root>
(or set FASTEQ_REFERENCE).  Writes tests/golden/e3nn_golden.npz (float64).  The e3nn sources are imported in
place from the reference's model bundle; the one missing dependency
(opt_einsum_fx, an einsum-order optimiser) is replaced by an identity stub.
"""
import glob
import os
import sys
import types

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FASTEQ_REFERENCE")
if not REF:
    raise SystemExit("usage: make_golden.py <reference-root>  (the FastEq source tree)")
bundle = glob.glob(os.path.join(REF, "test/nequip_allegro_test/NequIP_OAM_R_4.5*nequip"))[0]
sys.path.insert(0, bundle)
stub = types.ModuleType("opt_einsum_fx")
stub.optimize_einsums_full = lambda model, example_inputs=None, *a, **k: model
stub.jitable = lambda x: x
sys.modules["opt_einsum_fx"] = stub

from e3nn.o3._wigner import wigner_3j  # noqa: E402
from e3nn.o3._irreps import Irreps  # noqa: E402
from e3nn.o3._spherical_harmonics import spherical_harmonics  # noqa: E402
from e3nn.o3._tensor_product._tensor_product import TensorProduct  # noqa: E402
from e3nn.o3._linear import Linear  # noqa: E402

torch.set_default_dtype(torch.float64)
out = {}

# 1. Wigner 3j
for l1 in range(4):
    for l2 in range(5):
        for l3 in range(abs(l1 - l2), min(l1 + l2, 4) + 1):
            out[f"w3j_{l1}_{l2}_{l3}"] = wigner_3j(l1, l2, l3).numpy()

# 2. spherical harmonics + gradient
g = torch.Generator().manual_seed(11)
vec = torch.randn(24, 3, generator=g) * 2.0
vec.requires_grad_(True)
for normalize in (True, False):
    sh = spherical_harmonics([0, 1, 2, 3, 4], vec, normalize=normalize, normalization="component")
    r = torch.randn(sh.shape, generator=g)
    (gv,) = torch.autograd.grad((sh * r).sum(), vec)
    tag = "n" if normalize else "u"
    out[f"sh_{tag}_val"], out[f"sh_{tag}_r"], out[f"sh_{tag}_grad"] = sh.detach().numpy(), r.numpy(), gv.numpy()
out["sh_vec"] = vec.detach().numpy()


def all_paths(in1, in2, lmax, natural=False):
    in1, in2 = Irreps(in1), Irreps(in2)
    blocks, ins = [], []
    for i1, (mul, ir1) in enumerate(in1):
        for i2, (_, ir2) in enumerate(in2):
            for ir in ir1 * ir2:
                if ir.l <= lmax and (not natural or ir.p == (-1) ** ir.l):
                    ins.append((i1, i2, len(blocks), "uvu", True))
                    blocks.append((mul, ir))
    return Irreps(blocks), ins


def tp_case(name, in1, in2, irreps_out, ins, z, seed):
    tp = TensorProduct(in1, in2, irreps_out, ins, shared_weights=False, internal_weights=False)
    g = torch.Generator().manual_seed(seed)
    x1 = torch.randn(z, tp.irreps_in1.dim, generator=g, requires_grad=True)
    v = torch.randn(z, 3, generator=g)
    x2 = spherical_harmonics(list(range(Irreps(in2).lmax + 1)), v, normalize=True, normalization="component").requires_grad_(True)
    w = torch.randn(z, tp.weight_numel, generator=g, requires_grad=True)
    o = tp(x1, x2, w)
    r = torch.randn(o.shape, generator=g)
    g1, g2, gw = torch.autograd.grad((o * r).sum(), (x1, x2, w))
    out[f"tp_{name}_irreps"] = np.array([str(tp.irreps_in1), str(tp.irreps_in2), str(tp.irreps_out)])
    out[f"tp_{name}_ins"] = np.array([(a, b, c) for a, b, c, *_ in ins], dtype=np.int64)
    for k, t in dict(x1=x1, x2=x2, w=w, out=o, r=r, g1=g1, g2=g2, gw=gw).items():
        out[f"tp_{name}_{k}"] = t.detach().numpy()


# 3a. one output block per path (MACE-style), all parities, l <= 3
io, ins = all_paths("4x0e+4x1o+4x2e", "1x0e+1x1o+1x2e+1x3o", 3)
tp_case("full", "4x0e+4x1o+4x2e", "1x0e+1x1o+1x2e+1x3o", io, ins, z=7, seed=3)
# 3b. shared output blocks (NequIP-style): several instructions feed one irreps_out block
in1, in2, o3 = Irreps("3x0e+3x1o+3x1e"), Irreps("1x0e+1x1o+1x2e"), Irreps("3x0e+3x1o+3x1e+3x2e")
ins = [(i1, i2, io_, "uvu", True) for i1, (_, a) in enumerate(in1) for i2, (_, b) in enumerate(in2)
       for io_, (_, c) in enumerate(o3) if c in a * b]
tp_case("shared", in1, in2, o3, ins, z=5, seed=4)

# 4. e3nn Linear
for name, a, b in (("simple", "4x0e+4x1o+4x2e", "6x0e+6x1o+6x2e"), ("multi", "4x0e+4x0e+4x1o", "5x0e+5x1o+5x1o")):
    lin = Linear(a, b, internal_weights=False, shared_weights=True)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(9, lin.irreps_in.dim, generator=g)
    w = torch.randn(lin.weight_numel, generator=g)
    out[f"lin_{name}_irreps"] = np.array([str(lin.irreps_in), str(lin.irreps_out)])
    out[f"lin_{name}_x"], out[f"lin_{name}_w"], out[f"lin_{name}_out"] = x.numpy(), w.numpy(), lin(x, w).numpy()
    out[f"lin_{name}_ins"] = np.array([(i.i_in, i.i_out) for i in lin.instructions], dtype=np.int64)
    out[f"lin_{name}_pw"] = np.array([i.path_weight for i in lin.instructions])

# 5. e3nn Gate (scalars through SiLU / tanh, gated irreps times SiLU(gates)), with the second-moment
#    normalisation constants e3nn attaches to the activations
from e3nn.nn._gate import Gate  # noqa: E402
gate = Gate("6x0e+6x0o", [torch.nn.functional.silu, torch.tanh], "18x0e", [torch.nn.functional.silu], "6x1o+6x1e+6x2e")
g = torch.Generator().manual_seed(9)
gx = torch.randn(11, gate.irreps_in.dim, generator=g, requires_grad=True)
gout = gate(gx)
gr = torch.randn(gout.shape, generator=g)
(ggx,) = torch.autograd.grad((gout * gr).sum(), gx)
out["gate_irreps"] = np.array([str(gate.irreps_in), str(gate.irreps_out)])
out["gate_x"], out["gate_out"], out["gate_r"], out["gate_gx"] = gx.detach().numpy(), gout.detach().numpy(), gr.numpy(), ggx.numpy()
out["gate_cst_scalars"] = np.array([a.cst if a is not None else 1.0 for a in gate.act_scalars.acts])
out["gate_cst_gates"] = np.array([a.cst if a is not None else 1.0 for a in gate.act_gates.acts])

# 6. Symmetric powers: e3nn's ReducedTensorProducts gives, per output irrep, a basis of the equivariant maps
#    Sym^nu(V) -> irrep.  Stored as polynomial coefficients over index multisets a_1 <= .. <= a_nu
#    (coefficient = sum of the symmetric tensor's entries over the distinct permutations of the multiset),
#    for the output irreps the symmetric-contraction tests use.  The symmetric contraction of the MACE-style
#    model contracts exactly these spaces with learned weights, so its table must span the same space.
import itertools  # noqa: E402
from e3nn.o3._reduce import ReducedTensorProducts  # noqa: E402
FORMULA = {2: ("ij=ji", "ij"), 3: ("ijk=jik=ikj", "ijk")}
for case, irr_in, wanted in (("l3", "1x0e+1x1o+1x2e+1x3o", ("0e", "1o")), ("l2", "1x0e+1x1o+1x2e", ("0e", "1o", "2e"))):
    dim = Irreps(irr_in).dim
    for nu in (2, 3):
        rtp = ReducedTensorProducts(FORMULA[nu][0], i=irr_in)
        Q = rtp.change_of_basis.numpy()                      # [irreps_out.dim, dim, .., dim]
        multisets = list(itertools.combinations_with_replacement(range(dim), nu))
        out[f"stc_{case}_nu{nu}_multisets"] = np.array(multisets, dtype=np.int64)
        off = 0
        for mul, ir in rtp.irreps_out:
            rows = Q[off:off + mul * ir.dim].reshape((mul, ir.dim) + (dim,) * nu)
            off += mul * ir.dim
            if str(ir) not in wanted:
                continue
            poly = np.zeros((mul, ir.dim, len(multisets)))
            for t, ms in enumerate(multisets):
                for perm in set(itertools.permutations(ms)):
                    poly[:, :, t] += rows[(slice(None), slice(None)) + perm]
            out[f"stc_{case}_nu{nu}_{ir}"] = poly
    out[f"stc_{case}_irreps_in"] = np.array([irr_in])

# 7. Radial basis of the reference's NequIP bundle: 8 Bessel functions times the p = 5 polynomial cutoff of the
#    normalised length x = r / r_max (module output: sinc(x n) n * cutoff(x); torch.sinc(z) = sin(pi z) / (pi z)).
from nequip.nn.embedding._edge import BesselEdgeLengthEncoding  # noqa: E402
from nequip.nn.embedding.cutoffs import PolynomialCutoff  # noqa: E402
enc = BesselEdgeLengthEncoding(cutoff=PolynomialCutoff(p=5), num_bessels=8)
xs = torch.cat([torch.linspace(0.02, 0.999, 40), torch.tensor([1.0, 1.05, 1.3])]).reshape(-1, 1)
res = enc({enc.norm_length_field: xs})
out["radial_x"] = xs.reshape(-1).numpy()
out["radial_cutoff_p5"] = PolynomialCutoff(p=5)(xs).reshape(-1).numpy()
out["radial_bessel8_times_cutoff"] = res[enc.edge_invariant_field].detach().numpy()

dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "e3nn_golden.npz")
np.savez_compressed(dst, **out)
print("wrote", dst, os.path.getsize(dst), "bytes,", len(out), "arrays")
