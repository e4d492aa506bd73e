"""Path tables ("descriptors") for the three operators of the message-passing hot path.

The reference receives these tables from cuEquivariance descriptors
(``cue.descriptors.channelwise_tensor_product`` etc., called at
test/bench_tensor_product_uniform1d.py:127-130); that package is not part of
the reference tree, so the tables are generated here from e3nn's published
``TensorProduct`` semantics (e3nn/o3/_tensor_product/_tensor_product.py:277-323
for the path normalisation, _codegen.py:166-187 for the uvu contraction).

A Uniform1D table is the flat list ``(i, j, k, v, coeff)`` of the reference's
``meta`` dict (fasteq/ops/uniform1d_jit.py:3216-3235):
``out[v, u] += coeff * w[i, u] * x[j, u] * y[k, (u|0)]``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from math import sqrt
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .irreps import Irreps, Irrep
from .wigner import wigner_3j


@dataclass(frozen=True)
class Instruction:
    """One (l1, l2, l3) coupling: rows of x, y, out it touches and its weight segment."""
    w_seg: int
    x_off: int
    y_off: int
    out_off: int
    l1: int
    l2: int
    l3: int
    path_weight: float  # e3nn's sqrt(alpha)


@dataclass
class Uniform1DDescriptor:
    i_list: np.ndarray
    j_list: np.ndarray
    k_list: np.ndarray
    v_list: np.ndarray
    coeff_list: np.ndarray  # float64
    w_seg_num: int
    x_seg_num: int
    y_seg_num: int
    out_seg_num: int
    u_dim: int
    y_u_dim: int = 1  # 1 = "u,u,,u" (scalar y per segment), u_dim = "u,u,u,u"
    instructions: Tuple[Instruction, ...] = ()
    irreps_in1: Optional[Irreps] = None
    irreps_in2: Optional[Irreps] = None
    irreps_out: Optional[Irreps] = None

    @property
    def num_paths(self) -> int:
        return int(self.i_list.shape[0])

    def meta(self, dtype=None, device=None) -> Dict:
        """The ``meta`` dict ``fast_uniform1d_jit`` takes (same keys as the reference)."""
        import torch
        dtype = dtype or torch.float32
        t = lambda a: torch.as_tensor(np.ascontiguousarray(a), dtype=torch.int32, device=device)
        return dict(
            i_list=t(self.i_list), j_list=t(self.j_list), k_list=t(self.k_list), v_list=t(self.v_list),
            coeff_list=torch.as_tensor(self.coeff_list, dtype=dtype, device=device),
            w_seg_num=self.w_seg_num, x_seg_num=self.x_seg_num, y_seg_num=self.y_seg_num,
            out_seg_num=self.out_seg_num, u_dim=self.u_dim,
            size_list=[self.w_seg_num * self.u_dim, self.x_seg_num * self.u_dim,
                       self.y_seg_num * self.y_u_dim, self.out_seg_num * self.u_dim],
        )


def full_channelwise_instructions(irreps_in1, irreps_in2, lmax_out: int, sort: bool = False,
                                  parity_filter: Optional[str] = None):
    """All allowed uvu couplings of ``irreps_in1 x irreps_in2`` up to ``lmax_out``.

    Returns ``(irreps_out, instructions)`` with one output block per coupling
    (the MACE / NequIP convolution construction).  ``parity_filter='natural'``
    keeps only outputs with parity ``(-1)^l`` (MACE's default).  ``sort=True``
    orders the output blocks by (l, parity) the way e3nn's ``Irreps.sort`` does
    and remaps the instructions.
    """
    irreps_in1, irreps_in2 = Irreps(irreps_in1), Irreps(irreps_in2)
    out_blocks, instr = [], []
    for i1, b1 in enumerate(irreps_in1):
        for i2, b2 in enumerate(irreps_in2):
            for ir in b1.ir * b2.ir:
                if ir.l > lmax_out:
                    continue
                if parity_filter == "natural" and ir.p != (-1) ** ir.l:
                    continue
                k = len(out_blocks)
                out_blocks.append((b1.mul, ir))
                instr.append((i1, i2, k, "uvu", True))
    if sort:
        # e3nn orders irreps by (l, then even before odd for even l / odd before even for odd l);
        # a stable sort on (l, -p*(-1)^l) reproduces Irrep.__lt__.
        order = sorted(range(len(out_blocks)), key=lambda n: (out_blocks[n][1].l, -out_blocks[n][1].p * (-1) ** out_blocks[n][1].l))
        inv = {old: new for new, old in enumerate(order)}
        out_blocks = [out_blocks[o] for o in order]
        instr = sorted([(a, b, inv[c], m, h) for a, b, c, m, h in instr], key=lambda t: t[2])
    return Irreps(out_blocks), instr


def channelwise_tensor_product(irreps_in1, irreps_in2, irreps_out, instructions,
                               irrep_normalization: str = "component",
                               path_normalization: str = "element") -> Uniform1DDescriptor:
    """Flatten an e3nn ``TensorProduct`` with ``uvu`` instructions into a Uniform1D table.

    ``instructions`` are e3nn tuples ``(i_in1, i_in2, i_out, "uvu", has_weight[, path_weight])``.
    Every ``irreps_in2`` block must have multiplicity 1 (edge attributes / spherical
    harmonics) and ``irreps_in1`` / ``irreps_out`` a uniform multiplicity ``u``.
    """
    irreps_in1, irreps_in2, irreps_out = Irreps(irreps_in1), Irreps(irreps_in2), Irreps(irreps_out)
    u = irreps_in1.uniform_mul()
    if any(b.mul != 1 for b in irreps_in2):
        raise ValueError("channelwise tensor product needs multiplicity 1 on irreps_in2")
    if any(b.mul != u for b in irreps_out):
        raise ValueError("irreps_out must carry the multiplicity of irreps_in1")
    norm = []
    for ins in instructions:
        ins = tuple(ins) + ((1.0,) if len(ins) == 5 else ())
        if ins[3] != "uvu" or not ins[4]:
            raise NotImplementedError("only weighted 'uvu' instructions are supported")
        norm.append(ins)
    x_offs, y_offs, o_offs = irreps_in1.segment_offsets(), irreps_in2.segment_offsets(), irreps_out.segment_offsets()

    il, jl, kl, vl, cl, table = [], [], [], [], [], []
    for n, (i1, i2, io, _, _, pw_user) in enumerate(norm):
        ir1, ir2, iro = irreps_in1[i1].ir, irreps_in2[i2].ir, irreps_out[io].ir
        if ir1.p * ir2.p != iro.p or not (abs(ir1.l - ir2.l) <= iro.l <= ir1.l + ir2.l):
            raise ValueError(f"instruction {n} violates the selection rules")
        alpha = {"component": float(iro.dim), "norm": float(ir1.dim * ir2.dim), "none": 1.0}[irrep_normalization]
        if path_normalization == "element":
            fan = sum(irreps_in2[t[1]].mul for t in norm if t[2] == io)
        elif path_normalization == "path":
            fan = irreps_in2[i2].mul * len([t for t in norm if t[2] == io])
        else:
            fan = 1
        if fan > 0:
            alpha /= fan
        alpha *= pw_user
        pw = sqrt(alpha)
        c3 = wigner_3j(ir1.l, ir2.l, iro.l)
        table.append(Instruction(n, x_offs[i1], y_offs[i2], o_offs[io], ir1.l, ir2.l, iro.l, pw))
        for m1, m2, m3 in zip(*np.nonzero(c3)):
            il.append(n); jl.append(x_offs[i1] + m1); kl.append(y_offs[i2] + m2); vl.append(o_offs[io] + m3)
            cl.append(pw * c3[m1, m2, m3])
    i32 = lambda a: np.asarray(a, dtype=np.int32)
    return Uniform1DDescriptor(
        i32(il), i32(jl), i32(kl), i32(vl), np.asarray(cl, dtype=np.float64),
        w_seg_num=len(norm), x_seg_num=irreps_in1.num_segments, y_seg_num=irreps_in2.num_segments,
        out_seg_num=irreps_out.num_segments, u_dim=u, y_u_dim=1, instructions=tuple(table),
        irreps_in1=irreps_in1, irreps_in2=irreps_in2, irreps_out=irreps_out,
    )


# --------------------------------------------------------------------------- SO3Linear

@dataclass(frozen=True)
class LinearPath:
    indices: Tuple[int, int, int]   # (weight block, input segment, output segment)
    coefficients: float


class LinearDescriptor:
    """``uv,iu,iv`` descriptor with the attribute protocol ``fast_equi_linear`` reads
    (fasteq/ops/auto_schedule/eqlinear_descriptor.py:228-310): ``operands`` (weight, input,
    output segment tuples), ``paths[q].indices / .coefficients``, ``get_dims``,
    ``get_dimensions_dict``, ``operands_and_subscripts``, ``coefficient_subscripts``."""

    coefficient_subscripts = ""

    def __init__(self, in_dims: Sequence[int], out_dims: Sequence[int], u: int, v: int, paths: Sequence[LinearPath]):
        self.u, self.v = int(u), int(v)
        self.paths = list(paths)
        self.operands = [tuple((self.u, self.v) for _ in self.paths), tuple((int(i), self.u) for i in in_dims),
                         tuple((int(i), self.v) for i in out_dims)]
        self.operands_and_subscripts = tuple(zip(self.operands, ("uv", "iu", "iv")))

    def get_dims(self, name: str):
        return {"u": [self.u], "v": [self.v]}[name]

    def get_dimensions_dict(self):
        return {"i": sorted({s[0] for s in self.operands[1] + self.operands[2]}), "u": [self.u], "v": [self.v]}

    @property
    def num_weights(self) -> int:
        return len(self.paths) * self.u * self.v


def linear(irreps_in, irreps_out, path_normalization: str = "element", scale: float = 1.0) -> LinearDescriptor:
    """e3nn ``o3.Linear(irreps_in, irreps_out)`` as a uv,iu,iv descriptor (all path coefficients times ``scale``).

    One path per (input block, output block) pair of equal irrep, in e3nn's instruction order
    (input-major); coefficient ``sqrt(1 / fan_in)`` with ``fan_in`` the summed input multiplicity
    feeding the output block (e3nn/o3/_linear.py:148-159).  Weight block q is e3nn's
    ``[mul_in, mul_out]`` matrix of instruction q, so ``weight.reshape(P, u, v)`` is the operand."""
    irreps_in, irreps_out = Irreps(irreps_in), Irreps(irreps_out)
    u, v = irreps_in.uniform_mul(), irreps_out.uniform_mul()
    pairs = [(a, b) for a, ba in enumerate(irreps_in) for b, bb in enumerate(irreps_out) if ba.ir == bb.ir]
    paths = []
    for q, (a, b) in enumerate(pairs):
        if path_normalization == "element":
            fan = sum(irreps_in[a2].mul for a2, b2 in pairs if b2 == b)
        elif path_normalization == "path":
            fan = irreps_in[a].mul * len([1 for a2, b2 in pairs if b2 == b])
        else:
            fan = 1
        paths.append(LinearPath((q, a, b), scale * sqrt(1.0 / fan)))
    return LinearDescriptor([b.ir.dim for b in irreps_in], [b.ir.dim for b in irreps_out], u, v, paths)


# --------------------------------------------------------------------------- SymmetricContraction

@dataclass
class STCDescriptor:
    """Path table of a symmetric tensor contraction in the reference's padded layout
    (fasteq/ops/auto_schedule/models.py:49-66): row p = ``[a_1 .. a_n, d, v, pad ...]`` meaning
    ``out[v] += coeff[p] * x1[a_1] * .. * x1[a_n] * x0[d]`` with ``n = 1..3``."""
    paths: np.ndarray        # int64 [P, max_len], suffix padded with ``pad_value``
    coeffs: np.ndarray       # float64 [P]
    x1_segs: int
    x0_segs: int
    out_segs: int
    u_dim: int
    pad_value: int = -1
    weight_layout: Tuple[Tuple[int, int, int], ...] = ()  # per x0 segment: (degree, out block, basis index)
    irreps_in: Optional[Irreps] = None
    irreps_out: Optional[Irreps] = None

    @property
    def num_paths(self) -> int:
        return int(self.paths.shape[0])

    def tensors(self, dtype=None, device=None):
        """``(coeffs_tensor, paths_tensor [P, L], idx_lists_tensor [L, P])`` for ``fast_stc_uniform1d_jit``."""
        import torch
        dtype = dtype or torch.float32
        p = torch.as_tensor(self.paths, dtype=torch.int32, device=device)
        return torch.as_tensor(self.coeffs, dtype=dtype, device=device), p.contiguous(), p.t().contiguous()


def _independent_rows(mat: np.ndarray, tol: float = 1e-9) -> List[int]:
    """Greedy choice of linearly independent rows (modified Gram-Schmidt), keeping the originals
    so that the selected basis tensors stay as sparse as the Clebsch-Gordan products they come from."""
    chosen, basis = [], []
    for r in range(mat.shape[0]):
        v = mat[r].astype(np.float64).copy()
        n0 = np.linalg.norm(v)
        if n0 < tol:
            continue
        for b in basis:
            v -= (b @ v) * b
        for b in basis:  # second pass for stability
            v -= (b @ v) * b
        n = np.linalg.norm(v)
        if n > tol * max(1.0, n0) and n > 1e-7 * n0:
            basis.append(v / n)
            chosen.append(r)
    return chosen


def symmetric_contraction(irreps_in, irreps_out, degrees: Sequence[int] = (1, 2, 3)) -> STCDescriptor:
    """Symmetric contraction ``out_L = sum_nu sum_eta W[nu, L, eta] * B^{nu,L,eta}[a_1..a_nu, m] x[a_1]..x[a_nu]``.

    For every degree ``nu`` and output irrep ``L`` the basis tensors ``B`` span the equivariant,
    permutation-symmetric maps ``Sym^nu(V) -> L``, ``V`` being ``irreps_in`` at multiplicity one:
    iterated real Clebsch-Gordan couplings are symmetrised over the inputs and a maximal
    independent subset is kept (each scaled to unit Frobenius norm).  The role of
    cuEquivariance's ``symmetric_contraction`` descriptor the reference benches call
    (test/bench_tensor_product_uniform1d.py:185); the basis differs from that package's by an
    invertible mix of the weights, which the learned weights absorb.  Entries that are equal under
    index permutation are stored once with ``a_1 <= a_2 <= a_3`` and their multiplicity in the coefficient."""
    import itertools
    from math import factorial
    irreps_in, irreps_out = Irreps(irreps_in), Irreps(irreps_out)
    u = irreps_in.uniform_mul()
    if any(b.mul != u for b in irreps_out):
        raise ValueError("irreps_out must carry the multiplicity of irreps_in")
    in_off = irreps_in.segment_offsets()
    out_off = irreps_out.segment_offsets()
    n_in = irreps_in.num_segments
    blocks = [(b.ir.l, b.ir.p, o) for b, o in zip(irreps_in, in_off)]

    def embed(t: np.ndarray, offs: Sequence[int]) -> np.ndarray:
        full = np.zeros((n_in,) * len(offs) + (t.shape[-1],))
        sl = tuple(slice(o, o + s) for o, s in zip(offs, t.shape[:-1])) + (slice(None),)
        full[sl] = t
        return full

    paths, coeffs, layout = [], [], []
    for ob, (oblk, ooff) in enumerate(zip(irreps_out, out_off)):
        L, P = oblk.ir.l, oblk.ir.p
        for nu in degrees:
            cands = []
            if nu == 1:
                for (l1, p1, o1) in blocks:
                    if l1 == L and p1 == P:
                        cands.append(embed(np.eye(2 * L + 1)[:, :], [o1]))
            elif nu == 2:
                for (l1, p1, o1), (l2, p2, o2) in itertools.product(blocks, repeat=2):
                    if p1 * p2 == P and abs(l1 - l2) <= L <= l1 + l2:
                        cands.append(embed(wigner_3j(l1, l2, L), [o1, o2]))
            elif nu == 3:
                for (l1, p1, o1), (l2, p2, o2), (l3, p3, o3) in itertools.product(blocks, repeat=3):
                    if p1 * p2 * p3 != P:
                        continue
                    for l12 in range(abs(l1 - l2), l1 + l2 + 1):
                        if abs(l12 - l3) <= L <= l12 + l3:
                            t = np.einsum("abn,ncm->abcm", wigner_3j(l1, l2, l12), wigner_3j(l12, l3, L))
                            cands.append(embed(t, [o1, o2, o3]))
            else:
                raise NotImplementedError("degrees 1..3 are supported")
            if not cands:
                continue
            sym = []
            for t in cands:
                s = sum(np.transpose(t, perm + (nu,)) for perm in itertools.permutations(range(nu))) / factorial(nu)
                sym.append(s)
            mat = np.stack([s.reshape(-1) for s in sym])
            keep = _independent_rows(mat)
            for eta, r in enumerate(keep):
                b = sym[r] / np.linalg.norm(sym[r])
                d = len(layout)
                layout.append((nu, ob, eta))
                for idx in zip(*np.nonzero(np.abs(b) > 1e-12)):
                    a, m = idx[:-1], idx[-1]
                    if tuple(sorted(a)) != tuple(a):
                        continue  # the sorted representative carries the whole orbit
                    mult = len(set(itertools.permutations(a)))
                    paths.append(list(a) + [d, ooff + m])
                    coeffs.append(mult * b[idx])
    max_len = max(len(p) for p in paths)
    arr = np.full((len(paths), max_len), -1, dtype=np.int64)
    for r, p in enumerate(paths):
        arr[r, :len(p)] = p
    return STCDescriptor(arr, np.asarray(coeffs, dtype=np.float64), n_in, len(layout), irreps_out.num_segments, u,
                         -1, tuple(layout), irreps_in, irreps_out)
