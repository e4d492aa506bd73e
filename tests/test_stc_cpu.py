"""Symmetric-contraction tables and oracle on the CPU: equivariance, permutation symmetry, gradients."""
import numpy as np
import pytest

from fasteq_b200.descriptors import symmetric_contraction
from fasteq_b200.irreps import Irreps
from fasteq_b200.sh import spherical_harmonics_host
from oracle import stc_ref


def wigner_d_from_sh(l, R, rng):
    """D^l(R) with Y_l(R r) = D^l(R) Y_l(r), solved from sample points (consistent with the 3j tensors)."""
    pts = rng.normal(size=(8 * (2 * l + 1), 3))
    def Y(p):
        return spherical_harmonics_host(l, p, normalize=True)[:, l * l:(l + 1) * (l + 1)]
    D, *_ = np.linalg.lstsq(Y(pts), Y(pts @ R.T), rcond=None)
    return D.T


def random_rotation(rng):
    q, r = np.linalg.qr(rng.normal(size=(3, 3)))
    q *= np.sign(np.diag(r))
    if np.linalg.det(q) < 0:
        q[:, 0] *= -1
    return q


def block_d(irreps, R, rng):
    n = irreps.num_segments
    D = np.zeros((n, n))
    for b, o in zip(irreps, irreps.segment_offsets()):
        D[o:o + b.ir.dim, o:o + b.ir.dim] = wigner_d_from_sh(b.ir.l, R, rng)
    return D


@pytest.mark.parametrize("irr_in,irr_out", [("2x0e+2x1o+2x2e+2x3o", "2x0e+2x1o"), ("3x0e+3x1o+3x2e", "3x0e+3x1o+3x2e")])
def test_tables_are_equivariant_and_match_counts(irr_in, irr_out):
    rng = np.random.default_rng(0)
    d = symmetric_contraction(irr_in, irr_out)
    U = d.u_dim
    B, S = 6, 3
    x1 = rng.normal(size=(B, d.x1_segs, U)); x0 = rng.normal(size=(S, d.x0_segs, U)); i0 = rng.integers(0, S, B)
    out = stc_ref.stc_forward(x1, x0, i0, d.paths, d.coeffs, d.out_segs)
    R = random_rotation(rng)
    Din, Dout = block_d(Irreps(irr_in), R, rng), block_d(Irreps(irr_out), R, rng)
    out_rot = stc_ref.stc_forward(np.einsum("ab,nbu->nau", Din, x1), x0, i0, d.paths, d.coeffs, d.out_segs)
    np.testing.assert_allclose(out_rot, np.einsum("ab,nbu->nau", Dout, out), rtol=1e-9, atol=1e-9)
    # every row stores a sorted index tuple; weights of degree 1..3 all present
    for a, dd, v in stc_ref.split_paths(d.paths):
        assert list(a) == sorted(a) and 0 <= dd < d.x0_segs and 0 <= v < d.out_segs
    assert {n for n, _, _ in d.weight_layout} == {1, 2, 3}


def test_config1_table_size():
    d = symmetric_contraction("128x0e+128x1o+128x2e+128x3o", "128x0e+128x1o")
    assert (d.x1_segs, d.out_segs, d.u_dim) == (16, 4, 128)
    assert d.num_paths == 550 and d.x0_segs == 29


def test_oracle_gradients_by_finite_differences():
    rng = np.random.default_rng(1)
    d = symmetric_contraction("2x0e+2x1o", "2x0e+2x1o")
    B, S, U = 3, 2, 2
    x1 = rng.normal(size=(B, d.x1_segs, U)); x0 = rng.normal(size=(S, d.x0_segs, U)); i0 = np.array([1, 0, 1])
    r = rng.normal(size=(B, d.out_segs, U))
    f = lambda a, b: (stc_ref.stc_forward(a, b, i0, d.paths, d.coeffs, d.out_segs) * r).sum()
    gx1, gx0 = stc_ref.stc_backward(r, x1, x0, i0, d.paths, d.coeffs)
    eps = 1e-6
    for arr, g, which in ((x1, gx1, 0), (x0, gx0, 1)):
        for idx in [tuple(rng.integers(0, s) for s in arr.shape) for _ in range(6)]:
            p = arr.copy(); p[idx] += eps; m = arr.copy(); m[idx] -= eps
            fd = (f(p, x0) - f(m, x0)) / (2 * eps) if which == 0 else (f(x1, p) - f(x1, m)) / (2 * eps)
            assert abs(fd - g[idx]) < 1e-6 * max(1.0, abs(fd))


def _table_polynomials(d, nu, out_block, multisets):
    """Polynomial coefficients of the table's degree-``nu`` basis elements that feed output block ``out_block``:
    ``[n_basis, 2l+1, n_multisets]`` (one basis element per weight segment)."""
    index = {tuple(ms): t for t, ms in enumerate(multisets.tolist())}
    irr = d.irreps_out[out_block]
    off = d.irreps_out.segment_offsets()[out_block]
    segs = [s for s, (n, ob, _) in enumerate(d.weight_layout) if n == nu and ob == out_block]
    poly = np.zeros((len(segs), irr.ir.dim, len(multisets)))
    for (a, dd, v), c in zip(stc_ref.split_paths(d.paths), d.coeffs):
        if dd in segs:
            assert len(a) == nu and off <= v < off + irr.ir.dim
            poly[segs.index(dd), v - off, index[tuple(a)]] += c
    return poly


@pytest.mark.parametrize("case,irr_out", [("l3", "1x0e+1x1o"), ("l2", "1x0e+1x1o+1x2e")])
def test_table_spans_the_space_e3nn_reduces_to(golden, case, irr_out):
    """Pin of the basis itself: for every output irrep and degree, the table's basis elements and the rows of
    e3nn's ``ReducedTensorProducts`` change of basis (golden file, generated from the e3nn shipped inside the
    reference) span the SAME space of polynomial maps Sym^nu(V) -> irrep: same dimension, and stacking both
    adds no rank.  The operator built on this table therefore differs from one built on e3nn's / MACE's basis only
    by an invertible mix of the learned weights."""
    irr_in = str(golden[f"stc_{case}_irreps_in"][0])
    d = symmetric_contraction(irr_in, irr_out)
    for nu in (2, 3):
        multisets = golden[f"stc_{case}_nu{nu}_multisets"]
        for ob, blk in enumerate(Irreps(irr_out)):
            ref = golden[f"stc_{case}_nu{nu}_{blk.ir}"]
            ours = _table_polynomials(d, nu, ob, multisets)
            assert ours.shape[0] == ref.shape[0], (nu, str(blk.ir), ours.shape, ref.shape)      # multiplicity of the irrep
            flat = lambda p: p.reshape(p.shape[0], -1)
            rank = lambda m: int(np.linalg.matrix_rank(m, tol=1e-9))
            n = ref.shape[0]
            assert rank(flat(ref)) == n and rank(flat(ours)) == n
            assert rank(np.concatenate([flat(ref), flat(ours)])) == n
            # and explicitly: ours = M @ ref with a well-conditioned mixing matrix M
            M, res, *_ = np.linalg.lstsq(flat(ref).T, flat(ours).T, rcond=None)
            np.testing.assert_allclose(flat(ref).T @ M, flat(ours).T, atol=1e-10)
            assert np.linalg.cond(M) < 1e3
    # degree 1 is the identity on the matching irrep (scaled to unit Frobenius norm like every basis element)
    for s, (nu, ob, _) in enumerate(d.weight_layout):
        if nu == 1:
            rows = [(a, v, c) for (a, dd, v), c in zip(stc_ref.split_paths(d.paths), d.coeffs) if dd == s]
            dim = Irreps(irr_out)[ob].ir.dim
            assert len(rows) == dim and all(abs(c - dim ** -0.5) < 1e-12 for _, _, c in rows)
            assert sorted(v for _, v, _ in rows) == list(range(Irreps(irr_out).segment_offsets()[ob], Irreps(irr_out).segment_offsets()[ob] + dim))
