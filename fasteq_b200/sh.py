"""Real spherical harmonics as explicit polynomials (e3nn convention, component normalisation).

``Y_0 = 1``, ``Y_1 = sqrt(3) (x, y, z)`` and ``Y_l = s_l * C^{l-1,1,l} . (Y_{l-1} (x) Y_1)`` with
the real Wigner 3j tensor and ``s_l > 0`` fixed by ``|Y_l|^2 = 2l+1`` on the unit sphere;
this reproduces e3nn's ``spherical_harmonics`` (the reference embeds the same functions as a
polynomial table, fasteq/triton/spherical_harmonics.py:66-238).  The polynomials are generated
here from the 3j tensors; they feed both a numpy evaluator for input preparation and the CUDA
emitters for the spherical-harmonics kernels.
"""
from __future__ import annotations

import functools
from math import sqrt
from typing import Dict, List, Tuple

import numpy as np

from .wigner import wigner_3j

Poly = Dict[Tuple[int, int, int], float]  # exponents of (x, y, z) -> coefficient


def _mul(a: Poly, b: Poly, scale: float = 1.0) -> Poly:
    out: Poly = {}
    for (ea, ca) in a.items():
        for (eb, cb) in b.items():
            e = (ea[0] + eb[0], ea[1] + eb[1], ea[2] + eb[2])
            out[e] = out.get(e, 0.0) + scale * ca * cb
    return out


def _add(dst: Poly, src: Poly) -> None:
    for e, c in src.items():
        dst[e] = dst.get(e, 0.0) + c


def _eval(p: Poly, v) -> float:
    return sum(c * v[0] ** e[0] * v[1] ** e[1] * v[2] ** e[2] for e, c in p.items())


@functools.lru_cache(maxsize=None)
def sh_polynomials(lmax: int) -> Tuple[Tuple[Poly, ...], ...]:
    """``result[l][m]`` is the homogeneous degree-l polynomial of Y_{l,m} (m index 0..2l)."""
    s3 = sqrt(3.0)
    ys: List[List[Poly]] = [[{(0, 0, 0): 1.0}]]
    if lmax >= 1:
        ys.append([{(1, 0, 0): s3}, {(0, 1, 0): s3}, {(0, 0, 1): s3}])
    probe = (0.3, 0.5, sqrt(1.0 - 0.09 - 0.25))
    for l in range(2, lmax + 1):
        c = wigner_3j(l - 1, 1, l)
        raw: List[Poly] = []
        for m3 in range(2 * l + 1):
            acc: Poly = {}
            for m1 in range(2 * l - 1):
                for m2 in range(3):
                    if c[m1, m2, m3] != 0.0:
                        _add(acc, _mul(ys[l - 1][m1], ys[1][m2], float(c[m1, m2, m3])))
            raw.append(acc)
        norm2 = sum(_eval(p, probe) ** 2 for p in raw)
        s = sqrt((2 * l + 1) / norm2)
        ys.append([{e: s * cf for e, cf in p.items() if abs(s * cf) > 1e-13} for p in raw])
    return tuple(tuple(level) for level in ys)


def derivative(p: Poly, axis: int) -> Poly:
    out: Poly = {}
    for e, c in p.items():
        if e[axis] > 0:
            ne = list(e); ne[axis] -= 1
            out[tuple(ne)] = out.get(tuple(ne), 0.0) + c * e[axis]
    return out


def spherical_harmonics_host(lmax: int, vec: np.ndarray, normalize: bool = True) -> np.ndarray:
    """numpy evaluation: ``[..., 3] -> [..., (lmax+1)^2]`` (component normalisation)."""
    v = np.asarray(vec, dtype=np.float64)
    if normalize:
        v = v / np.maximum(np.linalg.norm(v, axis=-1, keepdims=True), 1e-12)
    x, y, z = v[..., 0], v[..., 1], v[..., 2]
    pw = lambda a, n: np.ones_like(a) if n == 0 else a ** n
    cols = []
    for level in sh_polynomials(lmax):
        for p in level:
            acc = np.zeros_like(x)
            for e, c in p.items():
                acc = acc + c * pw(x, e[0]) * pw(y, e[1]) * pw(z, e[2])
            cols.append(acc)
    return np.stack(cols, axis=-1)
