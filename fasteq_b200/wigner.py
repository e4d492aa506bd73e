"""Real-basis Wigner 3j symbols (Clebsch-Gordan tensors of SO(3)).

The tensor ``wigner_3j(l1, l2, l3)[m1, m2, m3]`` is the unique (up to sign)
SO(3)-invariant 3-tensor on real irreps ``l1 x l2 x l3`` with unit Frobenius
norm.  The sign and basis conventions follow e3nn so that path tables built
from it reproduce e3nn's ``TensorProduct`` numerically (reference copy of that
convention: e3nn/o3/_wigner.py:31-47 for the real<->complex basis change and
:147-162 for the projection; vendored in the reference's model bundles).

Algorithm (published, restated here): complex SU(2) Clebsch-Gordan coefficients
from Racah's closed form in exact rational arithmetic, conjugated into the real
basis ``Y_{l,-m}.. Y_{l,m}`` with the ``(-i)^l`` phase that makes the result
real, then normalised.
"""
from __future__ import annotations

import functools
from fractions import Fraction
from math import factorial, sqrt

import numpy as np


def _racah_cg(j1: int, m1: int, j2: int, m2: int, j3: int, m3: int) -> float:
    """<j1 m1; j2 m2 | j3 m3> for integer spins (Racah's formula)."""
    if m1 + m2 != m3 or not (abs(j1 - j2) <= j3 <= j1 + j2):
        return 0.0
    if abs(m1) > j1 or abs(m2) > j2 or abs(m3) > j3:
        return 0.0
    f = factorial
    pref = Fraction(
        (2 * j3 + 1) * f(j1 + j2 - j3) * f(j1 - j2 + j3) * f(-j1 + j2 + j3),
        f(j1 + j2 + j3 + 1),
    ) * (f(j1 + m1) * f(j1 - m1) * f(j2 + m2) * f(j2 - m2) * f(j3 + m3) * f(j3 - m3))
    kmin = max(0, j2 - j3 - m1, j1 - j3 + m2)
    kmax = min(j1 + j2 - j3, j1 - m1, j2 + m2)
    s = Fraction(0)
    for k in range(kmin, kmax + 1):
        s += Fraction(
            (-1) ** k,
            f(k) * f(j1 + j2 - j3 - k) * f(j1 - m1 - k) * f(j2 + m2 - k) * f(j3 - j2 + m1 + k) * f(j3 - j1 - m2 + k),
        )
    return float(s) * sqrt(float(pref))


def real_to_complex(l: int) -> np.ndarray:
    """Unitary Q with (complex SH vector) = Q @ (real SH vector), including the (-i)^l phase."""
    q = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
    r = 1.0 / sqrt(2.0)
    for m in range(1, l + 1):
        # negative complex order -m
        q[l - m, l + m] = r
        q[l - m, l - m] = -1j * r
        # positive complex order +m
        q[l + m, l + m] = (-1) ** m * r
        q[l + m, l - m] = 1j * (-1) ** m * r
    q[l, l] = 1.0
    return ((-1j) ** l) * q


@functools.lru_cache(maxsize=None)
def _wigner_3j_cached(l1: int, l2: int, l3: int) -> np.ndarray:
    cg = np.zeros((2 * l1 + 1, 2 * l2 + 1, 2 * l3 + 1), dtype=np.complex128)
    for m1 in range(-l1, l1 + 1):
        for m2 in range(-l2, l2 + 1):
            m3 = m1 + m2
            if abs(m3) <= l3:
                cg[l1 + m1, l2 + m2, l3 + m3] = _racah_cg(l1, m1, l2, m2, l3, m3)
    q1, q2, q3 = real_to_complex(l1), real_to_complex(l2), real_to_complex(l3)
    c = np.einsum("ij,kl,mn,ikn->jlm", q1, q2, np.conj(q3.T), cg)
    if np.abs(c.imag).max() > 1e-9:
        raise AssertionError("real-basis Clebsch-Gordan tensor has an imaginary part")
    c = np.ascontiguousarray(c.real)
    c /= np.linalg.norm(c)
    c[np.abs(c) < 1e-14] = 0.0
    c.setflags(write=False)
    return c


def wigner_3j(l1: int, l2: int, l3: int) -> np.ndarray:
    """float64 array ``[2l1+1, 2l2+1, 2l3+1]``; zero-size selection rules raise."""
    if not (abs(l1 - l2) <= l3 <= l1 + l2):
        raise ValueError(f"({l1},{l2},{l3}) violates the triangle rule")
    return _wigner_3j_cached(int(l1), int(l2), int(l3)).copy()
