"""Symmetric tensor contraction (STC Uniform1D) oracle in numpy.

Restates the path semantics of fasteq/ops/auto_schedule/models.py:49-66 (padded rows
``[a.., d, v, pad]``) and the baseline loop fasteq/hip/src/stc_fwd.cpp:42-76:

    out[b, v, u] += c_p * prod_t x1[b, a_{p,t}, u] * x0[i0[b], d_p, u]

The reference's own tests hold no STC values.  The pins are: this path formula for the operator; for the
path TABLE, a span comparison with e3nn's ``ReducedTensorProducts`` (the e3nn shipped inside the reference's
model bundles, golden file ``tests/golden/e3nn_golden.npz``: per output irrep and degree the table's basis
elements and e3nn's change-of-basis rows span the same space) and an equivariance test.
"""
from __future__ import annotations

import numpy as np


def split_paths(paths, pad_value=-1):
    out = []
    for row in np.asarray(paths):
        vals = [int(v) for v in row if int(v) != pad_value]
        out.append((tuple(vals[:-2]), vals[-2], vals[-1]))
    return out


def stc_forward(x1, x0, i0, paths, coeffs, out_segs, pad_value=-1):
    """x1 [B, A, U], x0 [S, D, U], i0 [B] -> [B, V, U]."""
    x1 = x1.astype(np.float64); x0g = x0.astype(np.float64)[i0]
    out = np.zeros((x1.shape[0], out_segs, x1.shape[2]))
    for (a, d, v), c in zip(split_paths(paths, pad_value), coeffs):
        t = float(c) * x0g[:, d, :]
        for ai in a:
            t = t * x1[:, ai, :]
        out[:, v, :] += t
    return out


def stc_backward(grad_out, x1, x0, i0, paths, coeffs, pad_value=-1):
    """(grad_x1 [B, A, U], grad_x0 [S, D, U]) of sum(out * grad_out)."""
    x1 = x1.astype(np.float64); x0 = x0.astype(np.float64); go = grad_out.astype(np.float64)
    x0g = x0[i0]
    gx1 = np.zeros_like(x1); gx0g = np.zeros_like(x0g)
    for (a, d, v), c in zip(split_paths(paths, pad_value), coeffs):
        g = float(c) * go[:, v, :]
        prod_all = np.ones_like(g)
        for ai in a:
            prod_all = prod_all * x1[:, ai, :]
        gx0g[:, d, :] += g * prod_all
        for t, at in enumerate(a):
            others = g * x0g[:, d, :]
            for s, as_ in enumerate(a):
                if s != t:
                    others = others * x1[:, as_, :]
            gx1[:, at, :] += others
    gx0 = np.zeros_like(x0)
    np.add.at(gx0, i0, gx0g)
    return gx1, gx0
