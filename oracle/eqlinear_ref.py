"""SO3Linear ("eqlinear", uv,iu,iv) oracle in numpy.

Restates the direct-loop reference of the reference's own test (test/test_eqlinear.py:38-69):
paths with equal ``i`` that are adjacent form a run and accumulate into the same output rows

    out[b, j0(run) + t, :] = sum_{q in run} cg[q] * x[b, in_prefix[q] + t, :] @ W[q]

and the general path mapping ``(input_row, output_row, weight_path, rows)`` of
fasteq/cuda/src/eqlinear/common/eqlinear_common.h:32-37.
"""
from __future__ import annotations

import numpy as np


def runs_of(i_dims):
    runs, p = [], 0
    while p < len(i_dims):
        q = p + 1
        while q < len(i_dims) and i_dims[q] == i_dims[p]:
            q += 1
        runs.append((i_dims[p], p, q - p))
        p = q
    return runs


def out_rows(i_dims) -> int:
    return sum(i for i, _, _ in runs_of(i_dims))


def mapping_from_i_dims(i_dims):
    """[(in_row, out_row, weight_path, rows)] for the dense run-length layout."""
    m, in_row, out_row = [], 0, 0
    for i, p0, count in runs_of(i_dims):
        for q in range(p0, p0 + count):
            m.append((in_row, out_row, q, i))
            in_row += i
        out_row += i
    return m


def eqlinear_forward(x, w, mapping, cg, out_rows_total):
    """x [B, I, U], w [P, U, V] -> [B, J, V]; float64 accumulation, result in x's dtype."""
    B, _, U = x.shape
    V = w.shape[2]
    out = np.zeros((B, out_rows_total, V), dtype=np.float64)
    for (ir, orow, wp, rows), c in zip(mapping, cg):
        out[:, orow:orow + rows, :] += float(c) * (x[:, ir:ir + rows, :].astype(np.float64) @ w[wp].astype(np.float64))
    return out.astype(x.dtype)


def eqlinear_dgrad(grad_out, w, mapping, cg, in_rows_total):
    B, _, V = grad_out.shape
    U = w.shape[1]
    gx = np.zeros((B, in_rows_total, U), dtype=np.float64)
    for (ir, orow, wp, rows), c in zip(mapping, cg):
        gx[:, ir:ir + rows, :] += float(c) * (grad_out[:, orow:orow + rows, :].astype(np.float64) @ w[wp].astype(np.float64).T)
    return gx.astype(grad_out.dtype)


def eqlinear_wgrad(x, grad_out, mapping, cg, num_weight_blocks):
    """grad_w[wp] = cg * sum_b sum_t x[b, in+t, :]^T grad_out[b, out+t, :] -> [P, U, V] (float64).
    The adjoint of ``eqlinear_forward`` in ``w``; the reference's operator returns none
    (fasteq/ops/auto_schedule/eqlinear_runtime.py:104), so this follows from the forward formula."""
    U, V = x.shape[2], grad_out.shape[2]
    gw = np.zeros((num_weight_blocks, U, V), dtype=np.float64)
    for (ir, orow, wp, rows), c in zip(mapping, cg):
        xs = x[:, ir:ir + rows, :].astype(np.float64).reshape(-1, U)
        gs = grad_out[:, orow:orow + rows, :].astype(np.float64).reshape(-1, V)
        gw[wp] += float(c) * (xs.T @ gs)
    return gw
