"""Path-level Uniform1D (channelwise tensor product) oracle in numpy.

Restates fasteq/ops/auto_schedule/models.py:93-113 (forward term) and :142-172
(gradient terms) with the row indexing of
fasteq/ops/auto_schedule/uniform1d_forward.py:408-421:

    out[r_out, v, u] += c_p * w[r_w, i_p, u] * x[r_x, j_p, u] * y[r_y, k_p, u or 0]

``r_x = src[e]`` when x is gathered, ``r_y = src[e]`` when y is gathered,
``r_out = dst[e]`` when the output is scattered (summed over edges), ``r_w = 0``
when the weights are shared (one row), otherwise the edge id.
"""
from __future__ import annotations

import numpy as np


def _rows(t, idx, E):
    if idx is not None:
        return t[idx]
    if t.shape[0] == 1 and E != 1:
        return np.broadcast_to(t, (E,) + t.shape[1:])
    return t


def uniform1d_forward(w, x, y, paths, coeffs, out_seg_num, src_x=None, src_y=None, dst=None, num_out_rows=None):
    """w [E|1, I, U], x [*, J, U], y [*, K, U|1]; returns [rows, V, U] in the dtype of ``x``."""
    E = (dst if dst is not None else src_x if src_x is not None else src_y if src_y is not None else x).shape[0]
    ww, xx, yy = _rows(w, None, E), _rows(x, src_x, E), _rows(y, src_y, E)
    U = x.shape[2]
    acc = np.zeros((E, out_seg_num, U), dtype=np.float64)
    for (i, j, k, v), c in zip(paths, coeffs):
        acc[:, v, :] += float(c) * ww[:, i, :].astype(np.float64) * xx[:, j, :] * yy[:, k, :]
    if dst is not None:
        out = np.zeros((num_out_rows, out_seg_num, U), dtype=np.float64)
        np.add.at(out, dst, acc)
        acc = out
    return acc.astype(x.dtype)


def uniform1d_backward(grad_out, w, x, y, paths, coeffs, src_x=None, src_y=None, dst=None):
    """Gradients (gw, gx, gy) of sum(out * grad_out); accumulation in float64."""
    E = (dst if dst is not None else src_x if src_x is not None else src_y if src_y is not None else x).shape[0]
    ww, xx, yy = _rows(w, None, E), _rows(x, src_x, E), _rows(y, src_y, E)
    go = grad_out[dst] if dst is not None else grad_out
    go = go.astype(np.float64)
    gw_e = np.zeros((E,) + w.shape[1:], dtype=np.float64)
    gx_e = np.zeros((E,) + x.shape[1:], dtype=np.float64)
    gy_e = np.zeros((E,) + y.shape[1:], dtype=np.float64)
    scalar_y = y.shape[2] == 1
    for (i, j, k, v), c in zip(paths, coeffs):
        c = float(c)
        g = go[:, v, :]
        gw_e[:, i, :] += c * g * xx[:, j, :] * yy[:, k, :]
        gx_e[:, j, :] += c * g * ww[:, i, :] * yy[:, k, :]
        t = c * g * ww[:, i, :] * xx[:, j, :]
        gy_e[:, k, :] += t.sum(axis=1, keepdims=True) if scalar_y else t
    gw = gw_e.sum(axis=0, keepdims=True) if (w.shape[0] == 1 and E != 1) else gw_e
    if src_x is not None:
        gx = np.zeros(x.shape, dtype=np.float64); np.add.at(gx, src_x, gx_e)
    else:
        gx = gx_e
    if src_y is not None:
        gy = np.zeros(y.shape, dtype=np.float64); np.add.at(gy, src_y, gy_e)
    else:
        gy = gy_e
    return gw.astype(w.dtype), gx.astype(x.dtype), gy.astype(y.dtype)
