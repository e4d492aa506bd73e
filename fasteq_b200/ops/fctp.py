"""``fast_fctp``: drop-in for fasteq/ops/fctp.py:852 -- the fully connected tensor product of node
features with one-hot species attributes (MACE's species-dependent skip connection):

    out[b, k, :] = cg_val_0 * val_for_k[k] * x[b, i_for_k[k], :] @ w[p_for_k[k], :, species(b), :]

with ``species(b) = argmax(y[b])``, ``x [B, I_total * U]``, ``w`` of ``P * U * V * W`` elements viewed
``[P, U, V, W]``, ``out [B, K_total * W]``; output rows with ``i_for_k[k] < 0`` are zero
(reference: fasteq/ops/fctp.py:643-736; value semantics pinned by test/smoke_eqlinear_other_ops.py:38-56).

A one-hot second operand makes the product a species-indexed SO3Linear.  Nodes are grouped by species and
every group goes through the SO3Linear entry points of the C ABI (tcgen05 3xTF32 for FP32 data, FP64 FMA
for doubles): ``fasteq_eqlinear_forward`` for the values, ``_dgrad`` for grad_x and ``_wgrad`` for grad_w.
``y`` gets no gradient (it enters through an argmax, as in the reference).  First order only.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Tuple

import torch

from .. import _cabi
from .eqlinear import _core, _make_problem

__all__ = ["fast_fctp", "fctp_species_groups"]

_PLAN_CACHE: Dict[Tuple, Tuple] = {}


def _host_list(t, n, name):
    v = t.detach().cpu().tolist() if isinstance(t, torch.Tensor) else list(t)
    if len(v) < n:
        raise ValueError(f"fast_fctp: {name} must have one entry per output row ({n}), got {len(v)}")
    return v[:n]


def _runs(meta) -> Tuple[List[Tuple[int, int, int, int]], List[float], List[int]]:
    """Maximal runs of consecutive output rows that read consecutive input rows through one weight path
    with one coefficient: ``[(in_row, out_row, run, rows)]``, their coefficients and weight paths."""
    K = int(meta["K_total"])
    key = tuple(id(meta[k]) for k in ("i_for_k", "p_for_k", "val_for_k")) + (K, float(meta["cg_val_0"]))
    hit = _PLAN_CACHE.get(key)
    if hit is not None:
        return hit[0]
    i_k = [int(v) for v in _host_list(meta["i_for_k"], K, "i_for_k")]
    p_k = [int(v) for v in _host_list(meta["p_for_k"], K, "p_for_k")]
    v_k = [float(v) for v in _host_list(meta["val_for_k"], K, "val_for_k")]
    alpha = float(meta["cg_val_0"])
    mapping, coeff, paths = [], [], []
    k = 0
    while k < K:
        if i_k[k] < 0:
            k += 1
            continue
        n = 1
        while (k + n < K and i_k[k + n] == i_k[k] + n and p_k[k + n] == p_k[k] and v_k[k + n] == v_k[k]):
            n += 1
        mapping.append((i_k[k], k, len(mapping), n))
        coeff.append(alpha * v_k[k])
        paths.append(p_k[k])
        k += n
    if not mapping:
        raise ValueError("fast_fctp: no output row reads an input row")
    if len(mapping) > 64:
        raise NotImplementedError("fast_fctp: more than 64 (input row, weight path) runs")
    if len(_PLAN_CACHE) > 64:
        _PLAN_CACHE.clear()
    out = (mapping, coeff, paths)
    _PLAN_CACHE[key] = (out, [meta[k] for k in ("i_for_k", "p_for_k", "val_for_k")])   # keep the ids alive
    return out


def fctp_species_groups(y: torch.Tensor):
    """``(order, counts)``: the permutation that sorts the nodes by species ``argmax(y[b])`` and the host list of
    nodes per species.  Computing it costs one host synchronisation; the species of a structure do not change from
    step to step, so a caller can compute it once and pass it as ``meta["species_groups"]`` to ``fast_fctp``, which
    then makes no host synchronisation at all."""
    vstar = torch.argmax(y, dim=1)
    order = torch.argsort(vstar, stable=True)
    counts = torch.bincount(vstar, minlength=y.shape[1]).tolist()
    return order, counts


def _species_groups(y: torch.Tensor, V: int, meta):
    pre = meta.get("species_groups")
    if pre is not None:
        order, counts = pre
        counts = [int(c) for c in counts]
        if len(counts) != V or sum(counts) != y.shape[0] or order.numel() != y.shape[0]:
            raise ValueError("fast_fctp: meta['species_groups'] does not match y")
        return order.to(y.device), counts
    return fctp_species_groups(y)                                   # one host sync per call


def _precision(dtype) -> int:
    if dtype == torch.float64:
        return 2
    if dtype == torch.float32:
        return 0
    raise ValueError(f"fast_fctp: only float32 and float64 are supported; got {dtype}")


class FastFullyConnectedTensorProductPathFused(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, x, y, meta):
        if not (w.is_cuda and x.is_cuda and y.is_cuda):
            raise RuntimeError("fast_fctp: w, x and y must be CUDA tensors: fasteq_b200 has no CPU path")
        U, V, W, P = int(meta["U"]), int(meta["V"]), int(meta["W"]), int(meta["P"])
        K, I = int(meta["K_total"]), int(meta["I_total"])
        B = x.shape[0]
        if x.numel() != B * I * U or w.numel() != P * U * V * W or y.shape != (B, V) or x.dtype != w.dtype:
            raise ValueError("fast_fctp: operand shapes do not match the meta (x [B, I*U], w [P, U, V, W], y [B, V])")
        mapping, coeff, paths = _runs(meta)
        prec = _precision(x.dtype)
        order, counts = _species_groups(y, V, meta)
        xs = x.reshape(B, I, U)[order].contiguous()
        w4 = w.reshape(P, U, V, W)
        pidx = torch.tensor(paths, device=w.device)
        outs = torch.empty((B, K, W), dtype=x.dtype, device=x.device)
        lib = _core()
        ws, start = {}, 0
        with torch.cuda.device(x.device):
            stream = torch.cuda.current_stream(x.device).cuda_stream
            for s, n in enumerate(counts):
                if n == 0:
                    continue
                ws[s] = w4[:, :, s, :][pidx].contiguous()                       # [runs, U, W]
                prob = _make_problem(mapping, coeff, U, W, I, K, n, prec)
                _cabi.check(lib.fasteq_eqlinear_forward(C.byref(prob), ws[s].data_ptr(), xs[start:start + n].data_ptr(),
                                                        outs[start:start + n].data_ptr(), stream), lib, "fasteq_eqlinear_forward")
                start += n
        out = torch.empty_like(outs)
        out[order] = outs
        ctx.save_for_backward(xs if ctx.needs_input_grad[0] else None, order, pidx, *[ws[s] for s in sorted(ws)])
        ctx.cfg = (mapping, coeff, U, V, W, P, K, I, prec, counts, tuple(w.shape), tuple(x.shape))
        return out.reshape(B, K * W)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        xs, order, pidx, *wlist = ctx.saved_tensors
        mapping, coeff, U, V, W, P, K, I, prec, counts, w_shape, x_shape = ctx.cfg
        need_w, need_x = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if not (need_w or need_x):
            return None, None, None, None
        B = grad_out.shape[0]
        gs = grad_out.reshape(B, K, W)[order].contiguous()
        lib = _core()
        gxs = torch.empty((B, I, U), dtype=gs.dtype, device=gs.device) if need_x else None
        gw4 = torch.zeros((P, U, V, W), dtype=gs.dtype, device=gs.device) if need_w else None
        start, wi = 0, 0
        with torch.cuda.device(gs.device):
            stream = torch.cuda.current_stream(gs.device).cuda_stream
            for s, n in enumerate(counts):
                if n == 0:
                    continue
                prob = _make_problem(mapping, coeff, U, W, I, K, n, prec)
                if need_x:
                    _cabi.check(lib.fasteq_eqlinear_dgrad(C.byref(prob), wlist[wi].data_ptr(), gs[start:start + n].data_ptr(),
                                                          gxs[start:start + n].data_ptr(), stream), lib, "fasteq_eqlinear_dgrad")
                if need_w:
                    gws = torch.empty((len(mapping), U, W), dtype=gs.dtype, device=gs.device)
                    _cabi.check(lib.fasteq_eqlinear_wgrad(C.byref(prob), xs[start:start + n].data_ptr(), gs[start:start + n].data_ptr(),
                                                          gws.data_ptr(), stream), lib, "fasteq_eqlinear_wgrad")
                    gw4[:, :, s, :].index_add_(0, pidx, gws)                     # several runs may share a weight path
                start += n
                wi += 1
        gx = None
        if need_x:
            gx = torch.empty_like(gxs)
            gx[order] = gxs
            gx = gx.reshape(x_shape)
        return (gw4.reshape(w_shape) if need_w else None), gx, None, None


def fast_fctp(w, x, y, meta):
    """See the module docstring; same call as the reference's ``fast_fctp(w, x, y, meta)``."""
    return FastFullyConnectedTensorProductPathFused.apply(w, x, y, meta)
