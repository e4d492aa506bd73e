"""``fast_equi_linear``: drop-in for fasteq/ops/eqlinear.py:44-65 (forward and grad_x of the
uniform ``uv,iu,iv`` SO3Linear).

``x`` is ``[B, I*U]`` (viewed ``[B, I, U]``, irrep-row major, channel minor), ``w`` holds ``P*U*V``
elements (viewed ``[P, U, V]``), the result is ``[B, J*V]``.  Precision routing as in the reference
(fasteq/ops/eqlinear.py:24-41): float64 -> FP64; float32 -> ``compute_precision`` ``None`` /
``"tf32"`` / ``"tf32x3"`` (error bound of 3xTF32) or ``"fp32"``; anything else raises ``ValueError``.
The reference returns no gradient for ``w`` (eqlinear_runtime.py:104); here ``w`` gets one when it
requires grad (``fasteq_eqlinear_wgrad``, FP32 / FP64 FMA arithmetic), so the mixing weights can be trained.
Unsupported descriptors raise; there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import operator
from typing import Dict, List, Tuple

import torch

from .. import _cabi
from . import _prepared

__all__ = ["fast_equi_linear", "eqlinear_clear_plan_cache", "eqlinear_set_plan_cache", "eqlinear_debug_info"]

_TF32, _FP32, _FP64 = 0, 1, 2


class _Problem(C.Structure):
    _fields_ = [("precision", C.c_int32), ("u", C.c_int32), ("v", C.c_int32), ("in_rows", C.c_int32),
                ("out_rows", C.c_int32), ("num_paths", C.c_int32), ("batch", C.c_int64),
                ("in_row", C.POINTER(C.c_int32)), ("out_row", C.POINTER(C.c_int32)), ("rows", C.POINTER(C.c_int32)),
                ("coeff", C.POINTER(C.c_double))]


def _resolve_precision(x, w, compute_precision) -> int:
    if x.dtype != w.dtype:
        raise ValueError(f"eqlinear: x and w must have the same dtype; got {x.dtype} and {w.dtype}")
    if x.dtype == torch.float64:
        return _FP64
    if x.dtype != torch.float32:
        raise ValueError(f"eqlinear: only float32 and float64 are supported; got {x.dtype}")
    if compute_precision is None:
        return _TF32
    value = compute_precision.lower() if isinstance(compute_precision, str) else compute_precision
    if value in ("tf32", "tf32x3"):
        return _TF32
    if value == "fp32":
        return _FP32
    raise ValueError(f"eqlinear: compute_precision must be None, 'tf32', or 'fp32'; got {compute_precision!r}")


def _segments(operand) -> Tuple[Tuple[int, ...], ...]:
    segs = getattr(operand, "segments", operand)
    return tuple(tuple(operator.index(v) for v in seg) for seg in segs)


def _single(descriptor, name: str) -> int:
    vals = {operator.index(v) for v in descriptor.get_dims(name)}
    if len(vals) != 1:
        raise ValueError(f"eqlinear: descriptor must have exactly one {name!r} dimension, got {sorted(vals)}")
    return vals.pop()


def _descriptor_problem(descriptor):
    """(mapping [(in_row, out_row, weight_path, rows)], coefficients, u, v, I, J).

    Accepts both descriptor flavours the reference accepts (eqlinear_descriptor.py:228-310): paths
    with ``indices`` (explicit segment mapping) and index-free paths over a dense run-length layout."""
    if len(descriptor.operands) != 3:
        raise ValueError("eqlinear requires exactly three operands: uv, iu, iv")
    paths = list(descriptor.paths)
    if not paths:
        raise ValueError("eqlinear descriptor must contain at least one path")
    in_seg, out_seg = _segments(descriptor.operands[1]), _segments(descriptor.operands[2])
    u, v = _single(descriptor, "u"), _single(descriptor, "v")
    coeff = []
    for p in paths:
        c = p.coefficients
        c = float(c.item() if hasattr(c, "item") else c)
        coeff.append(c)
    if all(hasattr(p, "indices") for p in paths):
        subs = getattr(descriptor, "operands_and_subscripts", None)
        if subs is not None and tuple(s for _, s in subs) != ("uv", "iu", "iv") or getattr(descriptor, "coefficient_subscripts", ""):
            raise NotImplementedError("eqlinear requires scalar coefficients and uv,iu,iv subscripts")
        w_seg = _segments(descriptor.operands[0])
        if len(w_seg) != len(paths):
            raise NotImplementedError("eqlinear requires one weight block per path")
        if (any(len(s) != 2 or s[1] != u for s in in_seg) or any(len(s) != 2 or s[1] != v for s in out_seg)
                or any(tuple(s) != (u, v) for s in w_seg)):
            raise ValueError("eqlinear: inconsistent uniform operand segment dimensions")
        in_off, out_off, I, J = [], [], 0, 0
        for s in in_seg:
            in_off.append(I); I += s[0]
        for s in out_seg:
            out_off.append(J); J += s[0]
        mapping = []
        for p in paths:
            wp, ip, op = (operator.index(i) for i in p.indices)
            if not (0 <= wp < len(w_seg) and 0 <= ip < len(in_seg) and 0 <= op < len(out_seg)):
                raise ValueError("eqlinear: invalid descriptor path index")
            i = in_seg[ip][0]
            if i <= 0 or i != out_seg[op][0]:
                raise ValueError("eqlinear: path i dimensions disagree")
            mapping.append((in_off[ip], out_off[op], wp, i))
        return mapping, coeff, u, v, I, J
    i_dims = tuple(s[0] for s in in_seg)
    if len(i_dims) != len(paths):
        raise ValueError(f"eqlinear: derived {len(i_dims)} i_dims for {len(paths)} paths")
    mapping, in_row, out_row, prev = [], 0, 0, None
    for q, i in enumerate(i_dims):
        if prev is not None and prev != i:
            out_row += prev
        mapping.append((in_row, out_row, q, i))
        in_row += i
        prev = i
    J = out_row + i_dims[-1]
    if J != sum(s[0] for s in out_seg):
        raise NotImplementedError(f"eqlinear: output segments imply {sum(s[0] for s in out_seg)} rows, kernel grouping implies {J}")
    return mapping, coeff, u, v, in_row, J


_core_ready = False


def _core():
    global _core_ready
    lib = _cabi.core()
    if not _core_ready:
        lib.fasteq_eqlinear_forward.argtypes = [C.POINTER(_Problem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.fasteq_eqlinear_dgrad.argtypes = [C.POINTER(_Problem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.fasteq_eqlinear_wgrad.argtypes = [C.POINTER(_Problem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.fasteq_eqlinear_pack.argtypes = [C.POINTER(_Problem), C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.fasteq_eqlinear_forward_packed.argtypes = [C.POINTER(_Problem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.fasteq_eqlinear_dgrad_packed.argtypes = [C.POINTER(_Problem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        _core_ready = True
    return lib


def _make_problem(mapping, coeff, u, v, I, J, batch, precision):
    P = len(mapping)
    arr = lambda vals: (C.c_int32 * P)(*vals)
    prob = _Problem(precision, u, v, I, J, P, batch, arr([m[0] for m in mapping]), arr([m[1] for m in mapping]),
                    arr([m[3] for m in mapping]), (C.c_double * P)(*coeff))
    return prob


def _check_inputs(w, x, u, v, I, P):
    if not (x.is_cuda and w.is_cuda):
        raise RuntimeError("eqlinear: x and w must be CUDA tensors: fasteq_b200 has no CPU path")
    if x.shape[-1] != I * u and x.numel() % (I * u) != 0:
        raise ValueError(f"eqlinear: x has {x.numel()} elements, not a multiple of I*U = {I * u}")
    if w.numel() != P * u * v:
        raise ValueError(f"eqlinear: w has {w.numel()} elements, expected P*U*V = {P * u * v}")


def _order_weights(w3d, mapping):
    """Weight block of path q must sit at index q: reorder only if the descriptor says otherwise."""
    wps = [m[2] for m in mapping]
    if wps == list(range(len(wps))):
        return w3d
    return w3d[torch.tensor(wps, device=w3d.device)].contiguous()


def _packed_weights(w, w3, geom_key, prob, dgrad: bool, lib, stream):
    """Pre-scaled, K-major, TF32-split weight blocks of this problem and direction (cached per weight version)."""
    def build():
        packed = torch.empty(2 * w3.numel(), dtype=torch.float32, device=w3.device)
        rc = lib.fasteq_eqlinear_pack(C.byref(prob), 1 if dgrad else 0, w3.data_ptr(), packed.data_ptr(), stream)
        if rc == 1:      # FASTEQ_UNSUPPORTED
            return None
        _cabi.check(rc, lib, "fasteq_eqlinear_pack")
        return packed
    return _prepared.get((w,), ("eqlinear", geom_key, dgrad), build)


def _run(lib, prob, w, w3, a, c, geom_key, precision, dgrad: bool, stream):
    """One forward / grad_x launch: through prepared weights when the tensor-core path takes the problem."""
    if precision == _TF32:
        packed = _packed_weights(w, w3, geom_key, prob, dgrad, lib, stream)
        if packed is not None:
            fn = lib.fasteq_eqlinear_dgrad_packed if dgrad else lib.fasteq_eqlinear_forward_packed
            rc = fn(C.byref(prob), packed.data_ptr(), a.data_ptr(), c.data_ptr(), stream)
            if rc != 1:
                _cabi.check(rc, lib, "fasteq_eqlinear_dgrad_packed" if dgrad else "fasteq_eqlinear_forward_packed")
                return
    fn = lib.fasteq_eqlinear_dgrad if dgrad else lib.fasteq_eqlinear_forward
    _cabi.check(fn(C.byref(prob), w3.data_ptr(), a.data_ptr(), c.data_ptr(), stream), lib,
                "fasteq_eqlinear_dgrad" if dgrad else "fasteq_eqlinear_forward")


class _Plan:
    """One operator call resolved: geometry, precision and the three launches over the caller's tensors.
    ``w`` always has the caller's layout ``[P, u, v]`` flattened; ``x`` is ``[batch, I * u]``, ``g`` ``[batch, J * v]``."""

    def __init__(self, geom, precision, batch, w_shape):
        self.geom, self.precision, self.batch, self.w_shape = geom, precision, batch, tuple(w_shape)
        mapping, coeff, u, v, I, J = geom
        self.key = (tuple(mapping), tuple(coeff), u, v, I, J)
        self.table = [(m[0], m[1], q, m[3]) for q, m in enumerate(mapping)]

    def _problem(self):
        mapping, coeff, u, v, I, J = self.geom
        return _make_problem(self.table, coeff, u, v, I, J, self.batch, self.precision)

    def _w3(self, w):
        mapping, _, u, v, _, _ = self.geom
        return _order_weights(w.reshape(len(mapping), u, v).contiguous(), mapping)

    def forward(self, w, x):
        mapping, coeff, u, v, I, J = self.geom
        x3 = x.reshape(self.batch, I, u).contiguous()
        out = torch.empty((self.batch, J, v), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            _run(_core(), self._problem(), w, self._w3(w), x3, out, self.key, self.precision, False,
                 torch.cuda.current_stream(x.device).cuda_stream)
        return out.reshape(self.batch, J * v)

    def dgrad(self, w, g):
        mapping, coeff, u, v, I, J = self.geom
        g3 = g.reshape(self.batch, J, v).contiguous()
        dx = torch.empty((self.batch, I, u), dtype=g3.dtype, device=g3.device)
        with torch.cuda.device(g3.device):
            _run(_core(), self._problem(), w, self._w3(w), g3, dx, self.key, self.precision, True,
                 torch.cuda.current_stream(g3.device).cuda_stream)
        return dx.reshape(self.batch, I * u)

    def wgrad(self, x, g):
        mapping, coeff, u, v, I, J = self.geom
        x3 = x.reshape(self.batch, I, u).contiguous()
        g3 = g.reshape(self.batch, J, v).contiguous()
        dw = torch.empty((len(mapping), u, v), dtype=g3.dtype, device=g3.device)
        lib = _core()
        with torch.cuda.device(g3.device):
            _cabi.check(lib.fasteq_eqlinear_wgrad(C.byref(self._problem()), x3.data_ptr(), g3.data_ptr(), dw.data_ptr(),
                                                  torch.cuda.current_stream(g3.device).cuda_stream), lib, "fasteq_eqlinear_wgrad")
        wps = [m[2] for m in mapping]
        if wps != list(range(len(wps))):      # block q of the table is block wps[q] of the caller's tensor
            full = torch.empty_like(dw)
            full[torch.tensor(wps, device=dw.device)] = dw
            dw = full
        return dw.reshape(self.w_shape)


class _EqLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, x, geom, precision):
        mapping, coeff, u, v, I, J = geom
        _check_inputs(w, x, u, v, I, len(mapping))
        plan = _Plan(geom, precision, x.numel() // (I * u), w.shape)
        ctx.plan = plan
        ctx.save_for_backward(w, x)
        return plan.forward(w, x)

    @staticmethod
    def backward(ctx, grad_out):
        w, x = ctx.saved_tensors
        need_w, need_x = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if not (need_w or need_x):
            return None, None, None, None
        dw, dx = _EqLinearBackwardFn.apply(grad_out.contiguous(), w, x, ctx.plan, need_w, need_x)
        return (dw if need_w else None), (dx.reshape(x.shape) if need_x else None), None, None


class _EqLinearBackwardFn(torch.autograd.Function):
    """First backward as a differentiable function.  The operator is bilinear in (w, x), so each term of the
    second backward is one of the three launches again, with a second-order cotangent in place of an operand:

        d_go = F(w, ggx) + F(ggw, x)        d_w = Wg(ggx, go)        d_x = Dg(ggw, go)
    """

    @staticmethod
    def forward(ctx, go, w, x, plan, need_w, need_x):
        ctx.plan, ctx.need = plan, (need_w, need_x)
        ctx.save_for_backward(go, w, x)
        ctx.set_materialize_grads(False)
        dw = plan.wgrad(x, go) if need_w else w.new_empty((0,))
        dx = plan.dgrad(w, go) if need_x else x.new_empty((0,))
        return dw, dx

    @staticmethod
    def backward(ctx, ggw, ggx):
        go, w, x = ctx.saved_tensors
        plan = ctx.plan
        ggw = ggw.contiguous() if (ggw is not None and ctx.need[0]) else None
        ggx = ggx.contiguous() if (ggx is not None and ctx.need[1]) else None
        want_go, want_w, want_x = ctx.needs_input_grad[:3]
        d_go = d_w = d_x = None
        if want_go:
            if ggx is not None:
                d_go = plan.forward(w, ggx)
            if ggw is not None:
                t = plan.forward(ggw, x)
                d_go = t if d_go is None else d_go + t
            if d_go is not None:
                d_go = d_go.reshape(go.shape)
        if want_w and ggx is not None:
            d_w = plan.wgrad(ggx, go)
        if want_x and ggw is not None:
            d_x = plan.dgrad(ggw, go).reshape(x.shape)
        return d_go, d_w, d_x, None, None, None


def fast_equi_linear(descriptor, w, x, *, compute_precision=None):
    """Forward, grad_x and grad_w for the uniform uv/iu/iv eqlinear operator."""
    precision = _resolve_precision(x, w, compute_precision)
    geom = _descriptor_problem(descriptor)
    return _EqLinearFn.apply(w, x, geom, precision)


def eqlinear_clear_plan_cache() -> None:
    """Drop the prepared weights (same name as the reference's call, fasteq/ops/eqlinear.py)."""
    _prepared.clear()


def eqlinear_set_plan_cache(max_bytes=None) -> None:
    """Byte budget of the prepared-weight cache; ``0`` disables it, ``None`` restores the default (256 MiB)."""
    _prepared.set_budget(max_bytes)


def eqlinear_debug_info(descriptor, w, x, *, compute_precision=None) -> dict:
    mapping, coeff, u, v, I, J = _descriptor_problem(descriptor)
    return {"precision": _resolve_precision(x, w, compute_precision), "forward_impl": 0, "a_view": 1, "j_rows": J}
