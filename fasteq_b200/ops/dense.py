"""Dense layer ``y = x @ weight.T`` on the tensor cores with 3xTF32 arithmetic (FP32 data, relative
error near 1e-6), for the radial MLP that produces the tensor-product weights.  FP64 tensors and
shapes the kernel does not take go through ``torch.matmul`` (cuBLAS FP64 / FP32 without TF32).
The gradient with respect to ``x`` uses the same kernel; the weight gradient, needed only for
training, is a plain ``torch.matmul`` reduction over the edges.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _cabi
from . import _prepared

_ready = False


def _lib():
    global _ready
    lib = _cabi.core()
    if not _ready:
        lib.fasteq_gemm_tf32x3.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p]
        lib.fasteq_tensorcore_device_status.argtypes = [C.POINTER(C.c_int32)]
        lib.fasteq_gemm_tf32x3_split.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
        lib.fasteq_gemm_tf32x3_presplit.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p]
        _ready = True
    return lib


def tensorcore_device_status() -> int:
    v = C.c_int32(0)
    lib = _lib()
    _cabi.check(lib.fasteq_tensorcore_device_status(C.byref(v)), lib, "fasteq_tensorcore_device_status")
    return int(v.value)


def _usable(x: torch.Tensor, n: int, k: int) -> bool:
    return x.is_cuda and x.dtype == torch.float32 and k % 4 == 0 and n % 4 == 0 and k >= 4 and n >= 4 and x.shape[0] > 0


def _gemm(a: torch.Tensor, bt: torch.Tensor, weight: torch.Tensor = None, transposed: bool = False) -> torch.Tensor:
    """a [M, K] @ bt[N, K]^T -> [M, N].  ``weight`` (optional) is the parameter ``bt`` derives from: its TF32 parts
    are then prepared once per weight version instead of once per call."""
    a = a.contiguous()
    M, K = a.shape
    N = bt.shape[0]
    out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    lib = _lib()
    with torch.cuda.device(a.device):
        stream = torch.cuda.current_stream(a.device).cuda_stream
        split = None
        if weight is not None:
            def build():
                b = bt.contiguous()
                sp = torch.empty(2 * b.numel(), dtype=torch.float32, device=b.device)
                _cabi.check(lib.fasteq_gemm_tf32x3_split(b.data_ptr(), b.numel(), sp.data_ptr(), stream), lib, "fasteq_gemm_tf32x3_split")
                return sp
            split = _prepared.get((weight,), ("dense", transposed), build)
        if split is not None:
            rc = lib.fasteq_gemm_tf32x3_presplit(a.data_ptr(), split.data_ptr(), out.data_ptr(), M, N, K, stream)
        else:
            bt = bt.contiguous()
            rc = lib.fasteq_gemm_tf32x3(a.data_ptr(), bt.data_ptr(), out.data_ptr(), M, N, K, stream)
    if rc == 1:   # FASTEQ_UNSUPPORTED: alignment
        return a @ bt.t()
    _cabi.check(rc, lib, "fasteq_gemm_tf32x3")
    return out


class _Dense(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        return _gemm(x, weight, weight, False)

    @staticmethod
    def backward(ctx, grad_out):
        x, weight = ctx.saved_tensors
        need_x, need_w = ctx.needs_input_grad
        if not (need_x or need_w):
            return None, None
        gx, gw = _DenseBackward.apply(grad_out.contiguous(), x, weight, need_x, need_w)
        return (gx if need_x else None), (gw if need_w else None)


class _DenseBackward(torch.autograd.Function):
    """First backward as a differentiable function (``y = x W^T`` is bilinear):
    ``d_g = ggx W^T + x ggW^T``, ``d_x = g ggW``, ``d_W = g^T ggx``."""

    @staticmethod
    def forward(ctx, g, x, weight, need_x, need_w):
        ctx.need = (need_x, need_w)
        ctx.save_for_backward(g, x, weight)
        ctx.set_materialize_grads(False)
        gx = _gemm(g, weight.t(), weight, True) if need_x else x.new_empty((0,))     # [M, N] @ [N, K], Bt = weight^T [K, N]
        gw = g.t() @ x if need_w else weight.new_empty((0,))                         # reduction over the rows: plain matmul
        return gx, gw

    @staticmethod
    def backward(ctx, ggx, ggw):
        g, x, weight = ctx.saved_tensors
        ggx = ggx.contiguous() if (ggx is not None and ctx.need[0]) else None
        ggw = ggw.contiguous() if (ggw is not None and ctx.need[1]) else None
        want_g, want_x, want_w = ctx.needs_input_grad[:3]
        d_g = d_x = d_w = None
        if want_g:
            if ggx is not None:
                d_g = _gemm(ggx, weight, weight, False)
            if ggw is not None:
                t = _gemm(x, ggw)
                d_g = t if d_g is None else d_g + t
        if want_x and ggw is not None:
            d_x = _gemm(g, ggw.t())
        if want_w and ggx is not None:
            d_w = g.t() @ ggx
        return d_g, d_x, d_w, None, None


def dense(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x [..., K] @ weight[N, K]^T``."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if _usable(x2, weight.shape[0], weight.shape[1]) and weight.dtype == torch.float32:
        return _Dense.apply(x2, weight).reshape(*lead, weight.shape[0])
    return x @ weight.t()
