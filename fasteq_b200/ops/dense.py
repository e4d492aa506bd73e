"""Dense layer ``y = x @ weight.T`` for the radial MLP that produces the tensor-product weights.

FP32 data: tcgen05 tensor cores with 3xTF32 arithmetic (relative error near 1e-6); the gradient with respect
to ``x`` uses the same kernel.  FP64 data, FP32 shapes the tensor-core kernel does not take (a dimension that is
not a multiple of four, operands that are not 16-byte aligned) and every weight gradient go through the kernels of
the SO3Linear family: a plain GEMM is its one-path, one-row case (``fasteq_eqlinear_forward`` / ``_dgrad`` /
``_wgrad`` with ``u = K``, ``v = N``), so no library GEMM is called on CUDA tensors.  FP64 forward and grad_x with
even extents run on the FP64 tensor cores (DMMA, as the reference's FP64 back-end does:
fasteq/cuda/src/eqlinear/backends/fp64/direct_gemm_f64_tma.cu:204); the rest run on FMA tile kernels.
CPU tensors (the oracle's territory) fall through to ``torch.matmul``.
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


def _fma_problem(M: int, K: int, N: int, dtype):
    from .eqlinear import _FP32, _FP64, _make_problem
    return _make_problem([(0, 0, 0, 1)], [1.0], K, N, 1, 1, M, _FP64 if dtype == torch.float64 else _FP32)


def _fma_call(name: str, prob, p0, p1, out) -> None:
    from .eqlinear import _core
    lib = _core()
    with torch.cuda.device(out.device):
        rc = getattr(lib, name)(C.byref(prob), p0.data_ptr(), p1.data_ptr(), out.data_ptr(), torch.cuda.current_stream(out.device).cuda_stream)
    _cabi.check(rc, lib, name)


def _fma_gemm(a: torch.Tensor, w_kn: torch.Tensor) -> torch.Tensor:
    """``a [M, K] @ w_kn [K, N]`` on the one-path SO3Linear kernels (FP32: FMA tiles; FP64: DMMA, or FMA tiles for odd extents)."""
    a, w_kn = a.contiguous(), w_kn.contiguous()
    M, K = a.shape
    out = torch.empty((M, w_kn.shape[1]), dtype=a.dtype, device=a.device)
    if M > 0:
        _fma_call("fasteq_eqlinear_forward", _fma_problem(M, K, w_kn.shape[1], a.dtype), w_kn, a, out)
    return out


def _fma_gemm_nt(g: torch.Tensor, w_kn: torch.Tensor) -> torch.Tensor:
    """``g [M, N] @ w_kn[K, N]^T -> [M, K]`` (the grad_x launch of the same problem)."""
    g, w_kn = g.contiguous(), w_kn.contiguous()
    M, K = g.shape[0], w_kn.shape[0]
    out = torch.empty((M, K), dtype=g.dtype, device=g.device)
    if M > 0:
        _fma_call("fasteq_eqlinear_dgrad", _fma_problem(M, K, w_kn.shape[1], g.dtype), w_kn, g, out)
    return out


def _fma_wgrad(x: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """``x [M, K]^T @ g [M, N] -> [K, N]``: the reduction over the rows, in fixed order (``fasteq_eqlinear_wgrad``)."""
    x, g = x.contiguous(), g.contiguous()
    out = torch.empty((x.shape[1], g.shape[1]), dtype=x.dtype, device=x.device)
    if x.shape[0] == 0:
        return out.zero_()
    _fma_call("fasteq_eqlinear_wgrad", _fma_problem(x.shape[0], x.shape[1], g.shape[1], x.dtype), x, g, out)
    return out


def _matmul_nt(a: torch.Tensor, bt: torch.Tensor) -> torch.Tensor:
    """``a [M, K] @ bt[N, K]^T`` on this library's one-path SO3Linear kernels (CUDA) or torch (CPU)."""
    if a.is_cuda and a.dtype in (torch.float32, torch.float64) and a.dtype == bt.dtype:
        return _fma_gemm(a, bt.t())
    return a @ bt.t()


def _matmul_tn(g: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``g [M, N]^T @ x [M, K] -> [N, K]``."""
    if g.is_cuda and g.dtype in (torch.float32, torch.float64) and g.dtype == x.dtype:
        return _fma_wgrad(x, g).t().contiguous()
    return g.t() @ x


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
    if rc == 1:   # FASTEQ_UNSUPPORTED (operand alignment): the FP32 FMA tile kernel takes any shape and alignment
        return _fma_gemm(a, bt.t())
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
        gw = _matmul_tn(g, x) if need_w else weight.new_empty((0,))                  # reduction over the rows, fixed order
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
            d_w = _matmul_tn(g, ggx)
        return d_g, d_x, d_w, None, None


def dense(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x [..., K] @ weight[N, K]^T``."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if _usable(x2, weight.shape[0], weight.shape[1]) and weight.dtype == torch.float32:
        return _Dense.apply(x2, weight).reshape(*lead, weight.shape[0])
    if x2.is_cuda and x2.dtype in (torch.float32, torch.float64) and weight.dtype == x2.dtype:
        return _DenseFMA.apply(x2, weight).reshape(*lead, weight.shape[0])
    return x @ weight.t()


class _DenseFMA(torch.autograd.Function):
    """``y = x W^T`` on the one-path SO3Linear kernels (FP32 FMA tiles, FP64 DMMA), differentiable to every order (each gradient is
    another call of ``dense`` / the row reduction, which autograd differentiates again)."""

    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        return _fma_gemm(x, weight.t())

    @staticmethod
    def backward(ctx, grad_out):
        x, weight = ctx.saved_tensors
        need_x, need_w = ctx.needs_input_grad
        gx = _DenseFMA.apply(grad_out, weight.t()) if need_x else None       # g [M, N] @ W [N, K]
        gw = _RowReduce.apply(grad_out, x) if need_w else None               # g^T x  [N, K]
        return gx, gw


class _RowReduce(torch.autograd.Function):
    """``R(a, b) = a^T b`` (``a [M, N]``, ``b [M, K]`` -> ``[N, K]``); its gradients are dense products again."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return _matmul_tn(a, b)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        ga = _DenseFMA.apply(b, g) if ctx.needs_input_grad[0] else None          # b [M, K] @ g^T [K, N] -> [M, N]
        gb = _DenseFMA.apply(a, g.t()) if ctx.needs_input_grad[1] else None      # a [M, N] @ g [N, K]   -> [M, K]
        return ga, gb
