"""Equivariant gate (e3nn ``nn.Gate`` semantics) on ir_mul tensors, through ``fasteq_gate_forward`` /
``fasteq_gate_backward``.  ``x`` is ``[B, (n_scalar + n_gate + sum(2l+1)) * u]``: scalar segments, one
gate segment per gated irrep block, the gated irreps.  The backward is not itself differentiable."""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Sequence

import torch

from .. import _cabi

ACT_CODES = {"identity": 0, None: 0, "silu": 1, "tanh": 2, "sigmoid": 3, "abs": 4}


class _Problem(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("u", C.c_int32), ("n_scalar", C.c_int32), ("n_gate", C.c_int32), ("batch", C.c_int64),
                ("act", C.POINTER(C.c_int32)), ("cst", C.POINTER(C.c_double)), ("gated_dims", C.POINTER(C.c_int32))]


def second_moment_constant(name) -> float:
    """``1 / sqrt(E[act(z)^2])`` for ``z ~ N(0, 1)`` by Gauss-Hermite quadrature (e3nn estimates the same
    constant from one million samples, e3nn/math/_normalize_activation.py:22-47)."""
    import numpy as np
    if ACT_CODES[name] == 0:
        return 1.0
    z, wts = np.polynomial.hermite_e.hermegauss(200)
    f = {"silu": lambda t: t / (1 + np.exp(-t)), "tanh": np.tanh, "sigmoid": lambda t: 1 / (1 + np.exp(-t)), "abs": np.abs}[name]
    m2 = float((wts * f(z) ** 2).sum() / math.sqrt(2 * math.pi))
    return 1.0 / math.sqrt(m2)


_ready = False


def _lib():
    global _ready
    lib = _cabi.core()
    if not _ready:
        lib.fasteq_gate_forward.argtypes = [C.POINTER(_Problem), C.c_void_p, C.c_void_p, C.c_void_p]
        lib.fasteq_gate_backward.argtypes = [C.POINTER(_Problem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.fasteq_gate_double_backward.argtypes = [C.POINTER(_Problem)] + [C.c_void_p] * 6
        _ready = True
    return lib


class GateSpec:
    def __init__(self, u: int, scalar_acts: Sequence, gate_acts: Sequence, gated_ls: Sequence[int],
                 scalar_csts: Sequence[float] = None, gate_csts: Sequence[float] = None):
        if len(gate_acts) != len(gated_ls):
            raise ValueError("one gate activation per gated irrep block")
        self.u = int(u)
        self.acts = [ACT_CODES[a] for a in list(scalar_acts) + list(gate_acts)]
        csts = list(scalar_csts) if scalar_csts is not None else [second_moment_constant(a) for a in scalar_acts]
        csts += list(gate_csts) if gate_csts is not None else [second_moment_constant(a) for a in gate_acts]
        self.csts = [float(c) for c in csts]
        self.n_scalar, self.n_gate = len(scalar_acts), len(gate_acts)
        self.gated_dims = [2 * l + 1 for l in gated_ls]
        self.n_in = self.n_scalar + self.n_gate + sum(self.gated_dims)
        self.n_out = self.n_scalar + sum(self.gated_dims)

    def problem(self, batch: int, dtype) -> _Problem:
        n = self.n_scalar + self.n_gate
        return _Problem(0 if dtype == torch.float32 else 1, self.u, self.n_scalar, self.n_gate, batch,
                        (C.c_int32 * max(n, 1))(*self.acts), (C.c_double * max(n, 1))(*self.csts),
                        (C.c_int32 * max(self.n_gate, 1))(*self.gated_dims))


class _Gate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, spec: GateSpec):
        if not x.is_cuda:
            raise RuntimeError("gate needs a CUDA tensor: fasteq_b200 has no CPU path")
        if x.dtype not in (torch.float32, torch.float64):
            raise ValueError("gate supports float32 and float64")
        xc = x.contiguous()
        B = xc.numel() // (spec.n_in * spec.u)
        out = torch.empty((B, spec.n_out * spec.u), dtype=x.dtype, device=x.device)
        lib = _lib()
        prob = spec.problem(B, x.dtype)
        with torch.cuda.device(x.device):
            _cabi.check(lib.fasteq_gate_forward(C.byref(prob), xc.data_ptr(), out.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream),
                        lib, "fasteq_gate_forward")
        ctx.save_for_backward(x)       # the input itself, so that a second backward reaches it
        ctx.spec = spec
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (x,) = ctx.saved_tensors
        return _GateBackward.apply(grad_out.contiguous(), x.contiguous(), ctx.spec), None


class _GateBackward(torch.autograd.Function):
    """Input gradient as a differentiable function (second-order kernels ``fasteq_gate_double_backward``)."""

    @staticmethod
    def forward(ctx, go, xc, spec):
        gx = torch.empty_like(xc)
        B = xc.numel() // (spec.n_in * spec.u)
        lib = _lib()
        prob = spec.problem(B, xc.dtype)
        with torch.cuda.device(xc.device):
            _cabi.check(lib.fasteq_gate_backward(C.byref(prob), xc.data_ptr(), go.data_ptr(), gx.data_ptr(),
                                                 torch.cuda.current_stream(xc.device).cuda_stream), lib, "fasteq_gate_backward")
        ctx.save_for_backward(go, xc)
        ctx.spec = spec
        return gx

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, ggx):
        go, xc = ctx.saved_tensors
        spec = ctx.spec
        t = ggx.contiguous()
        d_go, d_x = torch.empty_like(go), torch.empty_like(xc)
        B = xc.numel() // (spec.n_in * spec.u)
        lib = _lib()
        prob = spec.problem(B, xc.dtype)
        with torch.cuda.device(xc.device):
            _cabi.check(lib.fasteq_gate_double_backward(C.byref(prob), xc.data_ptr(), go.data_ptr(), t.data_ptr(), d_go.data_ptr(),
                                                        d_x.data_ptr(), torch.cuda.current_stream(xc.device).cuda_stream),
                        lib, "fasteq_gate_double_backward")
        return d_go, d_x, None


def gate(x: torch.Tensor, spec: GateSpec) -> torch.Tensor:
    return _Gate.apply(x, spec)
