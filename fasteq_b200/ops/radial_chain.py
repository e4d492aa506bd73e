"""Fused hidden layers of the radial MLP: ``h_L = silu(W_L ... silu(W_1 basis))`` in one kernel, and
its gradient with respect to the basis in another (``fasteq_radial_chain_forward`` / ``_backward``).

Width 64, one to three hidden layers, at most 16 basis functions, FP32, no bias, weights that do not
require grad (inference and force evaluation); anything else returns ``None`` from
``radial_chain`` so that the caller takes the layered path.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from .. import _cabi
from . import _prepared

_ready = False
WIDTH = 64
MAX_BASIS = 16
MAX_HIDDEN = 3


def _lib():
    global _ready
    lib = _cabi.core()
    if not _ready:
        pp = C.POINTER(C.c_void_p)
        lib.fasteq_radial_chain_forward.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, pp, C.c_void_p, C.c_int32, C.c_void_p,
                                                    C.c_void_p, C.c_void_p]
        lib.fasteq_radial_chain_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, pp,
                                                     C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]
        lib.fasteq_radial_chain_prepare.argtypes = [pp, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
        _ready = True
    return lib


def _hidden_array(ws: Sequence[torch.Tensor]):
    arr = (C.c_void_p * max(1, len(ws)))()
    for i, w in enumerate(ws):
        arr[i] = w.data_ptr()
    return arr


def _prepared_hidden(ws, backward: bool, lib, stream):
    """TF32 parts of the 64 x 64 layers in the order (and orientation) the kernel of this direction multiplies with."""
    hidden = ws[1:]
    if not hidden:
        return None
    def build():
        prep = torch.empty(len(hidden) * 2 * WIDTH * WIDTH, dtype=torch.float32, device=hidden[0].device)
        _cabi.check(lib.fasteq_radial_chain_prepare(_hidden_array(hidden), len(ws), 1 if backward else 0, prep.data_ptr(), stream),
                    lib, "fasteq_radial_chain_prepare")
        return prep
    return _prepared.get(tuple(hidden), ("radial_chain", backward), build)


class _RadialChain(torch.autograd.Function):
    @staticmethod
    def forward(ctx, basis, *weights):
        E, nb = basis.shape
        ws = [w.contiguous() for w in weights]
        n_hidden = len(ws)
        out = torch.empty((E, WIDTH), dtype=torch.float32, device=basis.device)
        deriv = torch.empty((max(n_hidden - 1, 1), E, WIDTH), dtype=torch.float32, device=basis.device)
        lib = _lib()
        with torch.cuda.device(basis.device):
            stream = torch.cuda.current_stream(basis.device).cuda_stream
            prep = _prepared_hidden(ws, False, lib, stream)
            rc = lib.fasteq_radial_chain_forward(basis.data_ptr(), E, nb, ws[0].data_ptr(), _hidden_array(ws[1:]),
                                                 prep.data_ptr() if prep is not None else None, n_hidden,
                                                 out.data_ptr(), deriv.data_ptr(), stream)
        _cabi.check(rc, lib, "fasteq_radial_chain_forward")
        ctx.save_for_backward(basis, deriv, *ws)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        basis, deriv, *ws = ctx.saved_tensors
        if not ctx.needs_input_grad[0]:
            return (None,) * (1 + len(ws))
        E, nb = basis.shape
        g = grad_out.contiguous()
        gb = torch.empty((E, nb), dtype=torch.float32, device=basis.device)
        lib = _lib()
        with torch.cuda.device(basis.device):
            stream = torch.cuda.current_stream(basis.device).cuda_stream
            prep = _prepared_hidden(ws, True, lib, stream)
            rc = lib.fasteq_radial_chain_backward(g.data_ptr(), deriv.data_ptr(), basis.data_ptr(), E, nb, ws[0].data_ptr(),
                                                  _hidden_array(ws[1:]), prep.data_ptr() if prep is not None else None, len(ws),
                                                  gb.data_ptr(), stream)
        _cabi.check(rc, lib, "fasteq_radial_chain_backward")
        return (gb,) + (None,) * len(ws)


def radial_chain_usable(basis: torch.Tensor, weights: Sequence[torch.Tensor]) -> bool:
    if not (basis.is_cuda and basis.dtype == torch.float32 and basis.dim() == 2 and basis.shape[0] > 0):
        return False
    if not (1 <= len(weights) <= MAX_HIDDEN and 1 <= basis.shape[1] <= MAX_BASIS):
        return False
    if tuple(weights[0].shape) != (WIDTH, basis.shape[1]):
        return False
    for w in weights:
        if w.dtype != torch.float32 or not w.is_cuda or (torch.is_grad_enabled() and w.requires_grad):
            return False
    return all(tuple(w.shape) == (WIDTH, WIDTH) for w in weights[1:])


def radial_chain(basis: torch.Tensor, weights: Sequence[torch.Tensor]) -> Optional[torch.Tensor]:
    """``silu(W_L ... silu(W_1 basis^T))^T`` for ``basis [E, n_basis]`` and ``torch.nn.Linear`` style weights
    (``[out, in]``), or ``None`` when the fused kernels do not take the arguments."""
    if not radial_chain_usable(basis, weights):
        return None
    return _RadialChain.apply(basis.contiguous(), *weights)
