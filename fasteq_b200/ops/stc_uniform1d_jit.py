"""``fast_stc_uniform1d_jit``: drop-in for fasteq/ops/stc_uniform1d_jit.py:1108-1145.

``fast_stc_uniform1d_jit(x1, x0, i0, coeffs_tensor, paths_tensor, idx_lists_tensor, num_out_segments)``
with ``x1 [B, X1seg, U]`` node features (ir_mul), ``x0 [n_species, X0seg, U]`` weights, ``i0 [B]``
species index, ``paths_tensor [P, max_len]`` rows ``[a.., d, v, pad]`` (suffix padded with
``pad_value``), ``idx_lists_tensor`` its transpose.  Returns ``[B, V*U]``.  Differences from the
reference: the species gather is fused into the kernel, there are no device synchronisations or
prints in forward / backward, and only CUDA tensors are accepted.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from .. import _build, _cabi
from ..codegen import stc as _emit

STC_PAD_VALUE = -1
_EMITTER_VERSION = "stc-v2"
_lock = threading.Lock()


class STCDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("abi_version", "dtype", "u", "x1_segs", "x0_segs", "out_segs", "num_paths",
                                          "direction", "need_gx0")]


class STCModule:
    def __init__(self, so_path: str):
        self.path = so_path
        lib = C.CDLL(so_path, mode=C.RTLD_LOCAL)
        lib.fasteq_stc_describe.argtypes = [C.POINTER(STCDesc)]
        lib.fasteq_stc_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
        lib.fasteq_stc_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                            C.c_void_p, C.c_void_p, C.c_void_p]
        lib.fasteq_stc_double_backward.argtypes = [C.c_void_p] * 6 + [C.c_int64, C.c_int64] + [C.c_void_p] * 4
        lib.fasteq_stc_device_status.argtypes = [C.POINTER(C.c_int32)]
        lib.fasteq_last_cuda_error.restype = C.c_char_p
        self.lib = lib
        self.desc = STCDesc()
        _cabi.check(lib.fasteq_stc_describe(C.byref(self.desc)), lib, "fasteq_stc_describe")

    def device_status(self) -> int:
        v = C.c_int32(0)
        _cabi.check(self.lib.fasteq_stc_device_status(C.byref(v)), self.lib, "fasteq_stc_device_status")
        return int(v.value)


_MODULES: Dict[Tuple, STCModule] = {}
_SPECS: Dict[Tuple, Tuple] = {}


def get_module(spec: _emit.STCSpec, direction: str, need_gx0: bool = False) -> STCModule:
    key = (spec, direction, need_gx0)
    with _lock:
        mod = _MODULES.get(key)
    if mod is None:
        tag = spec.key(f"{_EMITTER_VERSION}|{direction}|{need_gx0}")
        so = _build.build_generated(f"stc_{direction}_{tag}", _emit.emit_stc(spec, direction, need_gx0))
        with _lock:
            mod = _MODULES.get(key)
            if mod is None:
                mod = STCModule(so)
                _MODULES[key] = mod
    return mod


def _spec_for(x1, coeffs_tensor, paths_tensor, x0_segs: int, num_out_segments: int, pad_value: int) -> _emit.STCSpec:
    key = (id(paths_tensor), paths_tensor._version, id(coeffs_tensor), coeffs_tensor._version, x1.shape[1], x1.shape[2],
           x0_segs, num_out_segments, x1.dtype, pad_value)
    hit = _SPECS.get(key)
    if hit is None:
        P = coeffs_tensor.numel()
        paths = paths_tensor.detach().cpu().numpy()
        if paths.ndim != 2:
            raise ValueError(f"paths_tensor must be 2-D, got shape {tuple(paths.shape)}")
        if paths.shape[0] != P and paths.shape[1] == P:
            paths = paths.T
        elif paths.shape[0] != P:
            raise ValueError(f"cannot match paths_tensor shape {tuple(paths.shape)} with {P} coefficients")
        spec = _emit.make_stc_spec(paths, coeffs_tensor.detach().cpu().double().numpy(), x1_segs=int(x1.shape[1]),
                                   x0_segs=int(x0_segs), out_segs=int(num_out_segments), u=int(x1.shape[2]),
                                   dtype="f32" if x1.dtype == torch.float32 else "f64", pad_value=pad_value)
        if len(_SPECS) > 64:
            _SPECS.clear()
        hit = (spec, paths_tensor, coeffs_tensor)   # keep the tables alive: their ids are the key
        _SPECS[key] = hit
    return hit[0]


def _validate(x1, x0, i0):
    for name, t in (("x1", x1), ("x0", x0), ("i0", i0)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor: fasteq_b200 has no CPU path")
    if x1.dim() != 3 or x0.dim() != 3:
        raise ValueError("x1 must be [B, X1seg, U] and x0 [n_species, X0seg, U]")
    if x1.dtype != x0.dtype or x1.dtype not in (torch.float32, torch.float64):
        raise ValueError("x1 and x0 must both be float32 or both float64")
    if x1.shape[2] != x0.shape[2]:
        raise ValueError("x1 and x0 must have the same channel count")
    if i0.numel() != x1.shape[0]:
        raise ValueError("i0 must have one entry per row of x1")


class FastSymmetricTensorContractionUniform1dFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x1, x0, i0, coeffs_tensor, paths_tensor, idx_lists_tensor, num_out_segments, pad_value):
        _validate(x1, x0, i0)
        if paths_tensor is None:
            paths_tensor = idx_lists_tensor
        spec = _spec_for(x1, coeffs_tensor, paths_tensor, x0.shape[1], num_out_segments, pad_value)
        x1c, x0c = x1.contiguous(), x0.contiguous()
        i32 = i0.to(torch.int32).contiguous()
        B = x1c.shape[0]
        out = torch.empty((B, spec.out_segs, spec.u), dtype=x1.dtype, device=x1.device)
        mod = get_module(spec, "fwd")
        with torch.cuda.device(x1.device):
            _cabi.check(mod.lib.fasteq_stc_forward(x1c.data_ptr(), x0c.data_ptr(), i32.data_ptr(), B, x0c.shape[0], out.data_ptr(),
                                                   torch.cuda.current_stream(x1.device).cuda_stream), mod.lib, "fasteq_stc_forward")
        ctx.save_for_backward(x1, x0, i32)      # the inputs themselves, so that a second backward reaches them
        ctx.spec = spec
        return out.view(B, spec.out_segs * spec.u)

    @staticmethod
    def backward(ctx, grad_out):
        x1, x0, i32 = ctx.saved_tensors
        spec = ctx.spec
        need_x1, need_x0 = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if not (need_x1 or need_x0):
            return (None,) * 8
        gx1, gx0n = FastSTCBackwardFunction.apply(grad_out.contiguous(), x1.contiguous(), x0.contiguous(), i32, spec, bool(need_x0))
        gx0 = None
        if need_x0:
            # summed over nodes of equal species here (differentiable torch op; the kernel writes per-node rows)
            gx0 = torch.zeros_like(x0).index_add(0, i32.long(), gx0n)
        return (gx1 if need_x1 else None), gx0, None, None, None, None, None, None


class FastSTCBackwardFunction(torch.autograd.Function):
    """First backward as a differentiable function (reference: fasteq/ops/stc_uniform1d_jit.py:801-901), so that
    force losses can be trained: its own backward is the generated second-order kernel."""

    @staticmethod
    def forward(ctx, go, x1, x0, i32, spec, need_x0):
        B = x1.shape[0]
        gx1 = torch.empty_like(x1)
        gx0n = torch.empty((B, spec.x0_segs, spec.u), dtype=x1.dtype, device=x1.device) if need_x0 else None
        mod = get_module(spec, "bwd", bool(need_x0))
        with torch.cuda.device(x1.device):
            _cabi.check(mod.lib.fasteq_stc_backward(go.data_ptr(), x1.data_ptr(), x0.data_ptr(), i32.data_ptr(), B, x0.shape[0],
                                                    gx1.data_ptr(), gx0n.data_ptr() if need_x0 else None,
                                                    torch.cuda.current_stream(x1.device).cuda_stream), mod.lib, "fasteq_stc_backward")
        ctx.save_for_backward(go, x1, x0, i32)
        ctx.spec, ctx.need_x0 = spec, need_x0
        return gx1, (gx0n if need_x0 else x1.new_empty((0,)))

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, ggx1, ggx0n):
        go, x1, x0, i32 = ctx.saved_tensors
        spec = ctx.spec
        B = x1.shape[0]
        ggx1 = ggx1.contiguous() if ggx1 is not None else torch.zeros_like(x1)
        if ctx.need_x0 and ggx0n is not None:
            ggx0n = ggx0n.contiguous()
        else:
            ggx0n = torch.zeros((B, spec.x0_segs, spec.u), dtype=x1.dtype, device=x1.device)
        d_go = torch.empty((B, spec.out_segs, spec.u), dtype=x1.dtype, device=x1.device)
        d_x1 = torch.empty_like(x1)
        d_x0n = torch.empty((B, spec.x0_segs, spec.u), dtype=x1.dtype, device=x1.device)
        mod = get_module(spec, "dbwd")
        with torch.cuda.device(x1.device):
            _cabi.check(mod.lib.fasteq_stc_double_backward(go.data_ptr(), x1.data_ptr(), x0.data_ptr(), i32.data_ptr(), ggx1.data_ptr(),
                                                           ggx0n.data_ptr(), B, x0.shape[0], d_go.data_ptr(), d_x1.data_ptr(),
                                                           d_x0n.data_ptr(), torch.cuda.current_stream(x1.device).cuda_stream),
                        mod.lib, "fasteq_stc_double_backward")
        want = ctx.needs_input_grad
        d_x0 = torch.zeros_like(x0).index_add_(0, i32.long(), d_x0n) if want[2] else None
        return (d_go.view(go.shape) if want[0] else None), (d_x1 if want[1] else None), d_x0, None, None, None


def fast_stc_uniform1d_jit(x1, x0, i0, coeffs_tensor, paths_tensor, idx_lists_tensor, num_out_segments: int, *,
                           pad_value: int = STC_PAD_VALUE, use_multiwarp_candidates: bool = False):
    """See module docstring.  ``use_multiwarp_candidates`` is accepted and ignored, as in the reference."""
    return FastSymmetricTensorContractionUniform1dFunction.apply(x1, x0, i0, coeffs_tensor, paths_tensor, idx_lists_tensor,
                                                                 int(num_out_segments), int(pad_value))
