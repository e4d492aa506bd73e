"""Edge vectors and radial basis of a radius graph in one kernel, with the force-pass gradient in another
(``fasteq_edge_geometry_forward`` / ``_backward``): ``vec = pos[src] + shift - pos[dst]``,
``basis = bessel(|vec|) * polynomial_cutoff(|vec|)``.  First order only."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _cabi

_ready = False


def _lib():
    global _ready
    lib = _cabi.core()
    if not _ready:
        v = C.c_void_p
        lib.fasteq_edge_geometry_forward.argtypes = [C.c_int32, v, v, v, v, C.c_int64, C.c_int64, C.c_double, C.c_int32, C.c_int32, v, v, v]
        lib.fasteq_edge_geometry_device_status.argtypes = [C.POINTER(C.c_int32)]
        lib.fasteq_edge_geometry_backward.argtypes = [C.c_int32, v, v, v, v, v, v, C.c_int64, C.c_int64, C.c_double, C.c_int32,
                                                      C.c_int32, v, v]
        _ready = True
    return lib


def _i32(t: torch.Tensor) -> torch.Tensor:
    return (t if t.dtype == torch.int32 else t.to(torch.int32)).contiguous()


class _EdgeGeometry(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pos, src, dst, shift, r_max, n_basis, p):
        pos, shift = pos.contiguous(), shift.to(pos.dtype).contiguous()
        src, dst = _i32(src), _i32(dst)
        E = src.numel()
        vec = torch.empty((E, 3), dtype=pos.dtype, device=pos.device)
        basis = torch.empty((E, n_basis), dtype=pos.dtype, device=pos.device)
        code = 0 if pos.dtype == torch.float32 else 1
        lib = _lib()
        with torch.cuda.device(pos.device):
            rc = lib.fasteq_edge_geometry_forward(code, pos.data_ptr(), src.data_ptr(), dst.data_ptr(), shift.data_ptr(), E, pos.shape[0], float(r_max),
                                                  n_basis, p, vec.data_ptr(), basis.data_ptr(), torch.cuda.current_stream(pos.device).cuda_stream)
        _cabi.check(rc, lib, "fasteq_edge_geometry_forward")
        ctx.save_for_backward(pos, src, dst, shift)
        ctx.cfg = (float(r_max), n_basis, p, code)
        ctx.set_materialize_grads(False)
        return vec, basis

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g_vec, g_basis):
        pos, src, dst, shift = ctx.saved_tensors
        r_max, n_basis, p, code = ctx.cfg
        if not ctx.needs_input_grad[0] or (g_vec is None and g_basis is None):
            return (None,) * 7
        gv = g_vec.contiguous() if g_vec is not None else None
        gb = g_basis.contiguous() if g_basis is not None else None
        g_pos = torch.empty_like(pos)
        lib = _lib()
        ptr = lambda t: t.data_ptr() if t is not None else None
        with torch.cuda.device(pos.device):
            rc = lib.fasteq_edge_geometry_backward(code, pos.data_ptr(), src.data_ptr(), dst.data_ptr(), shift.data_ptr(), ptr(gv), ptr(gb),
                                                   src.numel(), pos.shape[0], r_max, n_basis, p, g_pos.data_ptr(),
                                                   torch.cuda.current_stream(pos.device).cuda_stream)
        _cabi.check(rc, lib, "fasteq_edge_geometry_backward")
        return g_pos, None, None, None, None, None, None


def edge_geometry_usable(pos: torch.Tensor, n_basis: int) -> bool:
    return pos.is_cuda and pos.dtype in (torch.float32, torch.float64) and pos.dim() == 2 and pos.shape[1] == 3 and 1 <= n_basis <= 16


def edge_geometry(pos, edge_src, edge_dst, edge_shift, r_max: float, n_basis: int, envelope_p: int):
    """``(vec [E, 3], basis [E, n_basis])``; differentiable once with respect to ``pos``."""
    return _EdgeGeometry.apply(pos, edge_src, edge_dst, edge_shift, r_max, n_basis, envelope_p)


def edge_geometry_device_status() -> int:
    """Reads and clears the kernels' status word (synchronises): 0, or 2 after an edge index outside the position array
    (such an edge is skipped: zero features, no gradient)."""
    lib = _lib()
    v = C.c_int32(0)
    _cabi.check(lib.fasteq_edge_geometry_device_status(C.byref(v)), lib, "fasteq_edge_geometry_device_status")
    return int(v.value)
