"""e3nn-compatible spherical harmonics of edge vectors on the GPU (forward and vector gradient).

Mirror of the reference's ``SphericalHarmonics`` module and ``spherical_harmonics`` function
(fasteq/triton/spherical_harmonics.py:493-575): ``irreps_out`` may be an int, a list of degrees or an
irreps string; ``normalize`` divides by ``max(|r|, 1e-12)``; ``normalization`` is ``"integral"``
(default), ``"component"`` or ``"norm"``.  The kernels are generated per (degrees, dtype, flags) and
called through the C ABI (``fasteq_sh_forward`` / ``fasteq_sh_backward`` / ``fasteq_sh_double_backward``);
the backward is itself differentiable (Hessian-vector kernel), so force losses can be trained.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Dict, List, Tuple, Union

import torch

from .. import _build, _cabi
from ..codegen import sh as _emit
from ..irreps import Irreps

_MODULES: Dict[Tuple, C.CDLL] = {}
_lock = threading.Lock()


def _module(ls: Tuple[int, ...], dtype: torch.dtype, normalize: bool, normalization: str):
    key = (ls, dtype, normalize, normalization)
    with _lock:
        lib = _MODULES.get(key)
    if lib is None:
        dt = "f32" if dtype == torch.float32 else "f64"
        name = f"sh_{'_'.join(map(str, ls))}_{dt}_{int(normalize)}_{normalization}_v2"
        so = _build.build_generated(name, _emit.emit_sh(ls, dt, normalize, normalization))
        lib = C.CDLL(so, mode=C.RTLD_LOCAL)
        lib.fasteq_sh_forward.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
        lib.fasteq_sh_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
        lib.fasteq_sh_double_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.fasteq_last_cuda_error.restype = C.c_char_p
        with _lock:
            _MODULES.setdefault(key, lib)
    return lib


class _SH(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ls, normalize, normalization):
        flat = x.reshape(-1, 3)
        n = flat.shape[0]
        nout = sum(2 * l + 1 for l in ls)
        out = torch.empty((n, nout), dtype=x.dtype, device=x.device)
        lib = _module(ls, x.dtype, normalize, normalization)
        with torch.cuda.device(x.device):
            _cabi.check(lib.fasteq_sh_forward(flat.data_ptr(), n, out.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream),
                        lib, "fasteq_sh_forward")
        ctx.save_for_backward(x)       # the input itself: a view made here would be cut off from its autograd history
        ctx.cfg = (ls, normalize, normalization, x.shape)
        return out.reshape(*x.shape[:-1], nout)

    @staticmethod
    def backward(ctx, grad_out):
        (x,) = ctx.saved_tensors
        ls, normalize, normalization, shape = ctx.cfg
        flat = x.reshape(-1, 3)
        g = grad_out.reshape(flat.shape[0], grad_out.shape[-1]).contiguous()
        return _SHBackward.apply(g, flat, ls, normalize, normalization).reshape(shape), None, None, None


class _SHBackward(torch.autograd.Function):
    """Vector gradient as a differentiable function: its backward is the generated Hessian-vector kernel."""

    @staticmethod
    def forward(ctx, g, flat, ls, normalize, normalization):
        gv = torch.empty_like(flat)
        lib = _module(ls, flat.dtype, normalize, normalization)
        with torch.cuda.device(flat.device):
            _cabi.check(lib.fasteq_sh_backward(flat.data_ptr(), g.data_ptr(), flat.shape[0], gv.data_ptr(),
                                               torch.cuda.current_stream(flat.device).cuda_stream), lib, "fasteq_sh_backward")
        ctx.save_for_backward(g, flat)
        ctx.cfg = (ls, normalize, normalization)
        return gv

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, ggv):
        g, flat = ctx.saved_tensors
        ls, normalize, normalization = ctx.cfg
        t = ggv.reshape(flat.shape).contiguous()
        d_g, d_v = torch.empty_like(g), torch.empty_like(flat)
        lib = _module(ls, flat.dtype, normalize, normalization)
        with torch.cuda.device(flat.device):
            _cabi.check(lib.fasteq_sh_double_backward(flat.data_ptr(), g.data_ptr(), t.data_ptr(), flat.shape[0], d_g.data_ptr(),
                                                      d_v.data_ptr(), torch.cuda.current_stream(flat.device).cuda_stream),
                        lib, "fasteq_sh_double_backward")
        return d_g, d_v, None, None, None


class SphericalHarmonics(torch.nn.Module):
    def __init__(self, irreps_out: Union[int, List[int], str, Irreps], normalize: bool, normalization: str = "integral",
                 irreps_in=None) -> None:
        super().__init__()
        if normalization not in ("integral", "component", "norm"):
            raise ValueError("normalization must be 'integral', 'component' or 'norm'")
        self.normalize, self.normalization = bool(normalize), normalization
        if isinstance(irreps_out, str):
            irreps_out = Irreps(irreps_out)
        input_p = -1
        if irreps_in is not None:
            irreps_in = Irreps(irreps_in)
            if irreps_in not in (Irreps("1x1o"), Irreps("1x1e")):
                raise ValueError(f"irreps_in for SphericalHarmonics must be either a vector (`1x1o`) or a pseudovector (`1x1e`), not `{irreps_in}`")
            input_p = irreps_in[0].ir.p
        elif isinstance(irreps_out, Irreps) and any(b.ir.l % 2 == 1 and b.ir.p == 1 for b in irreps_out):
            input_p = 1
        if isinstance(irreps_out, Irreps):
            ls = []
            for b in irreps_out:
                if b.ir.p != input_p ** b.ir.l:
                    raise ValueError(f"irreps_out `{irreps_out}` asks for l = {b.ir.l} with parity {b.ir.p}, inconsistent with the input parity {input_p}")
                ls.extend([b.ir.l] * b.mul)
        elif isinstance(irreps_out, int):
            ls = [irreps_out]
        else:
            ls = list(irreps_out)
        if not ls or any(type(l) is not int or l < 0 for l in ls):
            raise ValueError("degrees must be a nonempty sequence of nonnegative integers")
        if max(ls) > 8:
            raise NotImplementedError("spherical_harmonics maximum l implemented is 8")
        self._ls = tuple(ls)
        self.irreps_in = Irreps("1x1o" if input_p == -1 else "1x1e")
        self.irreps_out = Irreps([(1, (l, input_p ** l)) for l in ls])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.ndim < 1 or x.shape[-1] != 3:
            raise ValueError(f"expected input shape (..., 3), got {tuple(x.shape)}")
        if x.dtype not in (torch.float32, torch.float64):
            raise TypeError(f"unsupported dtype: {x.dtype}")
        if not x.is_cuda:
            raise RuntimeError("SphericalHarmonics needs a CUDA tensor: fasteq_b200 has no CPU path")
        return _SH.apply(x.contiguous(), self._ls, self.normalize, self.normalization)


def spherical_harmonics(l, x: torch.Tensor, normalize: bool, normalization: str = "integral") -> torch.Tensor:
    return SphericalHarmonics(l, normalize, normalization)(x)
