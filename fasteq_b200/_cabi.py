"""ctypes bindings for the C ABI declared in include/fasteq_b200.h."""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional

from . import _build

STATUS = {0: "ok", 1: "unsupported", 2: "invalid argument", 3: "CUDA error", 4: "internal error", 5: "device fault"}


class FasteqError(RuntimeError):
    pass


class U1DDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "abi_version", "dtype", "u", "w_segs", "x_segs", "y_segs", "out_segs", "num_paths", "y_vec", "w_shared",
        "x_indexed", "y_indexed", "scattered", "direction", "need_gw", "need_gx", "need_gy", "ctas_per_sm",
        "threads", "smem_bytes")]


class U1DGraph(C.Structure):
    _fields_ = [("n_edges", C.c_int64), ("n_out_rows", C.c_int64), ("x_rows", C.c_int64), ("y_rows", C.c_int64),
                ("x_index", C.c_void_p), ("y_index", C.c_void_p), ("seg_ptr", C.c_void_p), ("perm", C.c_void_p),
                ("part_ptr", C.c_void_p), ("n_parts", C.c_int32)]


def check(rc: int, lib=None, what: str = "") -> None:
    if rc != 0:
        detail = ""
        if rc == 3 and lib is not None:
            try:
                detail = ": " + lib.fasteq_last_cuda_error().decode()
            except Exception:
                pass
        raise FasteqError(f"{what} failed with status {rc} ({STATUS.get(rc, '?')}){detail}")


_core = None


def core():
    """Load libfasteq_b200_core.so (building it if the in-tree copy is missing or stale)."""
    global _core
    if _core is None:
        lib = C.CDLL(_build.build_core(), mode=C.RTLD_LOCAL)
        lib.fasteq_status_string.restype = C.c_char_p
        lib.fasteq_status_string.argtypes = [C.c_int]
        lib.fasteq_last_cuda_error.restype = C.c_char_p
        lib.fasteq_core_abi_version.restype = C.c_int
        lib.fasteq_graph_check_sorted.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
        lib.fasteq_graph_build_csr.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
        lib.fasteq_graph_partition.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]
        _core = lib
    return _core


class U1DModule:
    """One generated Uniform1D module (forward or backward of one signature)."""

    def __init__(self, so_path: str):
        self.path = so_path
        lib = C.CDLL(so_path, mode=C.RTLD_LOCAL)
        lib.fasteq_u1d_describe.argtypes = [C.POINTER(U1DDesc)]
        lib.fasteq_u1d_forward.argtypes = [C.POINTER(U1DGraph)] + [C.c_void_p] * 5
        lib.fasteq_u1d_backward.argtypes = [C.POINTER(U1DGraph)] + [C.c_void_p] * 8
        lib.fasteq_u1d_device_status.argtypes = [C.POINTER(C.c_int32)]
        lib.fasteq_last_cuda_error.restype = C.c_char_p
        if hasattr(lib, "fasteq_u1d_forward_noalloc"):   # forward modules only
            lib.fasteq_u1d_forward_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64] + [C.c_void_p] * 5
        self.lib = lib
        self.desc = U1DDesc()
        check(lib.fasteq_u1d_describe(C.byref(self.desc)), lib, "fasteq_u1d_describe")
        if self.desc.abi_version != 1:
            raise FasteqError(f"{so_path}: ABI version {self.desc.abi_version} != 1; rebuild the module")

    def forward(self, graph: U1DGraph, w: int, x: int, y: int, out: int, stream: int) -> None:
        check(self.lib.fasteq_u1d_forward(C.byref(graph), w, x, y, out, stream), self.lib, "fasteq_u1d_forward")

    def forward_noalloc(self, dst_sorted: int, x_index, n_edges: int, n_out_rows: int, x_rows: int,
                        w: int, x: int, y: int, out: int, stream: int) -> int:
        """Raw status of fasteq_u1d_forward_noalloc (the caller decides how to treat a refusal)."""
        return int(self.lib.fasteq_u1d_forward_noalloc(dst_sorted, x_index, n_edges, n_out_rows, x_rows, w, x, y, out, stream))

    def last_error(self) -> str:
        return self.lib.fasteq_last_cuda_error().decode()

    def backward(self, graph: U1DGraph, go: int, w: int, x: int, y: int, gw, gx, gy, stream: int) -> None:
        check(self.lib.fasteq_u1d_backward(C.byref(graph), go, w, x, y, gw, gx, gy, stream), self.lib,
              "fasteq_u1d_backward")

    def device_status(self) -> int:
        v = C.c_int32(0)
        check(self.lib.fasteq_u1d_device_status(C.byref(v)), self.lib, "fasteq_u1d_device_status")
        return int(v.value)
