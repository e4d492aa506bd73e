"""Periodic radius graph built on the GPU (``fasteq_neighbors_*``): receiver-sorted edges in the
canonical (receiver, sender, image) order of ``fasteq_b200.graph.periodic_radius_graph`` plus the CSR
offsets, registered as a ready graph plan so that the tensor-product operator needs neither a
sortedness check nor a CSR build for the returned receiver index."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _cabi

MAX_DEGREE = 1024


class _Problem(C.Structure):
    _fields_ = [("n_atoms", C.c_int64), ("n_structs", C.c_int32), ("cutoff", C.c_double), ("pos", C.c_void_p),
                ("atom_struct", C.c_void_p), ("box", C.POINTER(C.c_double))]


_ready = False


def _lib():
    global _ready
    lib = _cabi.core()
    if not _ready:
        pp = C.POINTER(_Problem)
        lib.fasteq_neighbors_work_bytes.argtypes = [pp, C.POINTER(C.c_int64)]
        lib.fasteq_neighbors_count.argtypes = [pp, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.fasteq_neighbors_fill.argtypes = [pp, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        _ready = True
    return lib


@dataclass
class RadiusGraph:
    edge_src: torch.Tensor     # [E] int32 sender
    edge_dst: torch.Tensor     # [E] int32 receiver, non-decreasing
    edge_shift: torch.Tensor   # [E, 3] float64 cartesian image offset of the sender
    seg_ptr: torch.Tensor      # [N + 1] int32 CSR offsets of edge_dst
    max_degree: int


def radius_graph(pos: torch.Tensor, atom_struct: torch.Tensor, box, cutoff: float, register_plan: bool = True) -> RadiusGraph:
    """``pos [N, 3]`` (CUDA, wrapped into the box; evaluated in float64), ``atom_struct [N]`` structure id of
    each atom, ``box [S, 3]`` (or ``[S]`` for cubes) host array of box lengths.  One host sync (the edge count)."""
    if not pos.is_cuda:
        raise RuntimeError("radius_graph: pos must be a CUDA tensor: fasteq_b200 has no CPU path (use fasteq_b200.graph on the host)")
    box = np.ascontiguousarray(np.asarray(box, dtype=np.float64))
    if box.ndim == 1:
        box = np.repeat(box[:, None], 3, axis=1).copy()
    S = box.shape[0]
    N = int(pos.shape[0])
    p64 = pos.detach().to(torch.float64).contiguous()
    st = atom_struct.to(device=pos.device, dtype=torch.int32).contiguous()
    prob = _Problem(N, S, float(cutoff), p64.data_ptr(), st.data_ptr(), box.ctypes.data_as(C.POINTER(C.c_double)))
    lib = _lib()
    nbytes = C.c_int64(0)
    _cabi.check(lib.fasteq_neighbors_work_bytes(C.byref(prob), C.byref(nbytes)), lib, "fasteq_neighbors_work_bytes")
    dev = pos.device
    work = torch.empty(int(nbytes.value), dtype=torch.uint8, device=dev)
    seg_ptr = torch.empty(N + 1, dtype=torch.int32, device=dev)
    head = torch.zeros(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _cabi.check(lib.fasteq_neighbors_count(C.byref(prob), work.data_ptr(), nbytes.value, seg_ptr.data_ptr(), head.data_ptr(), stream),
                    lib, "fasteq_neighbors_count")
        n_edges, max_deg = (int(v) for v in torch.stack([seg_ptr[N], head[0]]).tolist())
        if max_deg > MAX_DEGREE:
            raise RuntimeError(f"radius_graph: an atom has {max_deg} neighbours, more than the {MAX_DEGREE} the builder sorts")
        src = torch.empty(n_edges, dtype=torch.int32, device=dev)
        dst = torch.empty(n_edges, dtype=torch.int32, device=dev)
        shift = torch.empty((n_edges, 3), dtype=torch.float64, device=dev)
        if n_edges > 0:
            _cabi.check(lib.fasteq_neighbors_fill(C.byref(prob), work.data_ptr(), nbytes.value, seg_ptr.data_ptr(), src.data_ptr(),
                                                  dst.data_ptr(), shift.data_ptr(), stream), lib, "fasteq_neighbors_fill")
    if register_plan:
        from .ops.uniform1d_jit import register_sorted_plan
        register_sorted_plan(dst, N, seg_ptr, owner=f"radius_graph:{dev}")
    return RadiusGraph(src, dst, shift, seg_ptr, max_deg)
