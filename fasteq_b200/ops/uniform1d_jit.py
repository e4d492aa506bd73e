"""``fast_uniform1d_jit``: drop-in for fasteq/ops/uniform1d_jit.py:3328-3349.

Same call: ``fast_uniform1d_jit(w, x, y, input_indices, output_indices, meta)`` with
``input_indices = {1: src}`` (gather x), ``{2: src}`` (gather y), ``output_indices =
{0: dst}`` (scatter-sum the result), ``meta`` the reference's dict
(``i_list, j_list, k_list, v_list, coeff_list, w_seg_num, x_seg_num, y_seg_num,
out_seg_num, u_dim, size_list``).  Tensors are 2-D ``[rows, segments * u]`` in
ir_mul layout, CUDA, contiguous (a non-contiguous operand raises ``RuntimeError``
as in the reference; there is no CPU path).

Underneath, the path table is compiled into an sm_100a module (one per
signature, cached in-tree) and called through the C ABI of
include/fasteq_b200.h.  Scattered outputs use a receiver-sorted CSR plan that is
built once per index tensor and cached.
"""
from __future__ import annotations

import ctypes
import threading
from collections import OrderedDict
from contextlib import contextmanager
from typing import Dict, List, Optional, Set, Tuple

import numpy as np
import torch

from .. import _build, _cabi
from .. import tuning as _tuning
from ..codegen import u1d as _emit
from ..codegen.u1d_common import U1DSpec, make_spec

_EMITTER_VERSION = "u1d-v2"
_MODULES: Dict[Tuple, _cabi.U1DModule] = {}
_TUNING_OVERRIDE: Dict[str, _emit.Tuning] = {}
_lock = threading.Lock()


def _dtype_str(t: torch.Tensor) -> str:
    if t.dtype == torch.float32:
        return "f32"
    if t.dtype == torch.float64:
        return "f64"
    raise ValueError(f"fast_uniform1d_jit supports float32 and float64, got {t.dtype}")


def get_module(spec: U1DSpec, direction: str, needs=(False, False, False), tuning: Optional[_emit.Tuning] = None) -> _cabi.U1DModule:
    """Build (or load from the in-tree cache) the module of one signature."""
    tun = tuning or _TUNING_OVERRIDE.get(direction) or _tuning.lookup(spec, direction, needs) or _emit.default_tuning(spec, direction)
    key = (spec, direction, tuple(needs), tun)
    with _lock:
        mod = _MODULES.get(key)
    if mod is None:
        # compile outside the lock: different signatures build in parallel; the build itself is
        # atomic (temporary file + rename), so a duplicate build of one signature is harmless
        tag = spec.key(f"{_EMITTER_VERSION}|{direction}|{tuple(needs)}|{tun}")
        if direction == "fwd":
            source = _emit.emit_forward(spec, tun)
        else:
            source = _emit.emit_backward(spec, tun, *needs)
        so = _build.build_generated(f"u1d_{direction}_{tag}", source)
        with _lock:
            mod = _MODULES.get(key)
            if mod is None:
                mod = _cabi.U1DModule(so)
                _MODULES[key] = mod
    return mod


# ----------------------------------------------------------------------------- graph plan

class GraphPlan:
    """Receiver-sorted CSR view of a scatter index: sortedness, permutation, segment offsets
    and per-grid partitions.  Built once per index tensor (one host sync) and cached.  Each build step
    leaves an event behind it; ``ready_on_current_stream`` makes a later user on another stream wait for them."""

    def __init__(self, dst: torch.Tensor, n_rows: int, seg_ptr: Optional[torch.Tensor] = None):
        if dst.dim() != 1:
            raise ValueError("scatter index must be 1-D")
        core = _cabi.core()
        self.n_rows = int(n_rows)
        self.n_edges = int(dst.numel())
        dev = dst.device
        self._parts: Dict[int, torch.Tensor] = {}
        self._ready: List[Tuple[int, torch.cuda.Event]] = []
        self._waited: Set[int] = set()          # streams already ordered behind every event in _ready
        self.device = dev
        if seg_ptr is not None:
            # the caller vouches for a receiver-sorted index and brings its CSR offsets (the GPU
            # neighbour-list builder does): nothing to check, nothing to build, no host sync
            if seg_ptr.numel() != self.n_rows + 1 or seg_ptr.dtype != torch.int32 or seg_ptr.device != dev:
                raise ValueError("seg_ptr must be an int32 tensor of n_rows + 1 offsets on the index's device")
            self.sorted, self.perm, self.seg_ptr = True, None, seg_ptr.contiguous()
            return
        stream = torch.cuda.current_stream(dev).cuda_stream
        dst32 = dst.to(torch.int32).contiguous()
        flag = torch.empty(1, dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            _cabi.check(core.fasteq_graph_check_sorted(dst32.data_ptr(), self.n_edges, flag.data_ptr(), stream), core,
                        "fasteq_graph_check_sorted")
            self.sorted = bool(flag.item())
            if self.sorted:
                self.perm = None
                sorted_dst = dst32
            else:
                sorted_dst64, perm = torch.sort(dst32.to(torch.int64), stable=True)
                self.perm = perm.to(torch.int32).contiguous()
                sorted_dst = sorted_dst64.to(torch.int32).contiguous()
            self.seg_ptr = torch.empty(self.n_rows + 1, dtype=torch.int32, device=dev)
            _cabi.check(core.fasteq_graph_build_csr(sorted_dst.data_ptr(), self.n_edges, self.n_rows,
                                                    self.seg_ptr.data_ptr(), stream), core, "fasteq_graph_build_csr")
        self._mark_built()

    def _mark_built(self) -> None:
        cur = torch.cuda.current_stream(self.device)
        if torch.cuda.is_current_stream_capturing():
            return
        ev = torch.cuda.Event()
        ev.record(cur)
        self._ready = [(sid, e) for sid, e in self._ready if sid != cur.cuda_stream] + [(cur.cuda_stream, ev)]
        self._waited = set()

    def ready_on_current_stream(self) -> None:
        """Order the current stream behind the kernels that built this plan on other streams."""
        if not self._ready or torch.cuda.is_current_stream_capturing():
            return
        cur = torch.cuda.current_stream(self.device)
        if cur.cuda_stream in self._waited:
            return
        foreign = False
        for sid, ev in self._ready:
            if sid != cur.cuda_stream:
                cur.wait_event(ev)
                foreign = True
        if foreign:
            # a reader on a stream other than the building one: tell the allocator, so that an evicted
            # plan's buffers are not handed out again while this stream still reads them
            for t in (self.seg_ptr, self.perm, *self._parts.values()):
                if t is not None:
                    t.record_stream(cur)
        self._waited.add(cur.cuda_stream)

    def partition(self, n_parts: int) -> torch.Tensor:
        p = self._parts.get(n_parts)
        if p is None:
            core = _cabi.core()
            p = torch.empty(n_parts + 1, dtype=torch.int32, device=self.device)
            with torch.cuda.device(self.device):
                stream = torch.cuda.current_stream(self.device).cuda_stream
                _cabi.check(core.fasteq_graph_partition(self.seg_ptr.data_ptr(), self.n_rows, self.n_edges, n_parts,
                                                        p.data_ptr(), stream), core, "fasteq_graph_partition")
            self._parts[n_parts] = p
            self._mark_built()
        return p


_PLANS: "OrderedDict[Tuple, GraphPlan]" = OrderedDict()   # least recently used first
_PLAN_LIMIT = 64
_OWNED: Dict[str, Tuple] = {}          # owner tag -> key of the plan that owner registered last
_RECORDERS: List[list] = []            # lists that collect every plan a call uses (see record_plans)


def _plan_key(dst: torch.Tensor, n_rows: int) -> Tuple:
    return (dst.data_ptr(), dst.numel(), dst._version, str(dst.device), dst.dtype, int(n_rows))


def _insert_plan(key: Tuple, plan: GraphPlan) -> None:
    while len(_PLANS) >= _PLAN_LIMIT:
        _PLANS.popitem(last=False)
    _PLANS[key] = plan


def graph_plan(dst: torch.Tensor, n_rows: int) -> GraphPlan:
    """Cached plan of a scatter index.  The key is the index tensor's storage address, length and torch
    version counter: an index rewritten in place OUTSIDE torch's version tracking (memory shared with an
    engine through DLPack / ``from_blob``, a write through ``.data``) keeps its key, so such callers must
    treat index tensors as immutable or call ``invalidate_plan`` after every rewrite."""
    key = _plan_key(dst, n_rows)
    plan = _PLANS.get(key)
    if plan is None:
        plan = GraphPlan(dst, n_rows)
        plan._keepalive = dst  # the key is the storage address: keep it from being recycled
        _insert_plan(key, plan)
    else:
        _PLANS.move_to_end(key)
    return plan


def register_sorted_plan(dst: torch.Tensor, n_rows: int, seg_ptr: torch.Tensor, owner: Optional[str] = None) -> GraphPlan:
    """Install the plan of a receiver-sorted index whose CSR offsets are already known.  ``owner``: a tag of
    the caller that rebuilds its graph over and over (a neighbour-list builder): its previous plan is dropped
    instead of filling the cache with dead index tensors."""
    key = _plan_key(dst, n_rows)
    if owner is not None:
        old = _OWNED.get(owner)
        if old is not None and old != key:
            _PLANS.pop(old, None)
        _OWNED[owner] = key
    _PLANS.pop(key, None)
    plan = GraphPlan(dst, n_rows, seg_ptr)
    plan._keepalive = dst
    _insert_plan(key, plan)
    return plan


def invalidate_plan(dst: torch.Tensor) -> int:
    """Forget every cached plan of this index tensor's storage (after an in-place rewrite that torch's
    version counter does not see).  Returns the number of plans dropped."""
    hits = [k for k in _PLANS if k[0] == dst.data_ptr() and k[3] == str(dst.device)]
    for k in hits:
        del _PLANS[k]
    return len(hits)


@contextmanager
def record_plans():
    """Collect the plans used by the operator calls made inside the block.  A CUDA graph captured there
    bakes the plans' device pointers into its launches; whoever owns the graph must hold the collected
    plans for as long as the graph is replayed (the cache alone may evict them)."""
    got: list = []
    _RECORDERS.append(got)
    try:
        yield got
    finally:
        _RECORDERS.remove(got)


_SM_COUNT: Dict[int, int] = {}


def _sm_count(dev: torch.device) -> int:
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


# ----------------------------------------------------------------------------- helpers

def _validate(w, x, y):
    for name, t in (("w", w), ("x", x), ("y", y)):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a tensor")
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor: fasteq_b200 has no CPU path")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    if not (w.dtype == x.dtype == y.dtype):
        raise ValueError("w, x, y must share one dtype")


def _index32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if t.dtype != torch.int32:
        t = t.to(torch.int32)
    return t.contiguous()


class _Call:
    """Resolved shapes / indices / plan of one operator call, shared by forward and backward."""

    def __init__(self, w, x, y, input_indices, output_indices, meta):
        input_indices = {} if input_indices is None else input_indices
        output_indices = {} if output_indices is None else output_indices
        self.u = int(meta["u_dim"])
        self.w_segs, self.x_segs = int(meta["w_seg_num"]), int(meta["x_seg_num"])
        self.y_segs, self.out_segs = int(meta["y_seg_num"]), int(meta["out_seg_num"])
        size_list = meta["size_list"]
        # extension of the reference's meta: "y_sh" = (degrees, normalize, normalization) says that the y
        # operand holds edge vectors [rows, 3] whose spherical harmonics the kernel evaluates itself
        self.y_sh = tuple(meta["y_sh"]) if meta.get("y_sh") else ()
        y_cols = int(size_list[2]) // self.y_segs
        if y_cols not in (1, self.u):
            raise ValueError("y must carry 1 or u_dim values per segment")
        self.y_vec = y_cols != 1
        y_row = 3 if self.y_sh else self.y_segs * y_cols
        if self.y_sh and (self.y_vec or y.shape[-1] != 3):
            raise ValueError("with in-kernel spherical harmonics y must be the edge vectors [rows, 3]")
        for name, t, cols in (("w", w, self.w_segs * self.u), ("x", x, self.x_segs * self.u), ("y", y, y_row)):
            if t.dim() < 2 or t.numel() % cols != 0:
                raise ValueError(f"{name} has {t.numel()} elements, not a multiple of {cols}")
        self.w_rows, self.x_rows, self.y_rows = w.numel() // (self.w_segs * self.u), x.numel() // (self.x_segs * self.u), y.numel() // y_row
        self.x_indexed, self.y_indexed = 1 in input_indices, 2 in input_indices
        self.scattered = 0 in output_indices
        src = input_indices.get(1, input_indices.get(2))
        self.src = _index32(src)
        dst = output_indices.get(0)
        # row count of the per-edge operands: dst, else src, else x (uniform1d_forward.py:163-168)
        if dst is not None:
            self.n_edges = int(dst.numel())
        elif src is not None:
            self.n_edges = int(src.numel())
        else:
            self.n_edges = self.x_rows
        self.w_shared = self.w_rows == 1 and self.n_edges != 1
        if not self.w_shared and self.w_rows != self.n_edges:
            raise ValueError(f"w has {self.w_rows} rows for {self.n_edges} edges")
        if not self.x_indexed and self.x_rows != self.n_edges:
            raise ValueError("x rows must equal the edge count when x is not gathered")
        if not self.y_indexed and self.y_rows != self.n_edges:
            raise ValueError("y rows must equal the edge count when y is not gathered")
        # scattered output has as many rows as x (uniform1d_forward.py:109)
        self.n_out_rows = self.x_rows if self.scattered else self.n_edges
        self.plan = graph_plan(dst, self.n_out_rows) if self.scattered else None
        self.dtype = _dtype_str(w)
        skey = tuple((id(meta[k]), getattr(meta[k], "_version", 0)) for k in ("i_list", "j_list", "k_list", "v_list", "coeff_list")) + (
            self.w_segs, self.x_segs, self.y_segs, self.out_segs, self.u, self.dtype, self.y_vec, self.w_shared,
            self.x_indexed, self.y_indexed, self.scattered, self.y_sh)
        hit = _SPEC_CACHE.get(skey)
        if hit is None:
            spec = make_spec(
                _np(meta["i_list"]), _np(meta["j_list"]), _np(meta["k_list"]), _np(meta["v_list"]), _np(meta["coeff_list"], True),
                w_segs=self.w_segs, x_segs=self.x_segs, y_segs=self.y_segs, out_segs=self.out_segs, u=self.u,
                dtype=self.dtype, y_vec=self.y_vec, w_shared=self.w_shared, x_indexed=self.x_indexed,
                y_indexed=self.y_indexed, scattered=self.scattered, y_sh=self.y_sh)
            if len(_SPEC_CACHE) > 256:
                _SPEC_CACHE.clear()
            # the entry holds the table objects so their ids stay unique while it exists
            hit = (spec, [meta[k] for k in ("i_list", "j_list", "k_list", "v_list", "coeff_list")])
            _SPEC_CACHE[skey] = hit
        self.spec = hit[0]

    def graph(self, mod: _cabi.U1DModule, dev) -> _cabi.U1DGraph:
        g = _cabi.U1DGraph()
        g.n_edges, g.n_out_rows, g.x_rows, g.y_rows = self.n_edges, self.n_out_rows, self.x_rows, self.y_rows
        g.x_index = self.src.data_ptr() if self.x_indexed else None
        g.y_index = self.src.data_ptr() if self.y_indexed else None
        if self.plan is not None:
            g.seg_ptr = self.plan.seg_ptr.data_ptr()
            g.perm = self.plan.perm.data_ptr() if self.plan.perm is not None else None
            n_parts = max(1, min(_sm_count(dev) * int(mod.desc.ctas_per_sm), self.n_out_rows))
            g.part_ptr = self.plan.partition(n_parts).data_ptr()
            g.n_parts = n_parts
            self.plan.ready_on_current_stream()
            for rec in _RECORDERS:
                if not any(p is self.plan for p in rec):
                    rec.append(self.plan)
        return g


_META_CACHE: Dict[Tuple, Tuple[torch.Tensor, np.ndarray]] = {}


def _np(t, is_float=False) -> np.ndarray:
    """Host copy of a meta tensor.  Cached by storage identity; the cache keeps the tensor alive,
    so its address cannot be handed to another tensor while the entry exists."""
    if isinstance(t, torch.Tensor):
        key = (t.data_ptr(), t.numel(), t._version, t.dtype, str(t.device))
        hit = _META_CACHE.get(key)
        if hit is None:
            a = t.detach().cpu().numpy().astype(np.float64 if is_float else np.int64)
            if len(_META_CACHE) > 512:
                _META_CACHE.clear()
            _META_CACHE[key] = (t, a)
            return a
        return hit[1]
    return np.asarray(t, dtype=np.float64 if is_float else np.int64)


_SPEC_CACHE: Dict[Tuple, U1DSpec] = {}


def _tuning_for(spec: U1DSpec, direction: str, tensors, needs=(False, False, False)) -> Optional[_emit.Tuning]:
    """The launch configuration of this call: the measured winner of the signature when the tuning database has one,
    else the heuristic default.  Packed two-channel modules read and write 8-byte pairs; operands at an odd 4-byte
    offset (a contiguous view into a larger buffer) get the one-channel-per-thread module instead."""
    tun = _TUNING_OVERRIDE.get(direction) or _tuning.lookup(spec, direction, needs) or _emit.default_tuning(spec, direction)
    if tun.vec == 2 and any(t is not None and t.data_ptr() % 8 for t in tensors):
        import dataclasses
        return dataclasses.replace(tun, vec=1, pipes=1, groups=max(tun.groups, 1), min_blocks=min(tun.min_blocks + 1, 3))
    return tun


def _run_fwd(call: _Call, w, x, y) -> torch.Tensor:
    dev = x.device
    out = torch.empty((call.n_out_rows, call.out_segs * call.u), dtype=x.dtype, device=dev)
    mod = get_module(call.spec, "fwd", tuning=_tuning_for(call.spec, "fwd", (w, x, y, out)))
    with torch.cuda.device(dev):
        g = call.graph(mod, dev)
        mod.forward(g, w.data_ptr(), x.data_ptr(), y.data_ptr(), out.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    return out


def _run_bwd(call: _Call, grad_out, w, x, y, needs):
    dev = x.device
    gw = torch.empty_like(w) if needs[0] else None
    gx = torch.empty_like(x) if needs[1] else None
    gy = torch.empty_like(y) if needs[2] else None
    mod = get_module(call.spec, "bwd", needs, tuning=_tuning_for(call.spec, "bwd", (grad_out, w, x, y, gw, gx, gy), needs))
    ptr = lambda t: t.data_ptr() if t is not None else None
    with torch.cuda.device(dev):
        g = call.graph(mod, dev)
        mod.backward(g, grad_out.data_ptr(), w.data_ptr(), x.data_ptr(), y.data_ptr(), ptr(gw), ptr(gx), ptr(gy),
                     torch.cuda.current_stream(dev).cuda_stream)
    return gw, gx, gy


class FastUniform1dBackwardFunction(torch.autograd.Function):
    """First backward as a differentiable function (reference: fasteq/ops/uniform1d_jit.py:3098-3188),
    so that force losses can be trained.  The operator is trilinear in (w, x, y), hence every term of
    the second backward is again a forward or a one-gradient backward of the same signature with two
    operands swapped for incoming second-order gradients; no separate double-backward kernels exist:

        d_go = F(ggw, x, y) + F(w, ggx, y) + F(w, x, ggy)
        d_w  = Bw(go; ggx, y) + Bw(go; x, ggy)      (Bw = gradient with respect to the weight slot)
        d_x  = Bx(go; ggw, y) + Bx(go; w, ggy)
        d_y  = By(go; ggw, x) + By(go; w, ggx)
    """

    @staticmethod
    def forward(ctx, grad_out, w, x, y, call, needs):
        gw, gx, gy = _run_bwd(call, grad_out, w, x, y, needs)
        ctx.call, ctx.needs = call, needs
        ctx.save_for_backward(grad_out, w, x, y)
        ctx.set_materialize_grads(False)
        outs = tuple(g if g is not None else t.new_empty((0,)) for g, t in ((gw, w), (gx, x), (gy, y)))
        return outs

    @staticmethod
    def backward(ctx, ggw, ggx, ggy):
        go, w, x, y = ctx.saved_tensors
        call, needs = ctx.call, ctx.needs
        ggw = ggw.contiguous() if (ggw is not None and needs[0]) else None
        ggx = ggx.contiguous() if (ggx is not None and needs[1]) else None
        ggy = ggy.contiguous() if (ggy is not None and needs[2]) else None
        want_go, want_w, want_x, want_y = ctx.needs_input_grad[:4]

        def add(a, b):
            return b if a is None else (a if b is None else a + b)

        d_go = d_w = d_x = d_y = None
        if want_go:
            if ggw is not None:
                d_go = add(d_go, _run_fwd(call, ggw, x, y))
            if ggx is not None:
                d_go = add(d_go, _run_fwd(call, w, ggx, y))
            if ggy is not None:
                d_go = add(d_go, _run_fwd(call, w, x, ggy))
        if want_w:
            if ggx is not None:
                d_w = add(d_w, _run_bwd(call, go, w, ggx, y, (True, False, False))[0])
            if ggy is not None:
                d_w = add(d_w, _run_bwd(call, go, w, x, ggy, (True, False, False))[0])
        if want_x:
            if ggw is not None:
                d_x = add(d_x, _run_bwd(call, go, ggw, x, y, (False, True, False))[1])
            if ggy is not None:
                d_x = add(d_x, _run_bwd(call, go, w, x, ggy, (False, True, False))[1])
        if want_y:
            if ggw is not None:
                d_y = add(d_y, _run_bwd(call, go, ggw, x, y, (False, False, True))[2])
            if ggx is not None:
                d_y = add(d_y, _run_bwd(call, go, w, ggx, y, (False, False, True))[2])
        return d_go, d_w, d_x, d_y, None, None


class FastUniform1dJITFunction(torch.autograd.Function):
    """Autograd wrapper (reference: fasteq/ops/uniform1d_jit.py:3194-3326).  The backward produces
    exactly the gradients autograd asks for and is itself differentiable."""

    @staticmethod
    def forward(ctx, w, x, y, input_indices, output_indices, meta):
        _validate(w, x, y)
        call = _Call(w, x, y, input_indices, output_indices, meta)
        ctx.call = call
        ctx.save_for_backward(w, x, y)
        return _run_fwd(call, w, x, y)

    @staticmethod
    def backward(ctx, grad_out):
        w, x, y = ctx.saved_tensors
        needs = tuple(bool(n) for n in ctx.needs_input_grad[:3])
        if not any(needs):
            return None, None, None, None, None, None
        if ctx.call.y_sh:
            # not trilinear in the edge vector: the composed second backward does not apply
            if torch.is_grad_enabled() and any(t.requires_grad for t in (grad_out, w, x, y)):
                raise RuntimeError("fast_uniform1d_jit: no second-order gradient with in-kernel spherical harmonics; "
                                   "pass the harmonics as the y operand instead")
            gw, gx, gy = _run_bwd(ctx.call, grad_out.contiguous(), w, x, y, needs)
        else:
            gw, gx, gy = FastUniform1dBackwardFunction.apply(grad_out.contiguous(), w, x, y, ctx.call, needs)
        return (gw if needs[0] else None), (gx if needs[1] else None), (gy if needs[2] else None), None, None, None


def fast_uniform1d_jit(w, x, y, input_indices, output_indices, meta, use_multiwarp_candidates: Optional[bool] = None):
    """See module docstring.  ``use_multiwarp_candidates`` is accepted and ignored, as in the reference."""
    return FastUniform1dJITFunction.apply(w, x, y, input_indices, output_indices, meta)
