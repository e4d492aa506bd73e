"""Multi-GPU decomposition of the message-passing path (one process per GPU, torch.distributed).

Two regimes, neither of which exists in the reference (it has no communication code; its model
packages rely on an MD engine's ghost exchange, …/nequip/nn/_ghost_exchange_lmp_mliap.py:11-31):

* batches of independent structures: split by whole structure (``graph.split_structures``), no
  communication in the layer loop;
* one large graph: ``partition_by_receiver_range`` gives every rank a contiguous range of nodes and
  all edges whose receiver is in that range, so the scatter-sum is rank-local.  Senders outside the
  range are *ghosts*: before each interaction ``HaloExchange`` sends every peer exactly the owned rows
  that peer reads (one variable-size all-to-all: a slab partition has two neighbours, and only they
  get data; it lands in local memory before any kernel reads it) and appends the received ghost rows
  to the local ones; its backward sends the ghost gradients back the same way and adds them onto
  their owners.  Positions go through the same exchange, so forces on owned atoms include the
  contributions of edges owned by other ranks.  (``mode="gather"`` keeps the earlier form: padded
  export slabs all-gathered to every rank, reduce-scatter in the backward.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist


@dataclass
class LocalGraph:
    """What one rank holds of a partitioned graph.  Local node ids: owned nodes first (global ids
    ``start .. stop-1`` in order), then ghosts in the order of ``ghost_global``."""
    rank: int
    world: int
    start: int
    stop: int
    ghost_global: np.ndarray          # [G] global ids of the ghost nodes
    edge_src: np.ndarray              # [E_local] local sender ids (may point at ghosts)
    edge_dst: np.ndarray              # [E_local] local receiver ids (< n_owned), non-decreasing
    edge_ids: np.ndarray              # [E_local] ids of these edges in the global edge list
    export_local: np.ndarray          # [X] owned rows (local ids) this rank exports, sorted
    max_export: int                   # slab rows per rank (max over ranks)
    ghost_slot: np.ndarray            # [G] position of each ghost in the gathered [world * max_export] slab
    send_idx: np.ndarray = None       # [sum(send_counts)] owned rows (local ids) to send, grouped by receiving rank
    send_counts: tuple = ()           # rows sent to each rank
    recv_counts: tuple = ()           # ghost rows received from each rank; in rank order they ARE the ghosts in order

    @property
    def n_owned(self) -> int:
        return self.stop - self.start

    @property
    def n_local(self) -> int:
        return self.n_owned + len(self.ghost_global)


def node_ranges(n_nodes: int, world: int, edge_dst: Optional[np.ndarray] = None) -> List[int]:
    """Contiguous node ranges with about equal edge counts (or node counts without an edge list)."""
    if edge_dst is None or len(edge_dst) == 0:
        return [n_nodes * r // world for r in range(world + 1)]
    counts = np.bincount(edge_dst, minlength=n_nodes).astype(np.int64) + 1
    cum = np.concatenate([[0], np.cumsum(counts)])
    bounds = [0]
    for r in range(1, world):
        bounds.append(int(np.searchsorted(cum, cum[-1] * r / world)))
    bounds.append(n_nodes)
    return [max(b, bounds[i - 1]) if i else b for i, b in enumerate(bounds)]


def partition_by_receiver_range(n_nodes: int, edge_src: np.ndarray, edge_dst: np.ndarray, world: int,
                                bounds: Optional[List[int]] = None) -> List[LocalGraph]:
    """Partition for every rank (host side; each rank normally keeps only its own entry)."""
    bounds = bounds or node_ranges(n_nodes, world, edge_dst)
    owner = np.searchsorted(np.asarray(bounds[1:]), np.arange(n_nodes), side="right")
    per_rank = []
    needed_by_any: List[set] = [set() for _ in range(world)]   # rows of rank r that someone else needs
    for r in range(world):
        lo, hi = bounds[r], bounds[r + 1]
        mask = (edge_dst >= lo) & (edge_dst < hi)
        ids = np.nonzero(mask)[0]
        order = np.argsort(edge_dst[ids], kind="stable")
        ids = ids[order]
        src, dst = edge_src[ids], edge_dst[ids]
        ghosts = np.unique(src[(src < lo) | (src >= hi)])
        for g in ghosts:
            needed_by_any[owner[g]].add(int(g))
        per_rank.append((lo, hi, ids, src, dst, ghosts))
    exports = [np.array(sorted(s), dtype=np.int64) for s in needed_by_any]
    max_export = max([len(e) for e in exports] + [1])
    slot_of = {}
    for r, e in enumerate(exports):
        for k, g in enumerate(e):
            slot_of[int(g)] = r * max_export + k
    out = []
    # per-peer tables: ghosts are sorted by global id and ownership ranges are contiguous, so a rank's ghosts are
    # already grouped by owner in rank order; owner q sends rank r the rows r's ghost list names, in that order
    need = [[ghosts[owner[ghosts] == q] if len(ghosts) else ghosts for q in range(world)] for (_, _, _, _, _, ghosts) in per_rank]
    for r, (lo, hi, ids, src, dst, ghosts) in enumerate(per_rank):
        n_owned = hi - lo
        ghost_pos = np.searchsorted(ghosts, src)
        ghost_pos = np.minimum(ghost_pos, max(len(ghosts) - 1, 0))
        inside = (src >= lo) & (src < hi)
        src_local = np.where(inside, src - lo, n_owned + ghost_pos).astype(np.int64)
        send = [need[q][r] - lo for q in range(world)]                    # what every rank q reads of r's rows
        out.append(LocalGraph(r, world, lo, hi, ghosts.astype(np.int64), src_local, (dst - lo).astype(np.int64), ids.astype(np.int64),
                              (exports[r] - lo).astype(np.int64), max_export,
                              np.array([slot_of[int(g)] for g in ghosts], dtype=np.int64),
                              np.concatenate(send).astype(np.int64) if world else np.zeros(0, np.int64),
                              tuple(int(len(t)) for t in send), tuple(int(len(need[r][q])) for q in range(world))))
    return out


class _Halo(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, export_idx, ghost_slot, max_export, group):
        world = dist.get_world_size(group)
        slab = x.new_zeros((max_export,) + x.shape[1:])
        slab[: export_idx.numel()] = x[export_idx]
        gathered = x.new_empty((world * max_export,) + x.shape[1:])
        dist.all_gather_into_tensor(gathered, slab.contiguous(), group=group)
        ctx.save_for_backward(export_idx, ghost_slot)
        ctx.meta = (max_export, group, x.shape[0])
        return torch.cat([x, gathered[ghost_slot]], dim=0)

    @staticmethod
    def backward(ctx, grad):
        export_idx, ghost_slot = ctx.saved_tensors
        max_export, group, n_owned = ctx.meta
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        buf = grad.new_zeros((world * max_export,) + grad.shape[1:])
        buf.index_add_(0, ghost_slot, grad[n_owned:])
        mine = grad.new_empty((max_export,) + grad.shape[1:])
        if dist.get_backend(group) == "nccl":
            dist.reduce_scatter_tensor(mine, buf, op=dist.ReduceOp.SUM, group=group)
        else:  # gloo has no reduce-scatter: all-reduce, then take this rank's slab
            dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
            mine = buf[rank * max_export:(rank + 1) * max_export]
        gx = grad[:n_owned].clone()
        gx.index_add_(0, export_idx, mine[: export_idx.numel()])
        return gx, None, None, None, None


class _HaloA2A(torch.autograd.Function):
    """Neighbour-only exchange: ``out = [x ; rows received]`` with one variable-size all-to-all.  The received rows,
    taken in rank order, are the ghost rows in local order, so nothing is re-indexed on arrival.  With ``defer`` the
    collective is left in flight and its handle is parked in ``pending``: the caller does node-local work and then
    calls ``HaloExchange.end`` before the first use of the ghost rows."""

    @staticmethod
    def forward(ctx, x, send_idx, send_counts, recv_counts, group, pending):
        n_owned, n_ghost = x.shape[0], int(sum(recv_counts))
        out = x.new_empty((n_owned + n_ghost,) + x.shape[1:])
        out[:n_owned] = x
        send = x.index_select(0, send_idx) if send_idx.numel() else x.new_empty((0,) + x.shape[1:])
        work = dist.all_to_all_single(out[n_owned:], send, list(recv_counts), list(send_counts), group=group,
                                      async_op=pending is not None)
        if pending is not None:
            pending.append((work, send))         # keeps the send buffer alive until the wait
        ctx.save_for_backward(send_idx)
        ctx.meta = (send_counts, recv_counts, group, n_owned)
        return out

    @staticmethod
    def backward(ctx, grad):
        (send_idx,) = ctx.saved_tensors
        send_counts, recv_counts, group, n_owned = ctx.meta
        ghost_grad = grad[n_owned:].contiguous()
        back = grad.new_empty((int(sum(send_counts)),) + grad.shape[1:])
        dist.all_to_all_single(back, ghost_grad, list(send_counts), list(recv_counts), group=group)
        gx = grad[:n_owned].clone()
        if send_idx.numel():
            gx.index_add_(0, send_idx, back)
        return gx, None, None, None, None, None


class HaloExchange:
    """``ext = halo(x_owned)``: owned rows followed by ghost rows, differentiable.

    ``begin`` / ``end`` split the call so that node-local work can run behind the exchange::

        t = halo.begin(x_owned)        # pack + start the all-to-all
        y = node_local_work(h)         # e.g. the self-connection, independent of the ghost rows
        ext = halo.end(t)              # wait; ghost rows are valid from here on
    """

    def __init__(self, local: LocalGraph, device, group=None, mode: str = "auto"):
        """``mode``: ``"alltoall"`` (neighbour-only exchange: least data), ``"gather"`` (padded slabs to every rank: one
        collective call, least host work) or ``"auto"``: the all-to-all while a CUDA graph is being captured -- a replayed
        step is bound by the GPU, so bytes matter -- and the gather in eager execution on CUDA, where at a few thousand
        atoms per rank the step is bound by the host's launch rate and a variable-size all-to-all (one send / receive
        pair per peer) costs several times the host time of a single all-gather.  Both deliver the same ghost rows."""
        if mode not in ("alltoall", "gather", "auto"):
            raise ValueError("mode must be 'alltoall', 'gather' or 'auto'")
        self.local, self.mode = local, mode
        self.export_idx = torch.as_tensor(local.export_local, device=device)
        self.ghost_slot = torch.as_tensor(local.ghost_slot, device=device)
        self.send_idx = torch.as_tensor(local.send_idx if local.send_idx is not None else np.zeros(0, np.int64), device=device)
        self.group = group
        self._pending: list = []

    def _gathers(self, x: torch.Tensor) -> bool:
        if self.mode != "auto":
            return self.mode == "gather"
        return x.is_cuda and not torch.cuda.is_current_stream_capturing()

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.local.world == 1:
            return x
        if self._gathers(x):
            return _Halo.apply(x, self.export_idx, self.ghost_slot, self.local.max_export, self.group)
        return _HaloA2A.apply(x, self.send_idx, self.local.send_counts, self.local.recv_counts, self.group, None)

    def begin(self, x: torch.Tensor) -> torch.Tensor:
        # inside a capture the exchange is issued in line: measured at 4 ranks, forking it there gains nothing
        if self.local.world == 1 or self._gathers(x) or (x.is_cuda and torch.cuda.is_current_stream_capturing()):
            return self(x)
        return _HaloA2A.apply(x, self.send_idx, self.local.send_counts, self.local.recv_counts, self.group, self._pending)

    def end(self, ext: torch.Tensor) -> torch.Tensor:
        while self._pending:
            work, _ = self._pending.pop()
            if work is not None:
                work.wait()
        return ext


class _EngineExchange(torch.autograd.Function):
    """Ghost rows filled by an MD engine's communication, differentiable: the forward hands the engine a
    buffer of ``ntotal`` rows whose first ``nlocal`` hold the owned values and lets it fill the rest; the
    backward hands it the gradient of all rows and gets back the owners' sums.  The engine object follows the
    protocol of LAMMPS ML-IAP data as the reference's models use it
    (.../nequip/nn/_ghost_exchange_lmp_mliap.py:11-31): ``nlocal``, ``ntotal``,
    ``forward_exchange(src [ntotal, w], dst [ntotal, w], w)``, ``reverse_exchange(grad [ntotal, w], dst [ntotal, w], w)``."""

    @staticmethod
    def forward(ctx, x_owned, engine):
        nlocal, ntotal = int(engine.nlocal), int(engine.ntotal)
        if x_owned.shape[0] != nlocal:
            raise ValueError(f"engine exchange: {x_owned.shape[0]} owned rows given, the engine owns {nlocal}")
        width = 1
        for d in x_owned.shape[1:]:
            width *= int(d)
        flat = x_owned.reshape(nlocal, width)          # explicit width: a rank may own no atoms
        src = torch.zeros((ntotal, flat.shape[1]), dtype=flat.dtype, device=flat.device)
        src[:nlocal] = flat
        out = torch.empty_like(src)
        engine.forward_exchange(src, out, out.shape[1])
        ctx.engine, ctx.nlocal, ctx.tail, ctx.width = engine, nlocal, x_owned.shape[1:], width
        return out.reshape((ntotal,) + tuple(x_owned.shape[1:]))

    @staticmethod
    def backward(ctx, grad_ext):
        g = grad_ext.reshape(grad_ext.shape[0], ctx.width).contiguous()
        out = torch.empty_like(g)
        ctx.engine.reverse_exchange(g, out, out.shape[1])
        return out[: ctx.nlocal].reshape((ctx.nlocal,) + tuple(ctx.tail)), None


class EngineGhostExchange:
    """``ext = halo(x_owned)`` with the ghost rows supplied by an MD engine (same calling convention as
    ``HaloExchange``, so the models' ``halo=`` hook takes either)."""

    def __init__(self, engine):
        self.engine = engine

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if int(self.engine.ntotal) == int(self.engine.nlocal):
            return x
        return _EngineExchange.apply(x, self.engine)

    # an engine's exchange is synchronous: begin does the whole call
    begin = __call__

    def end(self, ext: torch.Tensor) -> torch.Tensor:
        return ext
