"""Multi-GPU decomposition of the message-passing path (one process per GPU, torch.distributed).

Two regimes, neither of which exists in the reference (it has no communication code; its model
packages rely on an MD engine's ghost exchange, …/nequip/nn/_ghost_exchange_lmp_mliap.py:11-31):

* batches of independent structures: split by whole structure (``graph.split_structures``), no
  communication in the layer loop;
* one large graph: ``partition_by_receiver_range`` gives every rank a contiguous range of nodes and
  all edges whose receiver is in that range, so the scatter-sum is rank-local.  Senders outside the
  range are *ghosts*: before each interaction ``HaloExchange`` all-gathers the rows other ranks need
  (padded export slabs, data lands in local memory before any kernel reads it) and appends the
  ghost rows to the local ones; its backward sums the ghost gradients back onto their owners
  (reduce-scatter).  Positions go through the same exchange, so forces on owned atoms include the
  contributions of edges owned by other ranks.
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
    for r, (lo, hi, ids, src, dst, ghosts) in enumerate(per_rank):
        n_owned = hi - lo
        ghost_local = {int(g): n_owned + k for k, g in enumerate(ghosts)}
        src_local = np.array([s - lo if lo <= s < hi else ghost_local[int(s)] for s in src], dtype=np.int64)
        out.append(LocalGraph(r, world, lo, hi, ghosts.astype(np.int64), src_local, (dst - lo).astype(np.int64), ids.astype(np.int64),
                              (exports[r] - lo).astype(np.int64), max_export,
                              np.array([slot_of[int(g)] for g in ghosts], dtype=np.int64)))
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


class HaloExchange:
    """``ext = halo(x_owned)``: owned rows followed by ghost rows, differentiable."""

    def __init__(self, local: LocalGraph, device, group=None):
        self.local = local
        self.export_idx = torch.as_tensor(local.export_local, device=device)
        self.ghost_slot = torch.as_tensor(local.ghost_slot, device=device)
        self.group = group

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.local.world == 1:
            return x
        return _Halo.apply(x, self.export_idx, self.ghost_slot, self.local.max_export, self.group)


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
