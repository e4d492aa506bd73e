"""Host-side synthetic structures and neighbour lists for the benchmark configurations.

Periodic cubic boxes with uniformly placed atoms and a radius graph (both
directions, no self edges), ordered by (receiver, sender, image) so that edges
arrive receiver-sorted -- the order the CSR kernels want.  Pure numpy; this is
input preparation, not part of the timed path (model packages do this step with
ASE / matscipy outside the reference as well).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

import numpy as np


@dataclass
class Batch:
    positions: np.ndarray   # [N, 3] float64
    species: np.ndarray     # [N] int64
    edge_src: np.ndarray    # [E] int64 (sender)
    edge_dst: np.ndarray    # [E] int64 (receiver), non-decreasing
    edge_vec: np.ndarray    # [E, 3] float64, r_src + shift - r_dst
    edge_shift: np.ndarray  # [E, 3] float64 periodic image offset (cartesian) of the sender
    node_graph: np.ndarray  # [N] structure id of each atom
    n_graphs: int

    @property
    def n_nodes(self) -> int:
        return int(self.positions.shape[0])

    @property
    def n_edges(self) -> int:
        return int(self.edge_src.shape[0])


def periodic_radius_graph(pos: np.ndarray, side, cutoff: float):
    """All pairs (sender j, receiver i, image) with |r_j + shift - r_i| < cutoff in a periodic box
    (``side``: one length for a cube, or three for an orthorhombic box)."""
    n = pos.shape[0]
    side = np.broadcast_to(np.asarray(side, dtype=np.float64), (3,))
    rngs = [np.arange(-int(np.ceil(cutoff / s)), int(np.ceil(cutoff / s)) + 1) for s in side]
    images = np.stack(np.meshgrid(*rngs, indexing="ij"), -1).reshape(-1, 3).astype(np.float64) * side
    src_l, dst_l, vec_l, sh_l = [], [], [], []
    c2 = cutoff * cutoff
    for img in images:
        d = pos[None, :, :] + img[None, None, :] - pos[:, None, :]   # [i (receiver), j (sender), 3]
        r2 = (d * d).sum(-1)
        mask = r2 < c2
        if not img.any():
            np.fill_diagonal(mask, False)
        i, j = np.nonzero(mask)
        src_l.append(j); dst_l.append(i); vec_l.append(d[i, j]); sh_l.append(np.broadcast_to(img, (i.size, 3)))
    src = np.concatenate(src_l); dst = np.concatenate(dst_l)
    vec = np.concatenate(vec_l); sh = np.concatenate(sh_l)
    order = np.lexsort((sh[:, 2], sh[:, 1], sh[:, 0], src, dst))
    return src[order], dst[order], vec[order], sh[order]


def periodic_radius_graph_cells(pos: np.ndarray, side: float, cutoff: float):
    """Same result as ``periodic_radius_graph`` for ``cutoff <= side / 3``, by a cell list: O(N) memory.

    Atoms are binned into cubic cells at least ``cutoff`` wide; every cell is compared with its 27
    neighbours (periodic wrap carries the image shift)."""
    n = pos.shape[0]
    ncell = int(np.floor(side / cutoff))
    if ncell < 3:
        return periodic_radius_graph(pos, side, cutoff)
    w = side / ncell
    cell = np.minimum((pos / w).astype(np.int64), ncell - 1)
    cid = (cell[:, 0] * ncell + cell[:, 1]) * ncell + cell[:, 2]
    order = np.argsort(cid, kind="stable")
    cstart = np.searchsorted(cid[order], np.arange(ncell ** 3 + 1))
    maxocc = int(np.diff(cstart).max())
    # padded [cells, maxocc] table of atom ids (-1 = empty)
    table = np.full((ncell ** 3, maxocc), -1, dtype=np.int64)
    occ = np.arange(n) - cstart[cid[order]]
    table[cid[order], occ] = order
    c2 = cutoff * cutoff
    src_l, dst_l, vec_l, sh_l = [], [], [], []
    cx, cy, cz = np.meshgrid(np.arange(ncell), np.arange(ncell), np.arange(ncell), indexing="ij")
    base = np.stack([cx, cy, cz], -1).reshape(-1, 3)
    for off in np.stack(np.meshgrid([-1, 0, 1], [-1, 0, 1], [-1, 0, 1], indexing="ij"), -1).reshape(-1, 3):
        nb = base + off
        wrap = np.floor_divide(nb, ncell)
        nbw = nb - wrap * ncell
        nid = (nbw[:, 0] * ncell + nbw[:, 1]) * ncell + nbw[:, 2]
        shift = wrap.astype(np.float64) * side                      # image offset of the sender cell
        recv = table                                                # [C, m] receivers in the cell
        send = table[nid]                                           # [C, m] senders in the neighbour cell
        valid = (recv[:, :, None] >= 0) & (send[:, None, :] >= 0)
        pr = pos[np.maximum(recv, 0)]                               # [C, m, 3]
        ps = pos[np.maximum(send, 0)] + shift[:, None, :]
        d = ps[:, None, :, :] - pr[:, :, None, :]                   # [C, m_recv, m_send, 3]
        r2 = (d * d).sum(-1)
        mask = valid & (r2 < c2) & ~((recv[:, :, None] == send[:, None, :]) & (np.abs(shift).sum(-1) == 0)[:, None, None])
        ci, ri, si = np.nonzero(mask)
        src_l.append(send[ci, si]); dst_l.append(recv[ci, ri]); vec_l.append(d[ci, ri, si]); sh_l.append(shift[ci])
    src = np.concatenate(src_l); dst = np.concatenate(dst_l); vec = np.concatenate(vec_l); sh = np.concatenate(sh_l)
    order = np.lexsort((sh[:, 2], sh[:, 1], sh[:, 0], src, dst))
    return src[order], dst[order], vec[order], sh[order]


def large_box(n_atoms: int = 20000, side: float = 58.5, cutoff: float = 4.0, n_species: int = 2, seed: int = 0) -> Batch:
    """benchmark configuration 3 data: one periodic cube, atoms sorted along a space-filling order of the
    cells so that contiguous node ranges are spatially compact (small halos)."""
    rng = np.random.default_rng(seed)
    pos = rng.uniform(0.0, side, size=(n_atoms, 3))
    ncell = max(1, int(np.floor(side / cutoff)))
    cell = np.minimum((pos / (side / ncell)).astype(np.int64), ncell - 1)
    order = np.lexsort((cell[:, 2], cell[:, 1], cell[:, 0]))         # slabs along x, then y, then z
    pos = pos[order]
    spec = rng.integers(0, n_species, size=n_atoms)
    s, d, v, sh = periodic_radius_graph_cells(pos, side, cutoff)
    return Batch(pos, spec, s, d, v, sh, np.zeros(n_atoms, dtype=np.int64), 1)


def make_boxes(n_boxes: int, atoms, side, cutoff: float, n_species: int, seed: int = 0) -> Batch:
    """``atoms`` / ``side`` may be scalars or per-box sequences."""
    rng = np.random.default_rng(seed)
    atoms = np.broadcast_to(np.asarray(atoms), (n_boxes,))
    side = np.broadcast_to(np.asarray(side, dtype=np.float64), (n_boxes,))
    P, S, SRC, DST, VEC, SH, NG = [], [], [], [], [], [], []
    off = 0
    for b in range(n_boxes):
        n = int(atoms[b])
        pos = rng.uniform(0.0, float(side[b]), size=(n, 3))
        spec = rng.integers(0, n_species, size=n)
        s, d, v, sh = periodic_radius_graph(pos, float(side[b]), cutoff)
        P.append(pos); S.append(spec); SRC.append(s + off); DST.append(d + off); VEC.append(v); SH.append(sh)
        NG.append(np.full(n, b))
        off += n
    return Batch(np.concatenate(P), np.concatenate(S), np.concatenate(SRC), np.concatenate(DST), np.concatenate(VEC),
                 np.concatenate(SH), np.concatenate(NG), n_boxes)


def config1_batch(n_boxes: int = 64, seed: int = 0) -> Batch:
    """benchmark configuration 1 data: periodic cubic boxes of side 12.4 A, 192 atoms, 4 species, cutoff 5 A."""
    return make_boxes(n_boxes, 192, 12.4, 5.0, 4, seed)


def split_structures(edge_counts: np.ndarray, n_ranks: int) -> List[List[int]]:
    """Greedy longest-first assignment of whole structures to ranks, balanced by edge count."""
    order = np.argsort(-np.asarray(edge_counts), kind="stable")
    loads = [0] * n_ranks
    out: List[List[int]] = [[] for _ in range(n_ranks)]
    for s in order:
        r = loads.index(min(loads))
        out[r].append(int(s))
        loads[r] += int(edge_counts[s])
    return [sorted(o) for o in out]
