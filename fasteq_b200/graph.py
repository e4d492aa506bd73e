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


def periodic_radius_graph(pos: np.ndarray, side: float, cutoff: float):
    """All pairs (sender j, receiver i, image) with |r_j + shift - r_i| < cutoff in a cubic box."""
    n = pos.shape[0]
    reach = int(np.ceil(cutoff / side))
    rng = np.arange(-reach, reach + 1)
    images = np.stack(np.meshgrid(rng, rng, rng, indexing="ij"), -1).reshape(-1, 3).astype(np.float64) * side
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
    """BASELINE config 1 data: periodic cubic boxes of side 12.4 A, 192 atoms, 4 species, cutoff 5 A."""
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
