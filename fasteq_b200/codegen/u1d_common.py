"""Table analysis shared by the Uniform1D forward / backward emitters.

A Uniform1D table is a list of paths ``(i, j, k, v, c)``:
``out[v] += c * w[i] * x[j] * y[k]``.  The emitters evaluate it in the factored form

    out[v] += w[i] * sum_{paths of (i, v)} c * (x[j] * y[k])

and share every product ``x[j] * y[k]`` between the paths that use it.  Terms
``(i, v)`` whose paths share products are collected into *blocks* (for a table
that came from e3nn instructions a block is one ``(l1, l2)`` pair), so the
products of a block live in registers only while that block is evaluated.
The reference reaches the same kind of reuse with a greedy load-order
scheduler (fasteq/ops/auto_schedule/schedulers.py:34-673); this is a static
factorisation instead.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import numpy as np


@dataclass(frozen=True)
class U1DSpec:
    """Everything that selects one generated module (its signature)."""
    paths: Tuple[Tuple[int, int, int, int, float], ...]
    w_segs: int
    x_segs: int
    y_segs: int
    out_segs: int
    u: int
    dtype: str = "f32"          # "f32" | "f64"
    y_vec: bool = False         # y carries a channel axis ("u,u,u,u"); else one scalar per segment ("u,u,,u")
    w_shared: bool = False      # weights have one row shared by all edges
    x_indexed: bool = True      # x rows gathered through an index
    y_indexed: bool = False     # y rows gathered through an index
    scattered: bool = True      # output rows summed over the edges of a receiver segment
    y_sh: tuple = ()            # (degrees, normalize, normalization): y rows are edge vectors [rows, 3] and the
                                # kernel evaluates their spherical harmonics itself (scalar-y mode only)

    def __hash__(self) -> int:
        # specs key the module and tuning caches on every operator call; the path table has hundreds of entries, so its
        # hash is computed once per object
        h = self.__dict__.get("_hash")
        if h is None:
            h = hash((self.paths, self.w_segs, self.x_segs, self.y_segs, self.out_segs, self.u, self.dtype, self.y_vec,
                      self.w_shared, self.x_indexed, self.y_indexed, self.scattered, self.y_sh))
            object.__setattr__(self, "_hash", h)
        return h

    @property
    def ctype(self) -> str:
        return "float" if self.dtype == "f32" else "double"

    @property
    def elem_bytes(self) -> int:
        return 4 if self.dtype == "f32" else 8

    def key(self, extra: str = "") -> str:
        h = hashlib.sha256()
        h.update(repr((self.paths, self.w_segs, self.x_segs, self.y_segs, self.out_segs, self.u, self.dtype,
                       self.y_vec, self.w_shared, self.x_indexed, self.y_indexed, self.scattered, self.y_sh, extra)).encode())
        return h.hexdigest()[:16]


def make_spec(i_list, j_list, k_list, v_list, coeff_list, *, w_segs, x_segs, y_segs, out_segs, u, dtype,
              y_vec=False, w_shared=False, x_indexed=True, y_indexed=False, scattered=True, y_sh=()) -> U1DSpec:
    cs = np.asarray(coeff_list, dtype=np.float64)
    if dtype == "f32":
        cs = cs.astype(np.float32).astype(np.float64)  # the literal the kernel will hold
    paths = tuple((int(i), int(j), int(k), int(v), float(c)) for i, j, k, v, c in zip(i_list, j_list, k_list, v_list, cs))
    for (i, j, k, v, _) in paths:
        if not (0 <= i < w_segs and 0 <= j < x_segs and 0 <= k < y_segs and 0 <= v < out_segs):
            raise ValueError("path index outside its operand's segment count")
    if y_sh:
        ls, normalize, normalization = y_sh
        y_sh = (tuple(int(l) for l in ls), bool(normalize), str(normalization))
        if y_vec or y_indexed:
            raise ValueError("in-kernel spherical harmonics need a per-edge scalar y operand (no channel axis, no gather)")
        if sum(2 * l + 1 for l in y_sh[0]) != int(y_segs):
            raise ValueError("the spherical-harmonic degrees do not add up to the y segment count")
    return U1DSpec(paths, int(w_segs), int(x_segs), int(y_segs), int(out_segs), int(u), dtype,
                   bool(y_vec), bool(w_shared), bool(x_indexed), bool(y_indexed), bool(scattered), tuple(y_sh))


@dataclass
class Term:
    i: int
    v: int
    items: List[Tuple[int, int, float]]  # (j, k, c)


@dataclass
class Block:
    terms: List[Term]
    products: List[Tuple[int, int]]  # (j, k) pairs, sorted

    @property
    def cost(self) -> int:
        return len(self.products) + sum(len(t.items) + 1 for t in self.terms)


def build_blocks(spec: U1DSpec) -> List[Block]:
    """Group paths into (i, v) terms and terms into product-sharing blocks (union-find on (j, k))."""
    terms: Dict[Tuple[int, int], Term] = {}
    for (i, j, k, v, c) in spec.paths:
        if c == 0.0:
            continue
        t = terms.setdefault((i, v), Term(i, v, []))
        t.items.append((j, k, c))
    # merge duplicate (j, k) within a term
    for t in terms.values():
        acc: Dict[Tuple[int, int], float] = {}
        for j, k, c in t.items:
            acc[(j, k)] = acc.get((j, k), 0.0) + c
        t.items = [(j, k, c) for (j, k), c in sorted(acc.items()) if c != 0.0]
    parent: Dict[Tuple[int, int], Tuple[int, int]] = {}

    def find(a):
        while parent.setdefault(a, a) != a:
            parent[a] = parent[parent[a]]
            a = parent[a]
        return a

    for t in terms.values():
        first = None
        for j, k, _ in t.items:
            if first is None:
                first = find((j, k))
            else:
                parent[find((j, k))] = first
                first = find(first)
    groups: Dict[Tuple[int, int], List[Term]] = {}
    for key in sorted(terms):
        t = terms[key]
        if not t.items:
            continue
        groups.setdefault(find((t.items[0][0], t.items[0][1])), []).append(t)
    # one-product terms of the same weight segment (an l1 = 0 or l2 = 0 coupling: every output component is one product)
    # form ONE block, so that the emitters can sum over the components before they touch the shared operand
    merged: Dict[Tuple[int, int], List[Term]] = {}
    for root in sorted(groups):
        ts = groups[root]
        if all(len(t.items) == 1 for t in ts):
            merged.setdefault((-1, ts[0].i), []).extend(ts)
        else:
            merged[root] = ts
    blocks = []
    for root in sorted(merged, key=lambda r: min((t.i, t.v) for t in merged[r])):
        ts = sorted(merged[root], key=lambda t: (t.i, t.v))
        prods = sorted({(j, k) for t in ts for j, k, _ in t.items})
        blocks.append(Block(ts, prods))
    return blocks


def lit(c: float, dtype: str) -> str:
    """C++ literal of a coefficient in the compute type."""
    if dtype == "f32":
        return f"{float(np.float32(c))!r}f"
    return f"{float(c)!r}"


def split_out_segments(blocks: List[Block], out_segs: int, groups: int) -> List[List[int]]:
    """Partition output segments over ``groups`` thread groups with balanced work.

    Segments are ordered by the block that first writes them, then cut into
    contiguous ranges of about equal cost, so that most blocks stay whole inside
    one group and only the blocks at a cut are evaluated (in part) twice.
    """
    cost = [1] * out_segs
    first = [len(blocks)] * out_segs
    for bi, b in enumerate(blocks):
        for t in b.terms:
            cost[t.v] += 2 * len(t.items) + 1
            first[t.v] = min(first[t.v], bi)
    order = sorted(range(out_segs), key=lambda v: (first[v], v))
    total = sum(cost)
    owner: List[List[int]] = [[] for _ in range(groups)]
    run, g = 0, 0
    for v in order:
        if g < groups - 1 and run >= total * (g + 1) / groups:
            g += 1
        owner[g].append(v)
        run += cost[v]
    return [sorted(o) for o in owner]


def split_w_segments(blocks: List[Block], w_segs: int, groups: int) -> List[List[int]]:
    """Partition weight segments over ``groups`` thread groups with balanced work (the backward's split: a group owns
    the grad_w rows of its weight segments outright, so no two groups ever store the same row).  Segments are ordered
    by the block that first uses them and cut into contiguous ranges of about equal cost."""
    cost = [0] * w_segs
    first = [len(blocks)] * w_segs
    for bi, b in enumerate(blocks):
        for t in b.terms:
            cost[t.i] += 2 * len(t.items) + 2
            first[t.i] = min(first[t.i], bi)
    order = sorted(range(w_segs), key=lambda i: (first[i], i))
    total = sum(cost)
    owner: List[List[int]] = [[] for _ in range(groups)]
    run, g = 0, 0
    for i in order:
        if g < groups - 1 and run >= total * (g + 1) / groups:
            g += 1
        owner[g].append(i)
        run += cost[i]
    return [sorted(o) for o in owner]


def restrict_blocks(blocks: List[Block], w_owned) -> List[Block]:
    """The blocks reduced to the terms of the weight segments in ``w_owned`` (products no term uses are dropped)."""
    w_owned = set(w_owned)
    out = []
    for b in blocks:
        ts = [t for t in b.terms if t.i in w_owned]
        if ts:
            out.append(Block(ts, sorted({(j, k) for t in ts for j, k, _ in t.items})))
    return out
