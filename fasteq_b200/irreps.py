"""Minimal irreps bookkeeping with e3nn-compatible string syntax.

Only what the tensor-product hot path needs: parsing ``"128x0e+128x1o"``,
dimensions, segment offsets and the two memory layouts the operators use:

* ``mul_ir`` (e3nn): per irrep block, channel-major, ``m`` minor: ``[mul, 2l+1]``
* ``ir_mul`` (FastEq / cuEquivariance operators): ``m`` major, channel minor:
  ``[2l+1, mul]``; with a uniform ``mul`` this is the ``[segment, u]`` view the
  Uniform1D kernels consume (reference: fasteq/ops/uniform1d_jit.py:3239-3242).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Iterable, List, Sequence, Tuple, Union


@dataclass(frozen=True)
class Irrep:
    l: int
    p: int  # +1 even, -1 odd

    @property
    def dim(self) -> int:
        return 2 * self.l + 1

    def __str__(self) -> str:
        return f"{self.l}{'e' if self.p == 1 else 'o'}"

    def __mul__(self, other: "Irrep") -> List["Irrep"]:
        p = self.p * other.p
        return [Irrep(l, p) for l in range(abs(self.l - other.l), self.l + other.l + 1)]

    @staticmethod
    def parse(s: Union[str, "Irrep", Tuple[int, int]]) -> "Irrep":
        if isinstance(s, Irrep):
            return s
        if isinstance(s, tuple):
            return Irrep(int(s[0]), int(s[1]))
        m = re.fullmatch(r"\s*(\d+)([eoy])\s*", s)
        if not m:
            raise ValueError(f"cannot parse irrep {s!r}")
        l = int(m.group(1))
        c = m.group(2)
        p = {"e": 1, "o": -1, "y": (-1) ** l}[c]
        return Irrep(l, p)


@dataclass(frozen=True)
class MulIr:
    mul: int
    ir: Irrep

    @property
    def dim(self) -> int:
        return self.mul * self.ir.dim


class Irreps:
    """Ordered list of (multiplicity, irrep) blocks."""

    def __init__(self, spec: Union[str, "Irreps", Iterable] = ""):
        blocks: List[MulIr] = []
        if isinstance(spec, Irreps):
            blocks = list(spec.blocks)
        elif isinstance(spec, str):
            if spec.strip():
                for tok in spec.split("+"):
                    tok = tok.strip()
                    if "x" in tok:
                        mul, ir = tok.split("x")
                        blocks.append(MulIr(int(mul), Irrep.parse(ir)))
                    else:
                        blocks.append(MulIr(1, Irrep.parse(tok)))
        else:
            for item in spec:
                if isinstance(item, MulIr):
                    blocks.append(item)
                else:
                    mul, ir = item
                    blocks.append(MulIr(int(mul), Irrep.parse(ir)))
        self.blocks: Tuple[MulIr, ...] = tuple(blocks)

    # -- container protocol -------------------------------------------------
    def __iter__(self):
        return iter(self.blocks)

    def __len__(self):
        return len(self.blocks)

    def __getitem__(self, i):
        return self.blocks[i]

    def __eq__(self, other):
        return isinstance(other, Irreps) and self.blocks == other.blocks

    def __hash__(self):
        return hash(self.blocks)

    def __repr__(self):
        return "+".join(f"{b.mul}x{b.ir}" for b in self.blocks)

    # -- sizes ----------------------------------------------------------------
    @property
    def dim(self) -> int:
        return sum(b.dim for b in self.blocks)

    @property
    def num_segments(self) -> int:
        """Number of ``[u]`` segments in ir_mul layout (sum of 2l+1)."""
        return sum(b.ir.dim for b in self.blocks)

    @property
    def lmax(self) -> int:
        return max(b.ir.l for b in self.blocks)

    def uniform_mul(self) -> int:
        muls = {b.mul for b in self.blocks}
        if len(muls) != 1:
            raise ValueError(f"irreps {self} do not have a uniform multiplicity")
        return muls.pop()

    def segment_offsets(self) -> List[int]:
        """Offset (in segments of 2l+1 rows) of each block in ir_mul layout."""
        offs, o = [], 0
        for b in self.blocks:
            offs.append(o)
            o += b.ir.dim
        return offs

    def slices(self) -> List[slice]:
        out, o = [], 0
        for b in self.blocks:
            out.append(slice(o, o + b.dim))
            o += b.dim
        return out

    @staticmethod
    def spherical_harmonics(lmax: int, p: int = -1) -> "Irreps":
        return Irreps([(1, (l, p ** l)) for l in range(lmax + 1)])


def mul_ir_to_ir_mul(x, irreps: Irreps):
    """Transpose every block ``[mul, 2l+1] -> [2l+1, mul]`` along the last dim (torch or numpy)."""
    parts = []
    for b, sl in zip(irreps.blocks, irreps.slices()):
        blk = x[..., sl]
        blk = blk.reshape(*x.shape[:-1], b.mul, b.ir.dim)
        blk = blk.swapaxes(-1, -2) if hasattr(blk, "swapaxes") else blk.transpose(-1, -2)
        parts.append(blk.reshape(*x.shape[:-1], b.dim))
    import numpy as _np
    if isinstance(x, _np.ndarray):
        return _np.concatenate(parts, axis=-1)
    import torch
    return torch.cat(parts, dim=-1)


def ir_mul_to_mul_ir(x, irreps: Irreps):
    """Inverse of :func:`mul_ir_to_ir_mul`."""
    parts = []
    for b, sl in zip(irreps.blocks, irreps.slices()):
        blk = x[..., sl]
        blk = blk.reshape(*x.shape[:-1], b.ir.dim, b.mul)
        blk = blk.swapaxes(-1, -2) if hasattr(blk, "swapaxes") else blk.transpose(-1, -2)
        parts.append(blk.reshape(*x.shape[:-1], b.dim))
    import numpy as _np
    if isinstance(x, _np.ndarray):
        return _np.concatenate(parts, axis=-1)
    import torch
    return torch.cat(parts, dim=-1)
