"""Real spherical harmonics oracle (torch CPU, differentiable).

e3nn convention (e3nn/o3/_spherical_harmonics.py; same polynomials as the table
in fasteq/triton/spherical_harmonics.py:66-238): ``Y_0 = 1``, ``Y_1 = sqrt(3) (x, y, z)``
and ``Y_l`` is the coupling of ``Y_{l-1}`` with ``Y_1`` through the real Wigner 3j
tensor, scaled so that ``|Y_l|^2 = 2l+1`` on the unit sphere ("component").
``normalize=True`` divides the input by ``max(|r|, 1e-12)`` first
(fasteq/triton/spherical_harmonics.py:368-373; torch.nn.functional.normalize in e3nn).
Evaluated numerically by the recursion, not from generated polynomials, so it
is independent of the kernels' code generator.
"""
from __future__ import annotations

import math

import torch

from fasteq_b200.wigner import wigner_3j


def spherical_harmonics(lmax: int, vec: torch.Tensor, normalize: bool = True, normalization: str = "component") -> torch.Tensor:
    """[..., 3] -> [..., (lmax+1)^2], blocks l = 0..lmax, m = -l..l."""
    if normalize:
        vec = vec / vec.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    r2 = (vec * vec).sum(-1, keepdim=True)
    ys = [torch.ones_like(vec[..., :1])]
    if lmax >= 1:
        ys.append(math.sqrt(3.0) * vec)
    for l in range(2, lmax + 1):
        c = torch.as_tensor(wigner_3j(l - 1, 1, l), dtype=vec.dtype)
        raw = torch.einsum("ijk,...i,...j->...k", c, ys[l - 1], ys[1])
        # |raw|^2 = s_l^2 * r^(2l) * (2l+1) for a fixed scalar s_l: fix it on the unit vector e_y.
        e = torch.zeros(3, dtype=vec.dtype); e[1] = 1.0
        ys_e = [torch.ones(1, dtype=vec.dtype), math.sqrt(3.0) * e]
        for ll in range(2, l):
            ys_e.append(_SCALE[ll] * torch.einsum("ijk,i,j->k", torch.as_tensor(wigner_3j(ll - 1, 1, ll), dtype=vec.dtype), ys_e[ll - 1], ys_e[1]))
        raw_e = torch.einsum("ijk,i,j->k", c, ys_e[l - 1], ys_e[1])
        _SCALE[l] = math.sqrt((2 * l + 1) / float((raw_e * raw_e).sum()))
        ys.append(_SCALE[l] * raw)
    out = torch.cat(ys[: lmax + 1], dim=-1)
    if normalization == "component":
        return out
    parts = []
    for l in range(lmax + 1):
        blk = out[..., l * l:(l + 1) * (l + 1)]
        if normalization == "norm":
            blk = blk / math.sqrt(2 * l + 1)
        elif normalization == "integral":
            blk = blk / math.sqrt(4 * math.pi)
        else:
            raise ValueError(normalization)
        parts.append(blk)
    return torch.cat(parts, dim=-1)


_SCALE = {}
