"""e3nn-style module adapters.

The reference's callers build these with cuequivariance_torch (``FastEqSegmentedPolynomial`` for
the tensor product + scatter, ``SymmetricContraction``, ``Linear``) and convert layouts with
``TransposeIrrepsLayout`` (…/nequip/nn/_tp_scatter_cueq.py:124-177).  That package is not in the
reference tree, so the adapters here generate the path tables themselves
(``fasteq_b200.descriptors``) and call the operators of ``fasteq_b200.ops``.

Layout: every module takes and returns ``ir_mul`` tensors by default (segment-major, channel-minor,
what the kernels consume); ``layout="mul_ir"`` accepts / returns e3nn's layout and transposes at
the boundary.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import descriptors
from ..irreps import Irreps, ir_mul_to_mul_ir, mul_ir_to_ir_mul
from ..ops.eqlinear import fast_equi_linear
from ..ops.stc_uniform1d_jit import fast_stc_uniform1d_jit
from ..ops.uniform1d_jit import fast_uniform1d_jit


class ChannelwiseTensorProduct(torch.nn.Module):
    """``scatter(tp(x[edge_src], edge_attr, edge_weight), edge_dst, dim_size=len(x))`` for ``uvu``
    instructions with per-edge weights: NequIP's TensorProductScatter contract
    (…/nequip/nn/_tp_scatter_base.py:35-38), MACE's conv_tp + scatter_sum."""

    def __init__(self, irreps_in1, irreps_in2, irreps_out, instructions, layout: str = "ir_mul",
                 irrep_normalization: str = "component", path_normalization: str = "element"):
        super().__init__()
        self.irreps_in1, self.irreps_in2, self.irreps_out = Irreps(irreps_in1), Irreps(irreps_in2), Irreps(irreps_out)
        self.descriptor = descriptors.channelwise_tensor_product(self.irreps_in1, self.irreps_in2, self.irreps_out, instructions,
                                                                 irrep_normalization, path_normalization)
        self.weight_numel = self.descriptor.w_seg_num * self.descriptor.u_dim
        if layout not in ("ir_mul", "mul_ir"):
            raise ValueError("layout must be 'ir_mul' or 'mul_ir'")
        self.layout = layout
        self._meta = {}

    def meta(self, dtype, device, y_sh=()):
        key = (dtype, str(device), tuple(y_sh))
        if key not in self._meta:
            m = self.descriptor.meta(dtype, device)
            if y_sh:
                m["y_sh"] = tuple(y_sh)
            self._meta[key] = m
        return self._meta[key]

    def sh_degrees(self):
        """Degrees of ``irreps_in2`` when it is a set of spherical harmonics (one copy of each ``l`` with
        parity ``(-1)^l``), which is what the in-kernel evaluation from edge vectors needs."""
        ls = []
        for b in self.irreps_in2:
            if b.mul != 1 or b.ir.p != (-1) ** b.ir.l:
                raise ValueError(f"irreps_in2 = {self.irreps_in2} is not a set of spherical harmonics")
            ls.append(b.ir.l)
        return tuple(ls)

    def forward(self, x, edge_attr, edge_weight, edge_dst, edge_src, edge_vec=None, sh_normalize: bool = True,
                sh_normalization: str = "component"):
        """``edge_attr`` are the spherical harmonics of the edges; alternatively pass ``edge_attr=None`` and the
        edge vectors ``edge_vec [E, 3]``: the kernel then evaluates the harmonics itself (and the backward
        returns the gradient with respect to the vectors)."""
        if self.layout == "mul_ir":
            x = mul_ir_to_ir_mul(x, self.irreps_in1)
        if edge_vec is not None:
            if edge_attr is not None:
                raise ValueError("pass either edge_attr or edge_vec")
            y, meta = edge_vec, self.meta(x.dtype, x.device, (self.sh_degrees(), sh_normalize, sh_normalization))
        else:
            y, meta = edge_attr, self.meta(x.dtype, x.device)
        out = fast_uniform1d_jit(edge_weight.contiguous(), x.contiguous(), y.contiguous(), {1: edge_src}, {0: edge_dst}, meta)
        if self.layout == "mul_ir":
            out = ir_mul_to_mul_ir(out, self.irreps_out)
        return out


class SO3Linear(torch.nn.Module):
    """e3nn ``o3.Linear`` for uniform multiplicities: one ``[mul_in, mul_out]`` matrix per pair of equal
    irreps, normalised by the fan-in (e3nn/o3/_linear.py:148-159)."""

    def __init__(self, irreps_in, irreps_out, layout: str = "ir_mul", compute_precision: Optional[str] = None,
                 output_scale: float = 1.0):
        """``output_scale`` multiplies the result (folded into the path coefficients, e.g. 1 / <neighbours>)."""
        super().__init__()
        self.irreps_in, self.irreps_out = Irreps(irreps_in), Irreps(irreps_out)
        self.output_scale = float(output_scale)
        self.descriptor = descriptors.linear(self.irreps_in, self.irreps_out, scale=self.output_scale)
        self.weight = torch.nn.Parameter(torch.randn(self.descriptor.num_weights))
        self.layout, self.compute_precision = layout, compute_precision

    def forward(self, x, weight: Optional[torch.Tensor] = None):
        w = self.weight if weight is None else weight
        if self.layout == "mul_ir":
            x = mul_ir_to_ir_mul(x, self.irreps_in)
        out = fast_equi_linear(self.descriptor, w, x, compute_precision=self.compute_precision)
        if self.layout == "mul_ir":
            out = ir_mul_to_mul_ir(out, self.irreps_out)
        return out


class SymmetricContraction(torch.nn.Module):
    """MACE's product basis: ``out = sum_{nu <= correlation} W_nu[species] . B_nu . x^{(x) nu}`` with
    species-dependent per-channel weights."""

    def __init__(self, irreps_in, irreps_out, num_species: int, correlation: int = 3, layout: str = "ir_mul"):
        super().__init__()
        self.irreps_in, self.irreps_out = Irreps(irreps_in), Irreps(irreps_out)
        self.descriptor = descriptors.symmetric_contraction(self.irreps_in, self.irreps_out, tuple(range(1, correlation + 1)))
        d = self.descriptor
        self.weight = torch.nn.Parameter(torch.randn(num_species, d.x0_segs, d.u_dim) / math.sqrt(d.x0_segs))
        self.layout = layout
        self._tables = {}

    def tables(self, dtype, device):
        key = (dtype, str(device))
        if key not in self._tables:
            self._tables[key] = self.descriptor.tensors(dtype, device)
        return self._tables[key]

    def forward(self, x, species):
        d = self.descriptor
        if self.layout == "mul_ir":
            x = mul_ir_to_ir_mul(x, self.irreps_in)
        coeffs, paths, idx_lists = self.tables(x.dtype, x.device)
        out = fast_stc_uniform1d_jit(x.reshape(-1, d.x1_segs, d.u_dim), self.weight, species, coeffs, paths, idx_lists, d.out_segs)
        if self.layout == "mul_ir":
            out = ir_mul_to_mul_ir(out, self.irreps_out)
        return out
