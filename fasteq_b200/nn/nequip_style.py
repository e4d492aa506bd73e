"""Synthetic NequIP-style model for benchmark configuration 3 (energy + forces).

Hidden features ``C x (0e+0o+1e+1o+2e+2o)``, edge attributes SH(l <= 2), ``num_layers`` interaction
blocks of { SO3Linear, ChannelwiseTensorProduct + scatter-sum with radial-MLP weights, SO3Linear to the
gate's input, species-independent self connection, Gate (SiLU on even scalars, tanh on odd scalars,
SiLU gates) } following …/nequip/nn/interaction_block.py:79-198, then a scalar readout.  The
species-dependent self connection of NequIP is a FullyConnectedTensorProduct with a one-hot
operand (outside this path); a plain SO3Linear stands in for it.  With ``halo`` the sender features
are extended by ghost rows before every tensor product (…/interaction_block.py:183-198).
"""
from __future__ import annotations

import math
from typing import List

import torch

from ..descriptors import full_channelwise_instructions
from ..irreps import Irreps
from ..ops.gate import GateSpec, gate
from ..ops.spherical_harmonics import SphericalHarmonics
from ..ops.edge_geometry import edge_geometry, edge_geometry_usable
from .mace_style import RadialMLP, bessel_basis, polynomial_cutoff
from .modules import ChannelwiseTensorProduct, SO3Linear


def hidden_irreps(channels: int, lmax: int) -> Irreps:
    return Irreps([(channels, (l, p)) for l in range(lmax + 1) for p in (1, -1)])


class NequIPStyleLayer(torch.nn.Module):
    def __init__(self, irreps_in: Irreps, channels: int, lmax: int, sh_lmax: int, num_basis: int, radial_hidden: List[int],
                 avg_num_neighbors: float):
        super().__init__()
        sh = Irreps.spherical_harmonics(sh_lmax)
        hid = hidden_irreps(channels, lmax)
        gated = [b for b in hid if b.ir.l > 0]
        self.gate_in = Irreps([(channels, (0, 1)), (channels, (0, -1))] + [(channels, (0, 1))] * len(gated) + [(b.mul, b.ir) for b in gated])
        self.gate_spec = GateSpec(channels, ["silu", "tanh"], ["silu"] * len(gated), [b.ir.l for b in gated])
        self.linear_1 = SO3Linear(irreps_in, irreps_in)
        irreps_tp, instr = full_channelwise_instructions(irreps_in, sh, lmax)
        self.conv_tp = ChannelwiseTensorProduct(irreps_in, sh, irreps_tp, instr)
        self.radial = RadialMLP(num_basis, radial_hidden, self.conv_tp.weight_numel)
        self.linear_2 = SO3Linear(irreps_tp, self.gate_in, output_scale=1.0 / avg_num_neighbors)
        self.self_connection = SO3Linear(irreps_in, self.gate_in)
        self.inv_neighbors = 1.0 / avg_num_neighbors
        self.irreps_out = hid

    def forward(self, h, edge_sh, edge_radial, edge_dst, edge_src, halo=None, edge_vec=None):
        up = self.linear_1(h)
        n_owned = up.shape[0]
        begin = getattr(halo, "begin", None)
        if begin is not None:
            up = begin(up)                       # ghost exchange in flight ...
        elif halo is not None:
            up = halo(up)
        w = self.radial(edge_radial)             # ... behind the edge-local radial MLP and the node-local self-connection
        sc = self.self_connection(h)
        if begin is not None:
            up = halo.end(up)
        msg = self.conv_tp(up, edge_sh, w, edge_dst, edge_src, edge_vec=edge_vec)
        if msg.shape[0] != n_owned:
            msg = msg[:n_owned]
        pre = self.linear_2(msg) + sc            # 1 / <neighbours> is folded into linear_2's coefficients
        return gate(pre, self.gate_spec)


class NequIPStyleModel(torch.nn.Module):
    def __init__(self, num_species: int = 2, channels: int = 64, lmax: int = 2, sh_lmax: int = 2, num_layers: int = 4,
                 r_max: float = 4.0, num_basis: int = 8, radial_hidden=(64, 64), avg_num_neighbors: float = 27.0, envelope_p: int = 5,
                 fuse_sh: bool = True, fuse_geometry: bool = True):
        super().__init__()
        self.fuse_geometry = fuse_geometry    # edge vectors + radial basis as one kernel per direction
        self.fuse_sh = fuse_sh                # edge harmonics inside the tensor-product kernels
        self.r_max, self.num_basis, self.envelope_p, self.channels = r_max, num_basis, envelope_p, channels
        self.embedding = torch.nn.Parameter(torch.randn(num_species, channels))
        self.sh = SphericalHarmonics(list(range(sh_lmax + 1)), True, "component")
        layers, irreps_in = [], Irreps([(channels, (0, 1))])
        for _ in range(num_layers):
            layer = NequIPStyleLayer(irreps_in, channels, lmax, sh_lmax, num_basis, list(radial_hidden), avg_num_neighbors)
            layers.append(layer)
            irreps_in = layer.irreps_out
        self.layers = torch.nn.ModuleList(layers)
        self.readout = torch.nn.Parameter(torch.randn(channels) / math.sqrt(channels))

    def node_energies(self, pos, species, edge_src, edge_dst, edge_shift, halo=None, second_order: bool = False):
        """``second_order``: keep to operators whose backward is itself differentiable (force-loss training)."""
        pos_ext = pos if halo is None else halo(pos)
        if self.fuse_geometry and not second_order and edge_geometry_usable(pos_ext, self.num_basis):
            vec, radial = edge_geometry(pos_ext, edge_src, edge_dst, edge_shift, self.r_max, self.num_basis, self.envelope_p)
        else:
            vec = pos_ext[edge_src] + edge_shift - pos_ext[edge_dst]
            r = vec.norm(dim=-1)
            radial = bessel_basis(r, self.r_max, self.num_basis) * polynomial_cutoff(r, self.r_max, self.envelope_p).unsqueeze(-1)
        fused = self.fuse_sh and vec.is_cuda and not second_order
        edge_sh = None if fused else self.sh(vec)
        h = self.embedding[species]
        for layer in self.layers:
            h = layer(h, edge_sh, radial, edge_dst, edge_src, halo, vec if fused else None)
        return (h[:, : self.channels] * self.readout).sum(dim=-1)     # per-atom scalar readout: elementwise + row sum

    def forward(self, pos, species, edge_src, edge_dst, edge_shift, forces: bool = True, halo=None, create_graph: bool = False):
        """``create_graph``: keep the forces differentiable, for a force loss."""
        if forces:
            pos = pos.detach().requires_grad_(True)
        e_node = self.node_energies(pos, species, edge_src, edge_dst, edge_shift, halo, second_order=create_graph)
        out = {"energy": e_node.sum().reshape(1)}
        if forces:
            (g,) = torch.autograd.grad(e_node.sum(), pos, create_graph=create_graph)
            out["forces"] = -g
        return out
