"""Synthetic MACE-style model for the benchmark's model configurations (energy + forces).

Architecture (configuration 1): species embedding -> ``num_layers`` x { SO3Linear (up),
ChannelwiseTensorProduct with SH(l <= 3) edge attributes and radial-MLP weights + scatter-sum,
SO3Linear (mix to 128x{0e,1o,2e,3o}), SymmetricContraction (correlation 3) -> hidden, SO3Linear }
-> per-layer scalar readout; ``E = sum_atoms``; ``F = -dE/dpos`` by autograd.  Radial basis: 8 Bessel
functions times a p = 5 polynomial envelope (…/nequip/nn/embedding/_edge.py:174-189,
…/nequip/nn/embedding/cutoffs.py:17-27), fed to a 64-64-64 SiLU MLP per layer.  Random weights;
this is a throughput and parity vehicle, not a trained potential.

Every tensor between operators is ``ir_mul``; nothing is transposed.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..descriptors import full_channelwise_instructions
from ..irreps import Irreps
from ..ops.dense import dense
from ..ops.edge_geometry import edge_geometry, edge_geometry_usable
from ..ops.radial_chain import radial_chain
from ..ops.spherical_harmonics import SphericalHarmonics
from .modules import ChannelwiseTensorProduct, SO3Linear, SymmetricContraction


def bessel_basis(r: torch.Tensor, r_max: float, num_basis: int) -> torch.Tensor:
    n = torch.arange(1, num_basis + 1, device=r.device, dtype=r.dtype)
    return math.sqrt(2.0 / r_max) * torch.sin(n * math.pi * r.unsqueeze(-1) / r_max) / r.unsqueeze(-1)


def polynomial_cutoff(r: torch.Tensor, r_max: float, p: int = 5) -> torch.Tensor:
    x = r / r_max
    env = 1.0 - (p + 1.0) * (p + 2.0) / 2.0 * x ** p + p * (p + 2.0) * x ** (p + 1) - p * (p + 1.0) / 2.0 * x ** (p + 2)
    return env * (x < 1.0)


class RadialMLP(torch.nn.Module):
    def __init__(self, num_basis: int, hidden: List[int], out_dim: int):
        super().__init__()
        dims = [num_basis] + hidden + [out_dim]
        self.layers = torch.nn.ModuleList(torch.nn.Linear(a, b, bias=False) for a, b in zip(dims[:-1], dims[1:]))
        for lin in self.layers:
            torch.nn.init.normal_(lin.weight, std=1.0 / math.sqrt(lin.in_features))

    def forward(self, x):
        # inference / forces: all hidden layers in one kernel, then the wide last layer
        h = radial_chain(x, [lin.weight for lin in self.layers[:-1]]) if x.dim() == 2 else None
        if h is not None:
            return dense(h, self.layers[-1].weight)
        for i, lin in enumerate(self.layers):
            x = dense(x, lin.weight)
            if i + 1 < len(self.layers):
                x = torch.nn.functional.silu(x)
        return x


class InteractionLayer(torch.nn.Module):
    def __init__(self, irreps_in: Irreps, hidden: Irreps, sh_lmax: int, lmax_mid: int, num_species: int, num_basis: int,
                 radial_hidden: List[int], correlation: int, avg_num_neighbors: float, tp_parity: Optional[str] = "natural"):
        super().__init__()
        mul = irreps_in.uniform_mul()
        sh = Irreps.spherical_harmonics(sh_lmax)
        self.linear_up = SO3Linear(irreps_in, irreps_in)
        # MACE keeps only the couplings whose output irrep is one of the target irreps, i.e. parity (-1)^l
        # (mace/modules/irreps_tools.py tp_out_irreps_with_instructions; the reference's own operator bench
        # applies the same filter, test/bench_tensor_product_uniform1d.py:64-68): 0e+1o x SH(l<=3) gives
        # 10 weighted paths and 40 output rows instead of 13 / 55.
        irreps_tp, instr = full_channelwise_instructions(irreps_in, sh, lmax_mid, parity_filter=tp_parity)
        self.conv_tp = ChannelwiseTensorProduct(irreps_in, sh, irreps_tp, instr)
        self.radial = RadialMLP(num_basis, radial_hidden, self.conv_tp.weight_numel)
        self.irreps_mid = Irreps([(mul, (l, (-1) ** l)) for l in range(lmax_mid + 1)])
        self.linear_mid = SO3Linear(irreps_tp, self.irreps_mid, output_scale=1.0 / avg_num_neighbors)
        self.product = SymmetricContraction(self.irreps_mid, hidden, num_species, correlation)
        self.linear_out = SO3Linear(hidden, hidden)
        self.inv_neighbors = 1.0 / avg_num_neighbors

    def forward(self, h, species, edge_sh, edge_radial, edge_dst, edge_src, halo=None, edge_vec=None):
        up = self.linear_up(h)
        n_owned = up.shape[0]
        begin = getattr(halo, "begin", None)
        if begin is not None:
            up = begin(up)                   # owned rows, then ghost rows of the senders other ranks own (exchange in flight)
        elif halo is not None:
            up = halo(up)
        w = self.radial(edge_radial)         # edge-local work behind the exchange
        if begin is not None:
            up = halo.end(up)
        # edge_vec given: the tensor-product kernel evaluates the spherical harmonics of the edge itself
        msg = self.conv_tp(up, edge_sh, w, edge_dst, edge_src, edge_vec=edge_vec)
        if msg.shape[0] != n_owned:
            msg = msg[:n_owned]              # rows of ghost receivers (no edges end there)
        mid = self.linear_mid(msg)           # 1 / <neighbours> is folded into its path coefficients
        prod = self.product(mid, species)
        return self.linear_out(prod)


class MACEStyleModel(torch.nn.Module):
    def __init__(self, num_species: int = 4, channels: int = 128, hidden_lmax: int = 1, sh_lmax: int = 3, lmax_mid: int = 3,
                 num_layers: int = 2, r_max: float = 5.0, num_basis: int = 8, radial_hidden=(64, 64, 64), correlation: int = 3,
                 avg_num_neighbors: float = 52.0, envelope_p: int = 5, tp_parity: Optional[str] = "natural", fuse_sh: bool = True,
                 fuse_geometry: bool = True):
        super().__init__()
        self.fuse_geometry = fuse_geometry    # edge vectors + radial basis (and their force-pass gradient) as one kernel each
        self.fuse_sh = fuse_sh                # edge harmonics inside the tensor-product kernels (no [E, 16] tensor)
        self.r_max, self.num_basis, self.envelope_p, self.channels = r_max, num_basis, envelope_p, channels
        hidden = Irreps([(channels, (l, (-1) ** l)) for l in range(hidden_lmax + 1)])
        self.hidden = hidden
        self.embedding = torch.nn.Parameter(torch.randn(num_species, channels))
        self.sh = SphericalHarmonics(list(range(sh_lmax + 1)), True, "component")
        layers = []
        irreps_in = Irreps([(channels, (0, 1))])
        for _ in range(num_layers):
            layers.append(InteractionLayer(irreps_in, hidden, sh_lmax, lmax_mid, num_species, num_basis, list(radial_hidden),
                                           correlation, avg_num_neighbors, tp_parity))
            irreps_in = hidden
        self.layers = torch.nn.ModuleList(layers)
        self.readouts = torch.nn.ParameterList(torch.nn.Parameter(torch.randn(channels) / math.sqrt(channels)) for _ in range(num_layers))

    def edge_features(self, pos, edge_src, edge_dst, edge_shift, second_order: bool = False):
        """(harmonics or None, radial basis, edge vectors or None): with ``fuse_sh`` the vectors go to the layers.
        ``second_order``: keep to operators whose backward is itself differentiable (force-loss training)."""
        if self.fuse_geometry and not second_order and edge_geometry_usable(pos, self.num_basis):
            vec, radial = edge_geometry(pos, edge_src, edge_dst, edge_shift, self.r_max, self.num_basis, self.envelope_p)
        else:
            vec = pos[edge_src] + edge_shift - pos[edge_dst]
            r = vec.norm(dim=-1)
            radial = bessel_basis(r, self.r_max, self.num_basis) * polynomial_cutoff(r, self.r_max, self.envelope_p).unsqueeze(-1)
        if self.fuse_sh and not second_order and vec.is_cuda:
            return None, radial, vec
        return self.sh(vec), radial, None

    def node_energies(self, pos, species, edge_src, edge_dst, edge_shift, halo=None, second_order: bool = False):
        """``halo`` (a ``parallel.HaloExchange``) extends per-node tensors with ghost rows; ``pos`` and
        ``species`` then hold the owned nodes only and the edge indices are local ids."""
        pos_ext = pos if halo is None else halo(pos)
        edge_sh, edge_radial, edge_vec = self.edge_features(pos_ext, edge_src, edge_dst, edge_shift, second_order)
        h = self.embedding[species]
        e = pos.new_zeros(pos.shape[0])
        for layer, ro in zip(self.layers, self.readouts):
            h = layer(h, species, edge_sh, edge_radial, edge_dst, edge_src, halo, edge_vec)
            e = e + (h[:, : self.channels] * ro).sum(dim=-1)     # scalars are the first segment of the ir_mul row
        return e

    def forward(self, pos, species, edge_src, edge_dst, edge_shift, node_graph=None, n_graphs: int = 1, forces: bool = True,
                halo=None, create_graph: bool = False):
        """``create_graph``: keep the forces differentiable (a force loss can then be back-propagated to the weights);
        the evaluation then stays on operators with a second-order path (no in-kernel harmonics / fused geometry)."""
        if forces:
            pos = pos.detach().requires_grad_(True)
        e_node = self.node_energies(pos, species, edge_src, edge_dst, edge_shift, halo, second_order=create_graph)
        if node_graph is None:
            energy = e_node.sum().reshape(1)
        else:
            energy = torch.zeros(n_graphs, dtype=e_node.dtype, device=e_node.device).index_add(0, node_graph, e_node)
        out = {"energy": energy}
        if forces:
            (g,) = torch.autograd.grad(e_node.sum(), pos, create_graph=create_graph)
            out["forces"] = -g
        return out
