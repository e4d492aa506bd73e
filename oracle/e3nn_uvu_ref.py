"""e3nn-level oracle: ``scatter(TensorProduct_uvu(x[src], sh, w), dst)`` on the CPU with torch.

Restates e3nn's generated contraction for ``uvu`` instructions with per-edge
weights (e3nn/o3/_tensor_product/_codegen.py:166-187: one einsum against the
Wigner 3j tensor per instruction, general form ``zuv,ijk,zuvij->zuk``) and its
path normalisation (e3nn/o3/_tensor_product/_tensor_product.py:277-323), followed
by the scatter of nequip/nn/_tp_scatter_base.py:35-38.  Data layout is e3nn's
``mul_ir``.  Differentiable (torch autograd supplies the force backward), so it
doubles as the timed CPU baseline.
"""
from __future__ import annotations

from math import sqrt

import torch

from fasteq_b200.irreps import Irreps
from fasteq_b200.wigner import wigner_3j


class TensorProductUVU:
    def __init__(self, irreps_in1, irreps_in2, irreps_out, instructions, dtype=torch.float64):
        self.irreps_in1, self.irreps_in2, self.irreps_out = Irreps(irreps_in1), Irreps(irreps_in2), Irreps(irreps_out)
        ins = [tuple(t) + ((1.0,) if len(t) == 5 else ()) for t in instructions]
        self.ins = []
        for (i1, i2, io, mode, has_w, pw) in ins:
            assert mode == "uvu" and has_w
            iro = self.irreps_out[io].ir
            fan = sum(self.irreps_in2[t[1]].mul for t in ins if t[2] == io)
            alpha = iro.dim / fan * pw
            c = torch.as_tensor(wigner_3j(self.irreps_in1[i1].ir.l, self.irreps_in2[i2].ir.l, iro.l), dtype=dtype)
            self.ins.append((i1, i2, io, sqrt(alpha), c))
        self.weight_numel = sum(self.irreps_in1[i1].mul for i1, *_ in self.ins)

    def __call__(self, x1, x2, weight):
        z = x1.shape[0]
        x1s = [x1[:, sl].reshape(z, b.mul, b.ir.dim) for b, sl in zip(self.irreps_in1, self.irreps_in1.slices())]
        x2s = [x2[:, sl].reshape(z, b.mul, b.ir.dim) for b, sl in zip(self.irreps_in2, self.irreps_in2.slices())]
        outs = [None] * len(self.irreps_out)
        off = 0
        for (i1, i2, io, pw, c) in self.ins:
            mul = self.irreps_in1[i1].mul
            w = weight[:, off:off + mul].reshape(z, mul, 1)
            off += mul
            r = pw * torch.einsum("zuv,ijk,zui,zvj->zuk", w, c.to(x1.dtype), x1s[i1], x2s[i2])
            outs[io] = r if outs[io] is None else outs[io] + r
        parts = []
        for b, o in zip(self.irreps_out, outs):
            parts.append(o.reshape(z, b.dim) if o is not None else x1.new_zeros(z, b.dim))
        return torch.cat(parts, dim=1)


def tp_scatter(tp: TensorProductUVU, x, edge_attr, edge_weight, edge_dst, edge_src, num_nodes=None):
    """out[n] = sum_{e: dst[e]=n} tp(x[src[e]], edge_attr[e], edge_weight[e])."""
    msg = tp(x[edge_src], edge_attr, edge_weight)
    out = msg.new_zeros((x.shape[0] if num_nodes is None else num_nodes, msg.shape[1]))
    return out.index_add(0, edge_dst, msg)
