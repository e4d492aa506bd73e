"""CPU oracle of the synthetic MACE-style model: the same architecture evaluated with dense torch
operations straight from the path tables (float64, autograd for the forces).

Each operator is the path formula of the corresponding oracle (``uniform1d_ref``, ``eqlinear_ref``,
``stc_ref``) written with differentiable torch ops; the model structure follows
``fasteq_b200.nn.mace_style`` and takes its parameters from the model's state dict.  Of the product it reads only
the modules' path tables (``layer.*.descriptor``, pinned to e3nn by the golden-vector tests) and hyper-parameters;
the radial basis, the cutoff envelope and the SO3Linear row mapping are restated here.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from oracle import sh_ref


def u1d_scatter(w, x, y, d, src, dst, n_out):
    """ir_mul Uniform1D with gather + scatter: w [E, I*U], x [N, J*U], y [E, K]."""
    U = d.u_dim
    w3, x3 = w.reshape(-1, d.w_seg_num, U), x.reshape(-1, d.x_seg_num, U)[src]
    msg = torch.zeros(w.shape[0], d.out_seg_num, U, dtype=x.dtype)
    cols = [msg[:, v, :] for v in range(d.out_seg_num)]
    acc = [None] * d.out_seg_num
    for i, j, k, v, c in zip(d.i_list, d.j_list, d.k_list, d.v_list, d.coeff_list):
        t = float(c) * w3[:, i, :] * x3[:, j, :] * y[:, k:k + 1]
        acc[v] = t if acc[v] is None else acc[v] + t
    msg = torch.stack([a if a is not None else torch.zeros_like(w3[:, 0, :]) for a in acc], dim=1)
    out = torch.zeros(n_out, d.out_seg_num, U, dtype=x.dtype).index_add(0, dst, msg)
    return out.reshape(n_out, -1)


def bessel_basis(r, r_max: float, num_basis: int):
    """``sqrt(2 / r_max) * sin(n pi r / r_max) / r`` for n = 1 .. num_basis: NequIP's BesselEdgeLengthEncoding
    (…/nequip/nn/embedding/_edge.py:174-189 writes it as ``sinc(x n pi) n pi`` up to the same prefactor)."""
    n = torch.arange(1, num_basis + 1, dtype=r.dtype)
    return math.sqrt(2.0 / r_max) * torch.sin(r.unsqueeze(-1) * (n * math.pi / r_max)) / r.unsqueeze(-1)


def polynomial_cutoff(r, r_max: float, p: int = 5):
    """``1 - (p+1)(p+2)/2 x^p + p(p+2) x^(p+1) - p(p+1)/2 x^(p+2)`` for ``x = r / r_max < 1``, else 0
    (…/nequip/nn/embedding/cutoffs.py:17-27)."""
    x = r / r_max
    out = 1.0 - ((p + 1.0) * (p + 2.0) / 2.0) * torch.pow(x, p) + p * (p + 2.0) * torch.pow(x, p + 1) \
        - (p * (p + 1.0) / 2.0) * torch.pow(x, p + 2)
    return torch.where(x < 1.0, out, torch.zeros_like(out))


def linear_mapping(desc):
    """``[(in_row, out_row, weight_block, rows)]``, coefficients, u, v, I, J read from a ``uv,iu,iv`` descriptor's
    public attributes only (``operands`` = weight / input / output segment shapes, ``paths[q].indices`` =
    (weight block, input segment, output segment), ``paths[q].coefficients``): the segment protocol of
    fasteq/ops/auto_schedule/eqlinear_descriptor.py:228-310, restated here so that the oracle does not run
    the product's own descriptor parser."""
    w_seg, in_seg, out_seg = (list(op) for op in desc.operands)
    u, v = int(w_seg[0][0]), int(w_seg[0][1])
    in_off = np.concatenate(([0], np.cumsum([int(s[0]) for s in in_seg])))
    out_off = np.concatenate(([0], np.cumsum([int(s[0]) for s in out_seg])))
    mapping, coeff = [], []
    for path in desc.paths:
        wq, a, b = (int(t) for t in path.indices)
        rows = int(in_seg[a][0])
        assert rows == int(out_seg[b][0]) and tuple(int(t) for t in w_seg[wq]) == (u, v)
        mapping.append((int(in_off[a]), int(out_off[b]), wq, rows))
        coeff.append(float(path.coefficients))
    return mapping, coeff, u, v, int(in_off[-1]), int(out_off[-1])


def eqlinear(x, w, desc):
    mapping, coeff, u, v, I, J = linear_mapping(desc)
    x3, w3 = x.reshape(-1, I, u), w.reshape(len(mapping), u, v)
    rows = [None] * J
    for (ir, orow, wp, n), c in zip(mapping, coeff):
        t = float(c) * (x3[:, ir:ir + n, :] @ w3[wp])
        for k in range(n):
            rows[orow + k] = t[:, k, :] if rows[orow + k] is None else rows[orow + k] + t[:, k, :]
    zero = torch.zeros(x3.shape[0], v, dtype=x.dtype)
    return torch.stack([r if r is not None else zero for r in rows], dim=1).reshape(x3.shape[0], -1)


def stc(x1, x0, i0, d):
    from oracle.stc_ref import split_paths
    U = d.u_dim
    x3, wg = x1.reshape(-1, d.x1_segs, U), x0[i0]
    acc = [None] * d.out_segs
    for (a, dd, v), c in zip(split_paths(d.paths), d.coeffs):
        t = float(c) * wg[:, dd, :]
        for ai in a:
            t = t * x3[:, ai, :]
        acc[v] = t if acc[v] is None else acc[v] + t
    zero = torch.zeros(x3.shape[0], U, dtype=x1.dtype)
    return torch.stack([r if r is not None else zero for r in acc], dim=1).reshape(x3.shape[0], -1)


def energy_and_forces(model, pos, species, edge_src, edge_dst, edge_shift, params=None, create_graph=False):
    """Evaluate ``model`` (a ``MACEStyleModel`` whose parameters were moved to CPU/float64) with the oracle operators.
    ``params`` (optional) replaces the state dict, e.g. with leaves that require grad; with ``create_graph`` the
    forces stay attached to the graph so that a force loss can be differentiated."""
    pos = pos.detach().double().requires_grad_(True)
    p = params if params is not None else {k: v.detach().double().cpu() for k, v in model.state_dict().items()}
    vec = pos[edge_src] + edge_shift.double() - pos[edge_dst]
    r = vec.norm(dim=-1)
    radial = bessel_basis(r, model.r_max, model.num_basis) * polynomial_cutoff(r, model.r_max, model.envelope_p).unsqueeze(-1)
    ysh = sh_ref.spherical_harmonics(max(model.sh._ls), vec, normalize=True, normalization="component")
    h = p["embedding"][species]
    e = torch.zeros(pos.shape[0], dtype=torch.float64)
    for li, layer in enumerate(model.layers):
        pre = f"layers.{li}."
        up = eqlinear(h, p[pre + "linear_up.weight"], layer.linear_up.descriptor)
        w = radial
        n_lin = len(layer.radial.layers)
        for k in range(n_lin):
            w = w @ p[pre + f"radial.layers.{k}.weight"].T
            if k + 1 < n_lin:
                w = torch.nn.functional.silu(w)
        msg = u1d_scatter(w, up, ysh, layer.conv_tp.descriptor, edge_src, edge_dst, pos.shape[0])
        mid = eqlinear(msg, p[pre + "linear_mid.weight"], layer.linear_mid.descriptor)   # its coefficients carry 1 / <neighbours>
        prod = stc(mid, p[pre + "product.weight"], species, layer.product.descriptor)
        h = eqlinear(prod, p[pre + "linear_out.weight"], layer.linear_out.descriptor)
        e = e + h[:, : model.channels] @ p[f"readouts.{li}"]
    (g,) = torch.autograd.grad(e.sum(), pos, create_graph=create_graph)
    return (e if create_graph else e.detach()), -g


def force_loss_gradients(model, pos, species, edge_src, edge_dst, edge_shift, target_forces, names):
    """d/d(parameter) of ``sum |F - F_target|^2`` for the named parameters (float64, double backward on the CPU)."""
    p = {k: v.detach().double().cpu() for k, v in model.state_dict().items()}
    for n in names:
        p[n] = p[n].clone().requires_grad_(True)
    _, f = energy_and_forces(model, pos, species, edge_src, edge_dst, edge_shift, params=p, create_graph=True)
    loss = ((f - target_forces.double()) ** 2).sum()
    grads = torch.autograd.grad(loss, [p[n] for n in names])
    return float(loss.detach()), dict(zip(names, grads))


def gate_ref(x, spec):
    """Dense torch restatement of the gate on an ir_mul row (e3nn/nn/_gate.py: activations on the
    scalars, gated irreps times the activated gates)."""
    u = spec.u
    x3 = x.reshape(x.shape[0], spec.n_in, u)
    act = {0: lambda t: t, 1: torch.nn.functional.silu, 2: torch.tanh, 3: torch.sigmoid, 4: torch.abs}
    outs = [spec.csts[s] * act[spec.acts[s]](x3[:, s]) for s in range(spec.n_scalar)]
    pos = spec.n_scalar + spec.n_gate
    for k, dim in enumerate(spec.gated_dims):
        g = spec.n_scalar + k
        gv = spec.csts[g] * act[spec.acts[g]](x3[:, g])
        for m in range(dim):
            outs.append(gv * x3[:, pos + m])
        pos += dim
    return torch.stack(outs, dim=1).reshape(x.shape[0], -1)


def nequip_energy_and_forces(model, pos, species, edge_src, edge_dst, edge_shift):
    """Oracle evaluation of ``fasteq_b200.nn.nequip_style.NequIPStyleModel`` (float64, CPU)."""
    pos = pos.detach().double().requires_grad_(True)
    p = {k: v.detach().double().cpu() for k, v in model.state_dict().items()}
    vec = pos[edge_src] + edge_shift.double() - pos[edge_dst]
    r = vec.norm(dim=-1)
    radial = bessel_basis(r, model.r_max, model.num_basis) * polynomial_cutoff(r, model.r_max, model.envelope_p).unsqueeze(-1)
    ysh = sh_ref.spherical_harmonics(max(model.sh._ls), vec, normalize=True, normalization="component")
    h = p["embedding"][species]
    for li, layer in enumerate(model.layers):
        pre = f"layers.{li}."
        up = eqlinear(h, p[pre + "linear_1.weight"], layer.linear_1.descriptor)
        w = radial
        n_lin = len(layer.radial.layers)
        for k in range(n_lin):
            w = w @ p[pre + f"radial.layers.{k}.weight"].T
            if k + 1 < n_lin:
                w = torch.nn.functional.silu(w)
        msg = u1d_scatter(w, up, ysh, layer.conv_tp.descriptor, edge_src, edge_dst, pos.shape[0])
        x = eqlinear(msg, p[pre + "linear_2.weight"], layer.linear_2.descriptor) \
            + eqlinear(h, p[pre + "self_connection.weight"], layer.self_connection.descriptor)   # linear_2's coefficients carry 1 / <neighbours>
        h = gate_ref(x, layer.gate_spec)
    e = h[:, : model.channels] @ p["readout"]
    (g,) = torch.autograd.grad(e.sum(), pos)
    return e.detach(), -g
