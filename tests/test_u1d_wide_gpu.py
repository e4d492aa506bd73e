"""GPU parity, against the numpy oracle, of the 128-channel Uniform1D signatures that select the
"wide" kernel layout: one CTA of four producer/consumer pipelines, two channels per thread with
packed arithmetic.  These are the layouts the benchmark's headline figure and the MACE-style
model run on; each test asserts the layout it exercises so that it cannot drift onto another.
"""
import numpy as np
import pytest
import torch

from fasteq_b200.codegen.u1d import default_tuning
from fasteq_b200.codegen.u1d_common import make_spec
from fasteq_b200.descriptors import channelwise_tensor_product, full_channelwise_instructions
from fasteq_b200.irreps import Irreps
from fasteq_b200.sh import spherical_harmonics_host
from oracle import uniform1d_ref

pytestmark = pytest.mark.gpu

TOL = 1e-5   # FP32, relative to the largest reference magnitude

# (irreps_in1, parity filter, weight segments, output segments, deep-ring "small" variant)
SIGNATURES = [
    ("128x0e+128x1o", None, 13, 55, False),        # benchmark default: all couplings up to l = 3
    ("128x0e+128x1o", "natural", 10, 40, False),   # second interaction layer of the MACE-style model
    ("128x0e", "natural", 4, 16, True),            # first interaction layer: scalar senders
]


def _descriptor(in1, parity):
    sh = Irreps.spherical_harmonics(3)
    io, ins = full_channelwise_instructions(in1, sh, 3, parity_filter=parity)
    return channelwise_tensor_product(in1, sh, io, ins)


def _graph(n_nodes, g):
    """Receiver-sorted edges with empty receivers (also the first and the last row), single-edge
    receivers, and receivers whose edge count exceeds a producer batch (32) and every ring depth."""
    deg = torch.randint(0, 24, (n_nodes,), generator=g)
    deg[0] = 0
    deg[n_nodes - 1] = 0
    deg[5:9] = 0
    deg[9] = 1
    deg[17] = 33
    deg[40] = 97
    deg[41] = 64
    deg[n_nodes - 2] = 150
    dst = torch.repeat_interleave(torch.arange(n_nodes), deg)
    src = torch.randint(0, n_nodes, (int(dst.numel()),), generator=g)
    return src, dst


def _close(got, ref, what):
    got = got.detach().cpu().double().numpy().reshape(ref.shape)
    err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert err <= TOL, f"{what}: relative error {err:.3e} > {TOL:.0e}"


@pytest.mark.parametrize("in1,parity,w_segs,out_segs,small", SIGNATURES)
def test_default_tuning_is_the_four_pipeline_packed_layout(in1, parity, w_segs, out_segs, small):
    d = _descriptor(in1, parity)
    assert (d.w_seg_num, d.out_seg_num) == (w_segs, out_segs)
    spec = make_spec(d.i_list, d.j_list, d.k_list, d.v_list, d.coeff_list, w_segs=d.w_seg_num, x_segs=d.x_seg_num,
                     y_segs=d.y_seg_num, out_segs=d.out_seg_num, u=d.u_dim, dtype="f32")
    for direction in ("fwd", "bwd"):
        tun = default_tuning(spec, direction)
        assert (tun.pipes, tun.vec, tun.ct, tun.groups) == (4, 2, 128, 1), (direction, tun)
    assert (default_tuning(spec, "fwd").stages == 10) == small


@pytest.mark.parametrize("layout", ["four_pipelines", "tuned", "tensor_memory"])
@pytest.mark.parametrize("fused_sh", [False, True], ids=["y_harmonics", "y_vectors"])
@pytest.mark.parametrize("in1,parity,w_segs,out_segs,small", SIGNATURES)
def test_wide_layout_matches_oracle(in1, parity, w_segs, out_segs, small, fused_sh, layout):
    """``four_pipelines``: the heuristic layout (one CTA of four pipelines, packed arithmetic), forced; ``tuned``: whatever
    the tuning database selects for the signature (what the benchmark and the model actually run); ``tensor_memory``: the
    backward with the receiver's grad_out row parked in tensor memory (one lane per consumer thread) and the shared memory
    it frees given to deeper rings."""
    from fasteq_b200.ops import fast_uniform1d_jit
    from fasteq_b200.ops import uniform1d_jit as u1d
    d = _descriptor(in1, parity)
    spec0 = make_spec(d.i_list, d.j_list, d.k_list, d.v_list, d.coeff_list, w_segs=d.w_seg_num, x_segs=d.x_seg_num,
                      y_segs=d.y_seg_num, out_segs=d.out_seg_num, u=d.u_dim, dtype="f32")
    if layout == "four_pipelines":
        u1d._TUNING_OVERRIDE.update(fwd=default_tuning(spec0, "fwd"), bwd=default_tuning(spec0, "bwd"))
    elif layout == "tensor_memory":
        u1d._TUNING_OVERRIDE.update(bwd=tensor_memory_tuning(spec0))
    try:
        _check_against_oracle(d, w_segs, fused_sh, layout)
    finally:
        u1d._TUNING_OVERRIDE.clear()


def tensor_memory_tuning(spec):
    import dataclasses
    return dataclasses.replace(default_tuning(spec, "bwd"), go_smem=False, go_tmem=True, stages=6)


def _check_against_oracle(d, w_segs, fused_sh, layout):
    from fasteq_b200.ops import fast_uniform1d_jit
    from fasteq_b200.ops import uniform1d_jit as u1d
    U, N = d.u_dim, 211
    g = torch.Generator().manual_seed(20 + w_segs)
    src, dst = _graph(N, g)
    E = int(dst.numel())
    assert E > 2000
    w = torch.randn(E, d.w_seg_num * U, generator=g)
    x = torch.randn(N, d.x_seg_num * U, generator=g)
    vec = torch.randn(E, 3, generator=g) * 1.7
    r = torch.randn(N, d.out_seg_num * U, generator=g)
    y_ref = spherical_harmonics_host(3, vec.double().numpy(), normalize=True)           # float64 [E, 16]
    meta = dict(d.meta(torch.float32, "cuda"))
    if fused_sh:
        meta["y_sh"] = ((0, 1, 2, 3), True, "component")
        y_dev = vec.cuda().requires_grad_(True)
    else:
        y_dev = torch.from_numpy(y_ref).float().cuda().requires_grad_(True)
    wd, xd = w.cuda().requires_grad_(True), x.cuda().requires_grad_(True)
    idx_in, idx_out = {1: src.int().cuda()}, {0: dst.int().cuda()}
    out = fast_uniform1d_jit(wd, xd, y_dev, idx_in, idx_out, meta)
    gw, gx, gy = torch.autograd.grad(out, (wd, xd, y_dev), r.cuda())

    # the modules that just ran
    call = u1d._Call(wd, xd, y_dev, idx_in, idx_out, meta)
    for direction, needs in (("fwd", (False, False, False)), ("bwd", (True, True, True))):
        tun = u1d._tuning_for(call.spec, direction, (wd, xd, y_dev), needs)
        assert tun.vec == 2
        if layout == "four_pipelines":
            assert tun.pipes == 4 and tun.groups == 1
        if layout == "tensor_memory" and direction == "bwd":
            assert tun.go_tmem and not tun.go_smem and tun.pipes == 4 and tun.stages == 6
        mod = u1d.get_module(call.spec, direction, needs, tuning=tun)
        assert mod.desc.threads == tun.pipes * (tun.groups * 64 + 32)
        assert mod.device_status() == 0

    paths = list(zip(d.i_list.tolist(), d.j_list.tolist(), d.k_list.tolist(), d.v_list.tolist()))
    a = lambda t, s: t.double().numpy().reshape(t.shape[0], s, -1)
    y64 = y_ref if fused_sh else y_dev.detach().cpu().double().numpy()
    y3 = y64.reshape(E, d.y_seg_num, 1)
    kw = dict(src_x=src.numpy(), dst=dst.numpy())
    ref = uniform1d_ref.uniform1d_forward(a(w, d.w_seg_num), a(x, d.x_seg_num), y3, paths, d.coeff_list, d.out_seg_num,
                                          num_out_rows=N, **kw)
    rgw, rgx, rgy = uniform1d_ref.uniform1d_backward(a(r, d.out_seg_num), a(w, d.w_seg_num), a(x, d.x_seg_num), y3, paths,
                                                     d.coeff_list, **kw)
    _close(out, ref, "forward")
    _close(gw, rgw, "grad_w")
    _close(gx, rgx, "grad_x")
    if fused_sh:
        # chain the oracle's harmonic gradient through the harmonics' Jacobian (central differences in float64)
        v64 = vec.double().numpy()
        jac = np.zeros((E, 16, 3))
        h = 1e-6
        for ax in range(3):
            dv = np.zeros(3); dv[ax] = h
            jac[:, :, ax] = (spherical_harmonics_host(3, v64 + dv, True) - spherical_harmonics_host(3, v64 - dv, True)) / (2 * h)
        rgv = np.einsum("ek,eka->ea", rgy.reshape(E, 16).astype(np.float64), jac)
        got = gy.detach().cpu().double().numpy()
        err = np.abs(got - rgv).max() / max(np.abs(rgv).max(), 1e-30)
        assert err <= 2e-5, f"grad_vec: relative error {err:.3e}"   # the finite-difference Jacobian adds ~1e-9; FP32 harmonics ~1e-6
    else:
        _close(gy, rgy, "grad_y")
    # rows without edges are written as exact zeros
    empty = torch.ones(N, dtype=torch.bool)
    empty[dst.unique()] = False
    assert torch.count_nonzero(out.detach()[empty.cuda()]) == 0


@pytest.mark.parametrize("in1,parity,variant", [("128x0e+128x1o+128x2e", None, "groups2"), ("128x0e+128x1o", "natural", "groups2"),
                                                ("128x0e+128x1o+128x2e", None, "groups2_two_pass"), ("64x0e+64x1o", None, "groups2"),
                                                ("128x0e+128x1o", None, "fwd_groups2")])
def test_two_thread_groups_match_oracle(in1, parity, variant):
    """Launch configurations the tuner may pick: two consumer thread groups per pipeline.  In the backward each group
    differentiates the terms of its own weight segments (its grad_w rows are its alone; both add into grad_x and into the
    per-warp partial sums of grad_y); in the forward each group owns a share of the output segments."""
    import dataclasses
    from fasteq_b200.ops import fast_uniform1d_jit
    from fasteq_b200.ops import uniform1d_jit as u1d
    d = _descriptor(in1, parity)
    U, N = d.u_dim, 97
    g = torch.Generator().manual_seed(5)
    src, dst = _graph(N, g)
    E = int(dst.numel())
    w = torch.randn(E, d.w_seg_num * U, generator=g)
    x = torch.randn(N, d.x_seg_num * U, generator=g)
    y = torch.randn(E, d.y_seg_num, generator=g)
    r = torch.randn(N, d.out_seg_num * U, generator=g)
    spec = make_spec(d.i_list, d.j_list, d.k_list, d.v_list, d.coeff_list, w_segs=d.w_seg_num, x_segs=d.x_seg_num,
                     y_segs=d.y_seg_num, out_segs=d.out_seg_num, u=d.u_dim, dtype="f32")
    direction = "fwd" if variant.startswith("fwd") else "bwd"
    base = default_tuning(spec, direction)
    tun = dataclasses.replace(base, groups=2, pipes=min(base.pipes, 2), two_pass=variant.endswith("two_pass"),
                              stages=min(base.stages, 3 if direction == "bwd" else 4), min_blocks=1)
    u1d._TUNING_OVERRIDE[direction] = tun
    try:
        wd, xd, yd = (t.cuda().requires_grad_(True) for t in (w, x, y))
        out = fast_uniform1d_jit(wd, xd, yd, {1: src.int().cuda()}, {0: dst.int().cuda()}, d.meta(torch.float32, "cuda"))
        gw, gx, gy = torch.autograd.grad(out, (wd, xd, yd), r.cuda())
        mod = u1d.get_module(spec, direction, (True, True, True) if direction == "bwd" else (False, False, False), tuning=tun)
        assert mod.desc.threads == tun.pipes * (2 * tun.ct // tun.vec + 32) and mod.device_status() == 0
    finally:
        u1d._TUNING_OVERRIDE.pop(direction, None)
    paths = list(zip(d.i_list.tolist(), d.j_list.tolist(), d.k_list.tolist(), d.v_list.tolist()))
    a = lambda t, s: t.double().numpy().reshape(t.shape[0], s, -1)
    kw = dict(src_x=src.numpy(), dst=dst.numpy())
    ref = uniform1d_ref.uniform1d_forward(a(w, d.w_seg_num), a(x, d.x_seg_num), a(y, d.y_seg_num), paths, d.coeff_list, d.out_seg_num,
                                          num_out_rows=N, **kw)
    rgw, rgx, rgy = uniform1d_ref.uniform1d_backward(a(r, d.out_seg_num), a(w, d.w_seg_num), a(x, d.x_seg_num), a(y, d.y_seg_num), paths,
                                                     d.coeff_list, **kw)
    _close(out, ref, "forward"); _close(gw, rgw, "grad_w"); _close(gx, rgx, "grad_x"); _close(gy, rgy, "grad_y")


@pytest.mark.parametrize("in1,u_pipes", [("64x0e+64x1o", 4), ("128x0e+128x1o+128x2e", 3)])
def test_float64_backward_with_the_gradient_row_in_tensor_memory(in1, u_pipes):
    """FP64 on the tensor-memory layout (a double takes two 32-bit columns of the thread's lane; 64-channel tiles, so a
    pipeline has two consumer warps), all three gradients against the oracle at 1e-12."""
    import dataclasses
    from fasteq_b200.ops import fast_uniform1d_jit
    from fasteq_b200.ops import uniform1d_jit as u1d
    d = _descriptor(in1, None)
    U, N = d.u_dim, 97
    g = torch.Generator().manual_seed(8)
    src, dst = _graph(N, g)
    E = int(dst.numel())
    w = torch.randn(E, d.w_seg_num * U, generator=g, dtype=torch.float64)
    x = torch.randn(N, d.x_seg_num * U, generator=g, dtype=torch.float64)
    y = torch.randn(E, d.y_seg_num, generator=g, dtype=torch.float64)
    r = torch.randn(N, d.out_seg_num * U, generator=g, dtype=torch.float64)
    spec = make_spec(d.i_list, d.j_list, d.k_list, d.v_list, d.coeff_list, w_segs=d.w_seg_num, x_segs=d.x_seg_num,
                     y_segs=d.y_seg_num, out_segs=d.out_seg_num, u=d.u_dim, dtype="f64")
    base = default_tuning(spec, "bwd")
    tun = dataclasses.replace(base, pipes=u_pipes, go_smem=False, go_tmem=True, stages=2, min_blocks=1)
    u1d._TUNING_OVERRIDE["bwd"] = tun
    try:
        wd, xd, yd = (t.cuda().requires_grad_(True) for t in (w, x, y))
        out = fast_uniform1d_jit(wd, xd, yd, {1: src.int().cuda()}, {0: dst.int().cuda()}, d.meta(torch.float64, "cuda"))
        gw, gx, gy = torch.autograd.grad(out, (wd, xd, yd), r.cuda())
        mod = u1d.get_module(spec, "bwd", (True, True, True), tuning=tun)
        assert mod.device_status() == 0
    finally:
        u1d._TUNING_OVERRIDE.pop("bwd", None)
    paths = list(zip(d.i_list.tolist(), d.j_list.tolist(), d.k_list.tolist(), d.v_list.tolist()))
    a = lambda t, s: t.numpy().reshape(t.shape[0], s, -1)
    kw = dict(src_x=src.numpy(), dst=dst.numpy())
    rgw, rgx, rgy = uniform1d_ref.uniform1d_backward(a(r, d.out_seg_num), a(w, d.w_seg_num), a(x, d.x_seg_num), a(y, d.y_seg_num), paths,
                                                     d.coeff_list, **kw)
    for got, ref, name in ((gw, rgw, "grad_w"), (gx, rgx, "grad_x"), (gy, rgy, "grad_y")):
        err = np.abs(got.detach().cpu().numpy().reshape(ref.shape) - ref).max() / np.abs(ref).max()
        assert err <= 1e-12, f"{name}: relative error {err:.3e}"
