"""The allocation-free forward entry point against the regular one (collected last on purpose).

``fasteq_u1d_forward_noalloc`` serves callers that cannot allocate device memory at call time (a
simulation-engine plug-in with a fixed arena, a loop that must not hit an allocation's implicit sync): it derives the CSR
offsets and the CTA partition into an array built into the module instead of caller-owned buffers.
Two calls in a row with different graphs check that what the first call left in that shared array
does not leak into the second.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-5  # same relative bound as the FP32 parity tests


def _case(n_nodes, n_edges, seed):
    from fasteq_b200.descriptors import channelwise_tensor_product, full_channelwise_instructions
    from fasteq_b200.irreps import Irreps
    in1, sh = "64x0e+64x1o", Irreps.spherical_harmonics(3)
    io, ins = full_channelwise_instructions(in1, sh, 3)
    d = channelwise_tensor_product(in1, sh, io, ins)
    g = torch.Generator().manual_seed(seed)
    src = torch.randint(0, n_nodes, (n_edges,), generator=g)
    dst, order = torch.sort(torch.randint(0, n_nodes, (n_edges,), generator=g), stable=True)
    src = src[order]
    U = d.u_dim
    w = torch.randn(n_edges, d.w_seg_num * U, generator=g).cuda()
    x = torch.randn(n_nodes, d.x_seg_num * U, generator=g).cuda()
    y = torch.randn(n_edges, d.y_seg_num, generator=g).cuda()
    return d, src.int().cuda(), dst.int().cuda(), w, x, y


def test_noalloc_forward_matches_regular_entry_point_twice():
    from fasteq_b200.ops import fast_uniform1d_jit
    from fasteq_b200.ops import uniform1d_jit as u1d
    stream = torch.cuda.current_stream().cuda_stream
    for n_nodes, n_edges, seed in ((300, 4000, 1), (77, 650, 2)):
        d, src, dst, w, x, y = _case(n_nodes, n_edges, seed)
        meta = d.meta(torch.float32, "cuda")
        ref = fast_uniform1d_jit(w, x, y, {1: src}, {0: dst}, meta)
        call = u1d._Call(w, x, y, {1: src}, {0: dst}, meta)
        mod = u1d.get_module(call.spec, "fwd", tuning=u1d._tuning_for(call.spec, "fwd", (w, x, y)))
        out = torch.full_like(ref, float("nan"))
        rc = mod.forward_noalloc(dst.data_ptr(), src.data_ptr(), n_edges, n_nodes, n_nodes, w.data_ptr(), x.data_ptr(),
                                 y.data_ptr(), out.data_ptr(), stream)
        assert rc == 0, mod.last_error()
        torch.cuda.synchronize()
        scale = ref.abs().max().item()
        assert (out - ref).abs().max().item() <= TOL * scale
        assert mod.device_status() == 0


def _both(d, src, dst, w, x, y, n_nodes):
    """(regular entry point through the public operator, allocation-free entry point) on the same inputs."""
    from fasteq_b200.ops import fast_uniform1d_jit
    from fasteq_b200.ops import uniform1d_jit as u1d
    meta = d.meta(torch.float32, "cuda")
    ref = fast_uniform1d_jit(w, x, y, {1: src}, {0: dst}, meta)
    call = u1d._Call(w, x, y, {1: src}, {0: dst}, meta)
    mod = u1d.get_module(call.spec, "fwd", tuning=u1d._tuning_for(call.spec, "fwd", (w, x, y)))
    out = torch.full_like(ref, float("nan"))
    nz = lambda t: t.data_ptr() if t.numel() else None
    rc = mod.forward_noalloc(nz(dst), nz(src), int(dst.numel()), n_nodes, n_nodes, nz(w), x.data_ptr(), nz(y), out.data_ptr(),
                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0, mod.last_error()
    torch.cuda.synchronize()
    assert mod.device_status() == 0
    return ref, out


def test_noalloc_forward_with_empty_receivers_and_without_edges():
    """Receivers without edges in the middle and at both ends of the range, then a call with no edge at all
    (every row is written as zeros); each against the regular entry point."""
    n_nodes = 90
    d, src, dst, w, x, y = _case(n_nodes, 1200, 5)
    keep = (dst >= 7) & (dst < 71) & (dst % 5 != 0)          # rows 0-6, 71-89 and every fifth row stay empty
    src, dst, w, y = src[keep].contiguous(), dst[keep].contiguous(), w[keep].contiguous(), y[keep].contiguous()
    ref, out = _both(d, src, dst, w, x, y, n_nodes)
    assert (out - ref).abs().max().item() <= TOL * ref.abs().max().item()
    assert torch.count_nonzero(out[71:]) == 0 and torch.count_nonzero(out[:7]) == 0 and torch.count_nonzero(out[10]) == 0
    ref0, out0 = _both(d, src[:0], dst[:0], w[:0], x, y[:0], n_nodes)
    assert torch.count_nonzero(ref0) == 0 and torch.count_nonzero(out0) == 0 and not torch.isnan(out0).any()


def test_noalloc_forward_with_a_channel_tail():
    """33 channels: the last channel tile is partial (U is not a multiple of the tile)."""
    from fasteq_b200.descriptors import channelwise_tensor_product, full_channelwise_instructions
    from fasteq_b200.irreps import Irreps
    in1, sh = "33x0e+33x1o", Irreps.spherical_harmonics(2)
    io, ins = full_channelwise_instructions(in1, sh, 2)
    d = channelwise_tensor_product(in1, sh, io, ins)
    g = torch.Generator().manual_seed(8)
    n_nodes, n_edges = 40, 500
    src = torch.randint(0, n_nodes, (n_edges,), generator=g)
    dst, order = torch.sort(torch.randint(0, n_nodes, (n_edges,), generator=g), stable=True)
    src = src[order].int().cuda()
    w = torch.randn(n_edges, d.w_seg_num * 33, generator=g).cuda()
    x = torch.randn(n_nodes, d.x_seg_num * 33, generator=g).cuda()
    y = torch.randn(n_edges, d.y_seg_num, generator=g).cuda()
    ref, out = _both(d, src, dst.int().cuda(), w, x, y, n_nodes)
    assert (out - ref).abs().max().item() <= TOL * ref.abs().max().item()


def test_noalloc_forward_refuses_oversized_graphs():
    from fasteq_b200.ops import uniform1d_jit as u1d
    d, src, dst, w, x, y = _case(16, 40, 3)
    meta = d.meta(torch.float32, "cuda")
    call = u1d._Call(w, x, y, {1: src}, {0: dst}, meta)
    mod = u1d.get_module(call.spec, "fwd", tuning=u1d._tuning_for(call.spec, "fwd", (w, x, y)))
    out = torch.empty(16, d.out_seg_num * d.u_dim, device="cuda")
    rc = mod.forward_noalloc(dst.data_ptr(), src.data_ptr(), 40, 262145, 16, w.data_ptr(), x.data_ptr(), y.data_ptr(),
                             out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 1  # FASTEQ_UNSUPPORTED, nothing launched
    assert "262144" in mod.last_error()
