"""GPU parity of the Uniform1D (ChannelwiseTensorProduct) kernels against the CPU oracle,
through the public operator and therefore through the C ABI."""
import numpy as np
import pytest
import torch

from fasteq_b200.descriptors import channelwise_tensor_product, full_channelwise_instructions
from fasteq_b200.irreps import Irreps
from oracle import uniform1d_ref

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.float64: 1e-11}  # relative to the largest reference magnitude


def _close(got: torch.Tensor, ref: np.ndarray, dtype, what=""):
    got = got.detach().cpu().double().numpy().reshape(ref.shape)
    scale = max(np.abs(ref).max(), 1e-30)
    err = np.abs(got - ref).max() / scale
    assert err <= TOL[dtype], f"{what}: relative error {err:.3e} > {TOL[dtype]:.0e}"


def _run_case(desc_meta, paths, coeffs, segs, U, N, E, dtype, *, shared_w=False, gather_x=True, gather_y=False,
              scatter=True, y_vec=False, sort=True, seed=0, offset=False, check_grads=True):
    from fasteq_b200.ops import fast_uniform1d_jit
    I, J, K, V = segs
    g = torch.Generator().manual_seed(seed)
    src = torch.randint(0, N, (E,), generator=g)
    dst = torch.randint(0, N, (E,), generator=g)
    if sort:
        dst, order = torch.sort(dst, stable=True)
        src = src[order]
    Uy = U if y_vec else 1
    w = torch.randn(1 if shared_w else E, I * U, generator=g, dtype=torch.float64)
    x = torch.randn(N if gather_x else E, J * U, generator=g, dtype=torch.float64)
    y = torch.randn(N if gather_y else E, K * Uy, generator=g, dtype=torch.float64)
    r = torch.randn(N if scatter else E, V * U, generator=g, dtype=torch.float64)
    w, x, y, r = (t.to(dtype) for t in (w, x, y, r))

    def dev(t):
        if offset:  # contiguous view at a 1-element storage offset (not 16-byte aligned)
            return torch.cat((t.new_zeros(1), t.reshape(-1)))[1:].view(t.shape).cuda().requires_grad_(True) if False else \
                torch.cat((t.new_zeros(1).cuda(), t.reshape(-1).cuda()))[1:].view(t.shape).requires_grad_(True)
        return t.cuda().requires_grad_(True)

    wd, xd, yd = dev(w), dev(x), dev(y)
    inp = {}
    if gather_x:
        inp[1] = src.int().cuda()
    if gather_y:
        inp[2] = src.int().cuda()
    outi = {0: dst.int().cuda()} if scatter else {}
    out = fast_uniform1d_jit(wd, xd, yd, inp, outi, desc_meta(dtype))
    wn, xn, yn = (t.double().numpy() for t in (w, x, y))
    kw = dict(src_x=src.numpy() if gather_x else None, src_y=src.numpy() if gather_y else None,
              dst=dst.numpy() if scatter else None)
    ref = uniform1d_ref.uniform1d_forward(wn.reshape(-1, I, U), xn.reshape(-1, J, U), yn.reshape(-1, K, Uy), paths, coeffs, V,
                                          num_out_rows=N, **kw)
    _close(out, ref.reshape(out.shape), dtype, "forward")
    if check_grads:
        gw, gx, gy = torch.autograd.grad((out * r.cuda()).sum(), (wd, xd, yd))
        rgw, rgx, rgy = uniform1d_ref.uniform1d_backward(r.double().numpy().reshape(-1, V, U), wn.reshape(-1, I, U),
                                                         xn.reshape(-1, J, U), yn.reshape(-1, K, Uy), paths, coeffs, **kw)
        _close(gw, rgw.reshape(gw.shape), dtype, "grad_w")
        _close(gx, rgx.reshape(gx.shape), dtype, "grad_x")
        _close(gy, rgy.reshape(gy.shape), dtype, "grad_y")
    return out


def _tp(in1, lmax_sh, lmax_out):
    io, ins = full_channelwise_instructions(in1, Irreps.spherical_harmonics(lmax_sh), lmax_out)
    d = channelwise_tensor_product(in1, Irreps.spherical_harmonics(lmax_sh), io, ins)
    paths = list(zip(d.i_list.tolist(), d.j_list.tolist(), d.k_list.tolist(), d.v_list.tolist()))
    return d, paths


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_config0_forward_backward(dtype):
    """benchmark configuration 0: 128x0e+128x1o+128x2e (x) SH l<=3 -> all paths l<=3, 512 nodes, 4096 dst-sorted edges."""
    d, paths = _tp("128x0e+128x1o+128x2e", 3, 3)
    _run_case(lambda dt: d.meta(dt, "cuda"), paths, d.coeff_list, (d.w_seg_num, d.x_seg_num, d.y_seg_num, d.out_seg_num),
              128, 512, 4096, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_mace_layer_signature(dtype):
    """64x0e+64x1o (x) SH l<=3 -> l<=3 (13 weight segments, 64-channel tiles), receivers with no edges, unsorted dst.
    The 128-channel layouts of the same couplings are covered by tests/test_u1d_wide_gpu.py."""
    d, paths = _tp("64x0e+64x1o", 3, 3)
    _run_case(lambda dt: d.meta(dt, "cuda"), paths, d.coeff_list, (d.w_seg_num, d.x_seg_num, d.y_seg_num, d.out_seg_num),
              64, 300, 700, dtype, sort=False, seed=3)


REF_PATHS = [(0, 0, 0, 0), (1, 1, 1, 0), (0, 1, 0, 2)]
REF_PATHS_VEC = [(0, 0, 0, 0), (1, 1, 1, 0), (0, 1, 0, 1)]
REF_COEFFS = [.5, -.25, .75]


def _ref_meta(paths, U, V, y_vec):
    def make(dtype):
        cols = list(zip(*paths))
        m = {n: torch.tensor(c, dtype=torch.int32, device="cuda") for n, c in zip(["i_list", "j_list", "k_list", "v_list"], cols)}
        m.update(coeff_list=torch.tensor(REF_COEFFS, dtype=dtype, device="cuda"), w_seg_num=2, x_seg_num=2, y_seg_num=2,
                 out_seg_num=V, u_dim=U, size_list=[2 * U, 2 * U, 2 * (U if y_vec else 1), V * U])
        return m
    return make


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("kind", ["x_tail_holes", "xy_multi_path", "y_tail", "scatter_fallback"])
def test_reference_indexed_cases(dtype, kind):
    """The four cases of the reference's value test (tests/adapters/test_uniform1d_hip_forward.py:44-78):
    shared weights, channel tails U in {33, 65}, vector y, gathered y, an output segment no path
    writes, scatter, and contiguous operands at a non-zero storage offset."""
    N, E = 5, 11
    U = 65 if kind in ("x_tail_holes", "scatter_fallback") else (128 if kind == "xy_multi_path" else 33)
    vector = kind == "xy_multi_path"
    shared = kind in ("x_tail_holes", "xy_multi_path")
    sx = kind != "y_tail"
    sy = kind in ("xy_multi_path", "y_tail")
    scatter = kind == "scatter_fallback"
    paths = REF_PATHS_VEC if vector else REF_PATHS
    V = 2 if vector else 3
    out = _run_case(_ref_meta(paths, U, V, vector), paths, REF_COEFFS, (2, 2, 2, V), U, N, E, dtype, shared_w=shared,
                    gather_x=sx, gather_y=sy, scatter=scatter, y_vec=vector, sort=False, seed=1701, offset=True)
    if not vector:
        assert torch.count_nonzero(out.reshape(-1, V, U)[:, 1]) == 0


def test_rejects_non_contiguous_and_cpu():
    from fasteq_b200.ops import fast_uniform1d_jit
    meta = _ref_meta(REF_PATHS, 33, 3, False)(torch.float32)
    w = torch.randn(11, 2 * 33 * 2, device="cuda")[:, ::2]
    x = torch.randn(5, 66, device="cuda")
    y = torch.randn(11, 2, device="cuda")
    src = (torch.arange(11, device="cuda") * 3 % 5).int()
    with pytest.raises(RuntimeError, match="contiguous"):
        fast_uniform1d_jit(w, x, y, {1: src}, {}, meta)
    with pytest.raises(RuntimeError, match="CUDA"):
        fast_uniform1d_jit(w.contiguous().cpu(), x.cpu(), y.cpu(), {1: src.cpu()}, {}, meta)


def test_empty_graph_and_isolated_receivers():
    from fasteq_b200.ops import fast_uniform1d_jit
    d, paths = _tp("32x0e+32x1o", 2, 2)
    meta = d.meta(torch.float32, "cuda")
    N = 7
    x = torch.randn(N, d.x_seg_num * 32, device="cuda")
    for E in (0, 1):
        w = torch.randn(E, d.w_seg_num * 32, device="cuda", requires_grad=True)
        y = torch.randn(E, d.y_seg_num, device="cuda", requires_grad=True)
        src = torch.zeros(E, dtype=torch.int32, device="cuda")
        dst = torch.full((E,), 4, dtype=torch.int32, device="cuda")
        xg = x.clone().requires_grad_(True)
        out = fast_uniform1d_jit(w, xg, y, {1: src}, {0: dst}, meta)
        assert out.shape == (N, d.out_seg_num * 32)
        rows = out.detach().abs().sum(dim=1)
        assert torch.count_nonzero(rows) == (1 if E else 0)
        # backward of an empty edge list: empty per-edge gradients, a zero sender gradient
        gw, gx, gy = torch.autograd.grad(out.sum(), (w, xg, y))
        assert gw.shape == w.shape and gy.shape == y.shape and gx.shape == x.shape
        assert torch.count_nonzero(gx.abs().sum(dim=1)) == (1 if E else 0)


def test_no_device_fault_recorded():
    """After the parity cases no kernel may have recorded a wait timeout or a bad index."""
    from fasteq_b200.ops import uniform1d_jit
    torch.cuda.synchronize()
    for mod in uniform1d_jit._MODULES.values():
        assert mod.device_status() == 0


def test_double_backward_matches_torch_autograd():
    """Gradients of a function of the first-order gradients (a force-matching loss) against torch
    autograd through a dense float64 restatement of the operator."""
    from fasteq_b200.ops import fast_uniform1d_jit
    from oracle.mace_style_ref import u1d_scatter
    d, paths = _tp("32x0e+32x1o", 2, 2)
    N, E, U = 12, 60, d.u_dim
    g = torch.Generator().manual_seed(4)
    src = torch.randint(0, N, (E,), generator=g)
    dst, order = torch.sort(torch.randint(0, N, (E,), generator=g), stable=True)
    src = src[order]
    w = torch.randn(E, d.w_seg_num * U, generator=g, dtype=torch.float64)
    x = torch.randn(N, d.x_seg_num * U, generator=g, dtype=torch.float64)
    y = torch.randn(E, d.y_seg_num, generator=g, dtype=torch.float64)
    r = torch.randn(N, d.out_seg_num * U, generator=g, dtype=torch.float64)
    ax, ay, aw = (torch.randn(t.shape, generator=g, dtype=torch.float64) for t in (x, y, w))

    def loss(op, dev):
        wd, xd, yd = (t.to(dev).requires_grad_(True) for t in (w, x, y))
        out = op(wd, xd, yd)
        gw, gx, gy = torch.autograd.grad((out * r.to(dev)).sum(), (wd, xd, yd), create_graph=True)
        second = (gx * ax.to(dev)).sum() + (gy * ay.to(dev)).sum() + (gw * aw.to(dev)).sum() + (out ** 2).sum()
        return torch.autograd.grad(second, (wd, xd, yd))

    meta = d.meta(torch.float64, "cuda")
    got = loss(lambda a, b, c: fast_uniform1d_jit(a, b, c, {1: src.int().cuda()}, {0: dst.int().cuda()}, meta), "cuda")
    ref = loss(lambda a, b, c: u1d_scatter(a, b, c, d, src, dst, N), "cpu")
    for name, a, b in zip(("w", "x", "y"), got, ref):
        _close(a, b.numpy(), torch.float64, f"second-order gradient wrt {name}")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float64, 1e-11)])
@pytest.mark.parametrize("in1,lmax", [("32x0e+32x1o", 2), ("128x0e+128x1o", 3)])
def test_in_kernel_spherical_harmonics_match_the_two_step_path(in1, lmax, dtype, tol):
    """y = edge vectors, harmonics evaluated by the producer: same output and same gradients (w, x and the
    vectors) as harmonics computed first and passed as the y operand."""
    from fasteq_b200.nn.modules import ChannelwiseTensorProduct
    from fasteq_b200.ops.spherical_harmonics import SphericalHarmonics
    sh_ir = Irreps.spherical_harmonics(lmax)
    io, ins = full_channelwise_instructions(in1, sh_ir, lmax)
    tp = ChannelwiseTensorProduct(in1, sh_ir, io, ins)
    d = tp.descriptor
    g = torch.Generator().manual_seed(11)
    N, E = 57, 700
    dst = torch.sort(torch.randint(0, N, (E,), generator=g)).values.int().cuda()
    src = torch.randint(0, N, (E,), generator=g).int().cuda()
    w = torch.randn(E, d.w_seg_num * d.u_dim, generator=g, dtype=torch.float64).to(dtype).cuda().requires_grad_(True)
    x = torch.randn(N, d.x_seg_num * d.u_dim, generator=g, dtype=torch.float64).to(dtype).cuda().requires_grad_(True)
    vec = (torch.randn(E, 3, generator=g, dtype=torch.float64) * 2.0).to(dtype).cuda().requires_grad_(True)
    r = torch.randn(N, d.out_seg_num * d.u_dim, generator=g, dtype=torch.float64).to(dtype).cuda()
    sh = SphericalHarmonics(list(range(lmax + 1)), True, "component")
    out_ref = tp(x, sh(vec), w, dst, src)
    ref = torch.autograd.grad(out_ref, (w, x, vec), r)
    out = tp(x, None, w, dst, src, edge_vec=vec)
    got = torch.autograd.grad(out, (w, x, vec), r)
    scale = lambda t: float(t.detach().abs().max())
    assert float((out - out_ref).detach().abs().max()) <= tol * scale(out_ref)
    for a, b in zip(got, ref):
        assert a.shape == b.shape and float((a - b).abs().max()) <= tol * scale(b)
    with pytest.raises(RuntimeError):
        o = tp(x, None, w, dst, src, edge_vec=vec)
        (gv,) = torch.autograd.grad(o, vec, r, create_graph=True)
