"""GPU parity of the 3xTF32 tensor-core dense layer (radial MLP) against float64 matmul: shapes of the
config-1 radial MLP (8 -> 64 -> 64 -> 64 -> weight_numel), row counts that are not tile multiples,
and enough row tiles that every persistent CTA walks several tiles."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.double() - b).norm() / b.norm().clamp_min(1e-30))


@pytest.mark.parametrize("M,N,K", [
    (1, 64, 8), (77, 64, 64), (128, 8, 64), (1000, 64, 1664), (513, 1664, 64), (300, 512, 64), (257, 128, 128),
    (148 * 128 * 3 + 77, 64, 64), (148 * 128 * 2 + 5, 64, 8), (40000, 128, 128), (20000, 12, 20),
    # wide shallow layers: every persistent CTA of the A-stationary kernel walks several row blocks
    (148 * 128 * 3 + 77, 512, 64), (148 * 128 * 2 + 5, 256, 32), (5000, 260, 40), (148 * 128 + 1, 1280, 64),
])
def test_dense_forward_matches_float64(M, N, K):
    from fasteq_b200.ops.dense import dense, tensorcore_device_status
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) / K ** 0.5
    ref = x.double() @ w.double().t()
    out = dense(x.cuda(), w.cuda())
    assert out.shape == (M, N)
    assert _rel(out.cpu(), ref) <= (2e-6 if K <= 128 else 1e-5), _rel(out.cpu(), ref)   # long K: measured 4e-6 at K = 1664 (the reference allows 2e-5)
    # element-wise too: a misplaced tile would hide in a norm
    assert float((out.cpu().double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    assert tensorcore_device_status() == 0


def test_dense_gradients():
    from fasteq_b200.ops.dense import dense
    g = torch.Generator().manual_seed(3)
    M, N, K = 148 * 128 + 300, 64, 64
    x = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) / 8
    r = torch.randn(M, N, generator=g)
    xd, wd = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    gx, gw = torch.autograd.grad(dense(xd, wd), (xd, wd), r.cuda())
    assert _rel(gx.cpu(), r.double() @ w.double()) <= 2e-6
    assert _rel(gw.cpu(), r.double().t() @ x.double()) <= 1e-5


def test_dense_leading_dimensions_and_fallback_dtypes():
    from fasteq_b200.ops.dense import dense
    g = torch.Generator().manual_seed(4)
    x = torch.randn(5, 31, 8, generator=g, dtype=torch.float64)
    w = torch.randn(64, 8, generator=g, dtype=torch.float64)
    out = dense(x.cuda(), w.cuda())            # float64: the FP64 FMA tile kernel of the SO3Linear family
    assert out.shape == (5, 31, 64) and _rel(out.cpu(), x @ w.t()) <= 1e-14
    out32 = dense(x.float().cuda(), w.float().cuda())
    assert out32.shape == (5, 31, 64) and _rel(out32.cpu(), x @ w.t()) <= 2e-6


def test_dense_second_order():
    from fasteq_b200.ops.dense import dense
    g = torch.Generator().manual_seed(8)
    M, N, K = 300, 64, 64
    x, w, go = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g) / 8, torch.randn(M, N, generator=g)
    rx, rw = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)

    def second(fn, dev, dt):
        xt, wt, gt = (t.to(dt).to(dev).requires_grad_(True) for t in (x, w, go))
        gx, gw = torch.autograd.grad(fn(xt, wt), (xt, wt), gt, create_graph=True)
        L = (gx * rx.to(dt).to(dev)).sum() + (gw * rw.to(dt).to(dev)).sum()
        return [t.detach().cpu().double() for t in torch.autograd.grad(L, (gt, xt, wt))]

    ref = second(lambda a, b: a @ b.t(), "cpu", torch.float64)
    got = second(dense, "cuda", torch.float32)
    for a, b in zip(got, ref):
        assert _rel(a, b) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(1, 64, 8), (777, 64, 64), (1500, 4352, 64), (300, 70, 33), (130, 26, 10), (4000, 72, 200)])
def test_float64_dense_runs_on_the_library_kernels(M, N, K, monkeypatch):
    """FP64 (benchmark configuration 2's radial MLP): forward, both gradients and a second-order term on the kernels
    behind ``fasteq_eqlinear_forward / _dgrad / _wgrad`` -- no library GEMM: ``torch.matmul`` is made to fail for CUDA
    operands while the layer runs.  Even extents take the tensor-core (DMMA) kernel: a reduction of at most 64 keeps
    the A tile in shared memory across column blocks (1500 x 4352 x 64 forward), longer ones stream it (the same
    case's grad_x with K = 4352, and K = 200 with a partial column block); odd extents take the FMA kernel."""
    from fasteq_b200.ops import dense as dmod
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g, dtype=torch.float64)
    w = torch.randn(N, K, generator=g, dtype=torch.float64) / K ** 0.5
    r = torch.randn(M, N, generator=g, dtype=torch.float64)
    a = torch.randn(M, K, generator=g, dtype=torch.float64)

    def run(fn, dev):
        xt, wt = x.to(dev).requires_grad_(True), w.to(dev).requires_grad_(True)
        out = fn(xt, wt)
        gx, gw = torch.autograd.grad(out, (xt, wt), r.to(dev), create_graph=True)
        (d2w,) = torch.autograd.grad((gx * a.to(dev)).sum(), wt)          # d/dW of <g W, a> = g^T a
        return [t.detach().cpu() for t in (out, gx, gw, d2w)]

    ref = run(lambda p, q: p @ q.t(), "cpu")
    real = torch.Tensor.__matmul__

    def guarded(self, other):
        assert not (self.is_cuda or other.is_cuda), "a library GEMM was called on CUDA tensors"
        return real(self, other)
    monkeypatch.setattr(torch.Tensor, "__matmul__", guarded)
    got = run(dmod.dense, "cuda")
    monkeypatch.undo()
    for p, q in zip(got, ref):
        assert _rel(p, q) <= 1e-13


def test_misaligned_float32_operand_takes_the_fma_kernel():
    """An FP32 operand that is not 16-byte aligned is refused by the tensor-core kernel; the FP32 FMA kernel takes it."""
    from fasteq_b200.ops.dense import dense
    g = torch.Generator().manual_seed(5)
    M, N, K = 500, 64, 64
    buf = torch.randn(M * K + 1, generator=g).cuda()
    x = buf[1:].view(M, K)                                  # contiguous, 4 bytes past a 16-byte boundary
    assert x.data_ptr() % 16 == 4
    w = (torch.randn(N, K, generator=g) / 8).cuda()
    out = dense(x, w)
    assert _rel(out.cpu(), x.cpu().double() @ w.cpu().double().t()) <= 2e-6
