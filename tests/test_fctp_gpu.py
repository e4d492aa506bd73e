"""fast_fctp (species-indexed fully connected tensor product) against the direct torch equations of the
reference's own check (test/smoke_eqlinear_other_ops.py:38-56) and a larger multi-irrep case."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(w4, x3, species, i_for_k, p_for_k, val_for_k, alpha):
    B, K, Wd = x3.shape[0], len(i_for_k), w4.shape[3]
    out = x3.new_zeros(B, K, Wd)
    for k, (i, p, v) in enumerate(zip(i_for_k, p_for_k, val_for_k)):
        if i < 0:
            continue
        wsel = w4[p][:, species, :].permute(1, 0, 2)            # [B, U, W]
        out[:, k] = torch.einsum("bu,buw->bw", x3[:, i], wsel) * v * alpha
    return out.reshape(B, -1)


def _meta(i_for_k, p_for_k, val_for_k, alpha, P, U, V, W, I, dtype):
    meta = {key: None for key in ("cg_indices", "cg_values", "cg_i_all", "cg_j_all", "cg_k_all", "cg_val_all", "nnz_per_path",
                                  "K_per_path", "path_offset")}
    meta.update(i_for_k=torch.tensor(i_for_k, dtype=torch.int32, device="cuda"), p_for_k=torch.tensor(p_for_k, dtype=torch.int32, device="cuda"),
                val_for_k=torch.tensor(val_for_k, dtype=dtype, device="cuda"), cg_val_0=alpha, P=P, nnz0=2, U=U, V=V, W=W,
                K_total=len(i_for_k), I_total=I, can_use_empty_grad_x=True)
    return meta


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float64, 1e-12)])
def test_reference_smoke_case(dtype, tol):
    from fasteq_b200.ops.fctp import fast_fctp
    torch.manual_seed(23)
    batch, channels, species, width, paths = 8, 16, 4, 16, 2
    x = torch.randn(batch, paths * channels, device="cuda", dtype=dtype, requires_grad=True)
    y = torch.randn(batch, species, device="cuda", dtype=dtype)
    w = torch.randn(paths, channels, species, width, device="cuda", dtype=dtype, requires_grad=True)
    meta = _meta([0, 1], [0, 1], [0.5, 0.75], 0.8, paths, channels, species, width, paths, dtype)
    ref = _reference(w, x.reshape(batch, paths, channels), y.argmax(1), [0, 1], [0, 1], [0.5, 0.75], 0.8)
    out = fast_fctp(w, x, y, meta)
    torch.testing.assert_close(out, ref, rtol=tol, atol=tol)
    g = torch.randn_like(out)
    got = torch.autograd.grad(out, (x, w), g)
    exp = torch.autograd.grad(ref, (x, w), g)
    for a, b in zip(got, exp):
        torch.testing.assert_close(a, b, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float64, 1e-12)])
def test_mace_skip_connection_shape(dtype, tol):
    """128x0e+128x1o -> 128x0e+128x1o with 10 species: two weight paths, the three 1o rows share one; one
    masked output row; a species without nodes; batch that is not a tile multiple."""
    from fasteq_b200.ops.fctp import fast_fctp
    g = torch.Generator().manual_seed(5)
    B, U, V, Wd, P, I = 777, 128, 10, 128, 2, 4
    i_for_k, p_for_k, val = [0, 1, 2, 3, -1], [0, 1, 1, 1, 0], [0.3, 0.7, 0.7, 0.7, 1.0]
    x = torch.randn(B, I * U, generator=g, dtype=torch.float64).to(dtype).cuda().requires_grad_(True)
    w = (torch.randn(P * U * V * Wd, generator=g, dtype=torch.float64) / U ** 0.5).to(dtype).cuda().requires_grad_(True)
    sp = torch.randint(0, V - 1, (B,), generator=g)                 # species V-1 never occurs
    y = torch.nn.functional.one_hot(sp, V).to(dtype).cuda()
    meta = _meta(i_for_k, p_for_k, val, 1.25, P, U, V, Wd, I, dtype)
    xd, wd = x.detach().double().requires_grad_(True), w.detach().double().requires_grad_(True)
    ref = _reference(wd.reshape(P, U, V, Wd), xd.reshape(B, I, U), sp.cuda(), i_for_k, p_for_k, val, 1.25)
    out = fast_fctp(w, x, y, meta)
    assert out.shape == (B, 5 * Wd)
    scale = float(ref.abs().max())
    assert float((out.double() - ref).abs().max()) <= tol * scale
    assert float(out[:, 4 * Wd:].abs().max()) == 0.0
    r = torch.randn(out.shape, generator=g, dtype=torch.float64).cuda()
    gx, gw = torch.autograd.grad(out, (x, w), r.to(dtype))
    rx, rw = torch.autograd.grad(ref, (xd, wd), r)
    assert float((gx.double() - rx).abs().max()) <= tol * float(rx.abs().max())
    assert float((gw.double() - rw).abs().max()) <= tol * float(rw.abs().max())


def test_precomputed_species_groups_give_the_same_result():
    """``meta["species_groups"]`` (computed once per structure) removes the per-call host synchronisation; the result
    is bit-identical to the call that derives the groups itself."""
    from fasteq_b200.ops.fctp import fast_fctp, fctp_species_groups
    g = torch.Generator().manual_seed(6)
    B, U, V, Wd, P, I = 300, 64, 5, 64, 2, 4
    i_for_k, p_for_k, val = [0, 1, 2, 3], [0, 1, 1, 1], [0.3, 0.7, 0.7, 0.7]
    x = torch.randn(B, I * U, generator=g).cuda()
    w = (torch.randn(P * U * V * Wd, generator=g) / U ** 0.5).cuda()
    y = torch.nn.functional.one_hot(torch.randint(0, V, (B,), generator=g), V).float().cuda()
    meta = _meta(i_for_k, p_for_k, val, 1.0, P, U, V, Wd, I, torch.float32)
    ref = fast_fctp(w, x, y, meta)
    meta2 = dict(meta, species_groups=fctp_species_groups(y))
    assert torch.equal(fast_fctp(w, x, y, meta2), ref)
    with pytest.raises(ValueError):
        fast_fctp(w, x, y[:-1], dict(meta, species_groups=meta2["species_groups"]))
