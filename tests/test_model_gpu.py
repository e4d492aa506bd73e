"""Energy and forces of the synthetic MACE-style model: GPU operators against the CPU oracle model."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-11), (torch.float32, 1e-5)])
def test_energy_and_forces_match_oracle(dtype, tol):
    from fasteq_b200.graph import make_boxes
    from fasteq_b200.nn.mace_style import MACEStyleModel
    from oracle import mace_style_ref
    torch.manual_seed(0)
    batch = make_boxes(2, [20, 14], [7.0, 6.5], 3.5, 3, seed=5)
    model = MACEStyleModel(num_species=3, channels=32, r_max=3.5, avg_num_neighbors=12.0).to(dtype)
    pos = torch.from_numpy(batch.positions).to(dtype)
    species = torch.from_numpy(batch.species)
    src, dst = torch.from_numpy(batch.edge_src), torch.from_numpy(batch.edge_dst)
    shift = torch.from_numpy(batch.edge_shift).to(dtype)
    graph = torch.from_numpy(batch.node_graph)
    e_ref, f_ref = mace_style_ref.energy_and_forces(model, pos, species, src, dst, shift)
    m = model.cuda()
    out = m(pos.cuda(), species.cuda(), src.cuda(), dst.cuda(), shift.cuda(), graph.cuda(), batch.n_graphs)
    from fasteq_b200.status import device_status
    assert device_status() == {}           # no kernel gave up on a wait or skipped an index
    e_graph = torch.zeros(batch.n_graphs, dtype=torch.float64).index_add(0, graph, e_ref)
    e_err = float((out["energy"].cpu().double() - e_graph).abs().max() / e_graph.abs().max())
    f = out["forces"].cpu().double()
    f_err = float((f - f_ref).abs().max() / f_ref.abs().max())
    assert e_err <= tol and f_err <= tol, (e_err, f_err)
    # total force on a periodic box vanishes (translation invariance)
    assert f.sum(0).abs().max() <= 50 * tol * f.abs().max()


def test_energy_and_forces_match_oracle_at_128_channels():
    """The benchmark model's width (128 channels: the four-pipeline packed tensor-product kernels, the tcgen05 3xTF32
    SO3Linear / radial GEMMs, the fused radial chain, in-kernel harmonics and fused edge geometry) on a small box,
    FP32, against the float64 CPU oracle model."""
    from fasteq_b200.graph import make_boxes
    from fasteq_b200.nn.mace_style import MACEStyleModel
    from oracle import mace_style_ref
    torch.manual_seed(0)
    batch = make_boxes(2, [40, 31], [8.0, 7.5], 4.0, 4, seed=9)
    model = MACEStyleModel(num_species=4, channels=128, r_max=4.0, avg_num_neighbors=20.0)
    pos = torch.from_numpy(batch.positions).float()
    species = torch.from_numpy(batch.species)
    src, dst = torch.from_numpy(batch.edge_src), torch.from_numpy(batch.edge_dst)
    shift = torch.from_numpy(batch.edge_shift).float()
    e_ref, f_ref = mace_style_ref.energy_and_forces(model, pos, species, src, dst, shift)
    m = model.cuda()
    out = m(pos.cuda(), species.cuda(), src.cuda(), dst.cuda(), shift.cuda())
    from fasteq_b200.status import device_status
    assert device_status() == {}
    e_err = float((out["energy"].cpu().double() - e_ref.sum()).abs() / e_ref.abs().sum())
    f = out["forces"].cpu().double()
    f_err = float((f - f_ref).abs().max() / f_ref.abs().max())
    print(f"128-channel model, FP32: energy error {e_err:.2e} (relative to sum |e_atom|), force error {f_err:.2e}")
    assert e_err <= 1e-5 and f_err <= 1e-5


def test_cuda_graph_replay_survives_plan_cache_eviction():
    """A captured step keeps reading its graph plan's CSR offsets and partitions.  The plan cache is a bounded LRU;
    after more other graphs than it holds, the captured plan has left it, and only the graph object's own
    references keep those buffers from being recycled."""
    from fasteq_b200.graph import make_boxes
    from fasteq_b200.nn.graphed import GraphedEnergyForces
    from fasteq_b200.nn.mace_style import MACEStyleModel
    from fasteq_b200.ops import uniform1d_jit as u1d
    torch.manual_seed(0)
    b = make_boxes(2, [20, 14], [7.0, 6.5], 3.5, 3, seed=5)
    model = MACEStyleModel(num_species=3, channels=32, r_max=3.5, avg_num_neighbors=12.0).cuda()
    for p in model.parameters():
        p.requires_grad_(False)
    t = lambda a, dt=None: torch.from_numpy(a).cuda() if dt is None else torch.from_numpy(a).to(dt).cuda()
    pos = t(b.positions, torch.float32)
    args = (t(b.species), t(b.edge_src), t(b.edge_dst), t(b.edge_shift, torch.float32), t(b.node_graph), b.n_graphs)
    graphed = GraphedEnergyForces(model, pos, *args)
    assert graphed._plans, "the capture must have recorded the plans it uses"
    held = {id(p) for p in graphed._plans}
    n = b.n_nodes
    for k in range(u1d._PLAN_LIMIT + 8):            # more throw-away graphs than the cache holds
        junk = torch.sort(torch.randint(0, n, (b.n_edges,), device="cuda")).values.int()
        u1d.graph_plan(junk, n).partition(37)
        del junk
    assert not any(id(p) in held for p in u1d._PLANS.values()), "the captured plan should have been evicted"
    # recycle whatever the allocator got back, with a pattern that would break the kernels
    trash = [torch.full((b.n_edges + 64,), 0x7fffffff, dtype=torch.int32, device="cuda") for _ in range(64)]
    p2 = pos + 0.01 * torch.randn(pos.shape, generator=torch.Generator().manual_seed(3)).cuda()
    out = graphed(p2)
    e, f = out["energy"].clone(), out["forces"].clone()
    ref = model(p2, *args)
    assert (e - ref["energy"]).abs().max() <= 1e-6 * ref["energy"].abs().max()
    assert (f - ref["forces"]).abs().max() <= 1e-5 * ref["forces"].abs().max()
    del trash


def test_cuda_graph_replay_matches_eager():
    """A captured energy + forces step replayed with new positions equals the eager evaluation."""
    from fasteq_b200.graph import make_boxes
    from fasteq_b200.nn.graphed import GraphedEnergyForces
    from fasteq_b200.nn.mace_style import MACEStyleModel
    torch.manual_seed(0)
    b = make_boxes(2, [20, 14], [7.0, 6.5], 3.5, 3, seed=5)
    model = MACEStyleModel(num_species=3, channels=32, r_max=3.5, avg_num_neighbors=12.0).cuda()
    for p in model.parameters():
        p.requires_grad_(False)
    t = lambda a, dt=None: torch.from_numpy(a).cuda() if dt is None else torch.from_numpy(a).to(dt).cuda()
    pos = t(b.positions, torch.float32)
    args = (t(b.species), t(b.edge_src), t(b.edge_dst), t(b.edge_shift, torch.float32), t(b.node_graph), b.n_graphs)
    graphed = GraphedEnergyForces(model, pos, *args)
    for k in range(2):
        # small displacement: the neighbour list stays valid, the values change
        p2 = pos + 0.01 * (k + 1) * torch.randn(pos.shape, generator=torch.Generator().manual_seed(k)).cuda()
        out = graphed(p2)
        e, f = out["energy"].clone(), out["forces"].clone()
        ref = model(p2, *args)
        assert (e - ref["energy"]).abs().max() <= 1e-6 * ref["energy"].abs().max()
        assert (f - ref["forces"]).abs().max() <= 1e-5 * ref["forces"].abs().max()


def test_force_loss_gradients_match_oracle():
    """Force-loss training: d/d(weights) of sum |F - F_target|^2 through the second-order paths of every operator
    (tensor product, symmetric contraction, SO3Linear, spherical harmonics, dense layers) against the CPU oracle."""
    from fasteq_b200.graph import make_boxes
    from fasteq_b200.nn.mace_style import MACEStyleModel
    from oracle import mace_style_ref
    torch.manual_seed(1)
    batch = make_boxes(2, [16, 12], [6.5, 6.0], 3.5, 3, seed=7)
    model = MACEStyleModel(num_species=3, channels=32, r_max=3.5, avg_num_neighbors=12.0).double()
    pos = torch.from_numpy(batch.positions)
    species = torch.from_numpy(batch.species)
    src, dst = torch.from_numpy(batch.edge_src), torch.from_numpy(batch.edge_dst)
    shift = torch.from_numpy(batch.edge_shift)
    target = torch.randn(pos.shape, generator=torch.Generator().manual_seed(3), dtype=torch.float64) * 0.1
    names = ["layers.0.linear_up.weight", "layers.0.radial.layers.1.weight", "layers.1.product.weight",
             "layers.1.linear_mid.weight", "readouts.1", "embedding"]
    loss_ref, g_ref = mace_style_ref.force_loss_gradients(model, pos, species, src, dst, shift, target, names)
    m = model.cuda()
    out = m(pos.cuda(), species.cuda(), src.cuda(), dst.cuda(), shift.cuda(), create_graph=True)
    loss = ((out["forces"] - target.cuda()) ** 2).sum()
    params = dict(m.named_parameters())
    grads = torch.autograd.grad(loss, [params[n] for n in names])
    assert abs(float(loss) - loss_ref) <= 1e-10 * abs(loss_ref)
    for n, g in zip(names, grads):
        ref = g_ref[n]
        err = float((g.cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
        assert err <= 1e-9, f"{n}: relative error {err:.3e}"
