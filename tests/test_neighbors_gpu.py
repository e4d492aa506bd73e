"""The GPU radius-graph builder against the host (numpy) builder: identical edge lists, bit for bit,
in the canonical (receiver, sender, image) order; CSR offsets; use as a ready graph plan."""
import numpy as np
import pytest
import torch

from fasteq_b200.graph import periodic_radius_graph

pytestmark = pytest.mark.gpu


def _host(positions, structs, boxes, cutoff):
    src, dst, sh, off = [], [], [], 0
    for s, box in enumerate(boxes):
        p = positions[structs == s]
        a, b, _, c = periodic_radius_graph(p, box, cutoff)
        src.append(a + off); dst.append(b + off); sh.append(c)
        off += p.shape[0]
    return np.concatenate(src), np.concatenate(dst), np.concatenate(sh)


def _case(boxes, counts, seed):
    rng = np.random.default_rng(seed)
    boxes = np.asarray(boxes, dtype=np.float64)
    if boxes.ndim == 1:
        boxes = np.repeat(boxes[:, None], 3, 1)
    pos = np.concatenate([rng.uniform(0.0, 1.0, size=(n, 3)) * b for n, b in zip(counts, boxes)])
    structs = np.concatenate([np.full(n, s) for s, n in enumerate(counts)])
    return pos, structs, boxes


@pytest.mark.parametrize("name,boxes,counts,cutoff", [
    ("config1_box", [12.4], [192], 5.0),                       # 2 cells per side: both neighbours of a cell are the same cell
    ("three_cells", [15.6], [384], 5.0),
    ("many_cells", [30.0], [1500], 4.0),
    ("one_cell", [7.0], [60], 5.0),                            # cutoff <= side < 2 cutoff: one cell, images -1, 0, +1
    ("smaller_than_cutoff", [4.0], [12], 5.0),                 # two images per side
    ("orthorhombic", [[9.0, 14.0, 21.5]], [300], 4.5),
    ("ragged_batch", [6.8, 9.3, 13.7, 11.0, 8.2], [32, 80, 256, 133, 57], 5.0),
    ("empty_structure_inside", [10.0, 10.0, 10.0], [40, 0, 25], 4.0),
])
def test_edges_identical_to_the_host_builder(name, boxes, counts, cutoff):
    from fasteq_b200.neighbors import radius_graph
    pos, structs, boxes = _case(boxes, counts, seed=len(name))
    src, dst, sh = _host(pos, structs, boxes, cutoff)
    g = radius_graph(torch.from_numpy(pos).cuda(), torch.from_numpy(structs).cuda(), boxes, cutoff, register_plan=False)
    assert g.edge_src.numel() == src.size
    assert np.array_equal(g.edge_dst.cpu().numpy(), dst)
    assert np.array_equal(g.edge_src.cpu().numpy(), src)
    assert np.array_equal(g.edge_shift.cpu().numpy(), sh)
    seg = np.searchsorted(dst, np.arange(pos.shape[0] + 1))
    assert np.array_equal(g.seg_ptr.cpu().numpy(), seg)
    assert g.max_degree == (np.diff(seg).max() if src.size else 0)


def test_no_atoms_and_no_edges():
    from fasteq_b200.neighbors import radius_graph
    g = radius_graph(torch.zeros(0, 3, dtype=torch.float64).cuda(), torch.zeros(0, dtype=torch.int32).cuda(), [10.0], 3.0)
    assert g.edge_src.numel() == 0 and g.seg_ptr.tolist() == [0]
    pos = torch.tensor([[1.0, 1.0, 1.0], [9.0, 9.0, 9.0]], dtype=torch.float64).cuda()
    g = radius_graph(pos, torch.zeros(2, dtype=torch.int32).cuda(), [20.0], 3.0)
    assert g.edge_src.numel() == 0 and g.seg_ptr.tolist() == [0, 0, 0]


def test_graph_feeds_the_tensor_product_without_a_plan_build():
    """The receiver index of the builder carries a registered plan: the operator result equals the one
    computed from a host-built copy of the same edges (which goes through check + CSR build)."""
    from fasteq_b200.descriptors import channelwise_tensor_product, full_channelwise_instructions
    from fasteq_b200.irreps import Irreps
    from fasteq_b200.neighbors import radius_graph
    from fasteq_b200.ops import fast_uniform1d_jit
    from fasteq_b200.ops import uniform1d_jit as u1d
    pos, structs, boxes = _case([12.4, 12.4], [192, 192], seed=3)
    g = radius_graph(torch.from_numpy(pos).cuda(), torch.from_numpy(structs).cuda(), boxes, 5.0)
    key_hit = any(k[0] == g.edge_dst.data_ptr() for k in u1d._PLANS)
    assert key_hit
    sh = Irreps.spherical_harmonics(2)
    io, ins = full_channelwise_instructions("32x0e+32x1o", sh, 2)
    d = channelwise_tensor_product("32x0e+32x1o", sh, io, ins)
    meta = d.meta(torch.float32, "cuda")
    E, N = g.edge_src.numel(), pos.shape[0]
    gen = torch.Generator().manual_seed(0)
    w = torch.randn(E, d.w_seg_num * 32, generator=gen).cuda()
    x = torch.randn(N, d.x_seg_num * 32, generator=gen).cuda()
    y = torch.randn(E, d.y_seg_num, generator=gen).cuda()
    out1 = fast_uniform1d_jit(w, x, y, {1: g.edge_src}, {0: g.edge_dst}, meta)
    out2 = fast_uniform1d_jit(w, x, y, {1: g.edge_src.clone()}, {0: g.edge_dst.clone()}, meta)
    assert torch.equal(out1, out2)
