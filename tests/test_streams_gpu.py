"""Operators on a side stream: every launch goes to torch's current stream, and cached state built on one
stream (prepared weight forms, graph plans) is ordered before its first use on another."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _model_inputs(dtype=torch.float32):
    from fasteq_b200.graph import make_boxes
    b = make_boxes(2, [20, 14], [7.0, 6.5], 3.5, 3, seed=5)
    t = lambda a, dt=None: torch.from_numpy(a).cuda() if dt is None else torch.from_numpy(a).to(dt).cuda()
    return t(b.positions, dtype), (t(b.species), t(b.edge_src), t(b.edge_dst), t(b.edge_shift, dtype), t(b.node_graph), b.n_graphs)


def _same(e, f, e_ref, f_ref):
    # the position gradient is accumulated with floating-point atomics, so forces agree to rounding, not bit for bit
    return bool((e - e_ref).abs().max() <= 1e-6 * e_ref.abs().max()) and bool((f - f_ref).abs().max() <= 1e-5 * f_ref.abs().max())


def test_model_on_a_side_stream_matches_the_default_stream():
    from fasteq_b200.nn.mace_style import MACEStyleModel
    from fasteq_b200.ops import _prepared
    torch.manual_seed(0)
    model = MACEStyleModel(num_species=3, channels=32, r_max=3.5, avg_num_neighbors=12.0).cuda()
    for p in model.parameters():
        p.requires_grad_(False)
    pos, args = _model_inputs()
    ref = model(pos, *args)
    e_ref, f_ref = ref["energy"].clone(), ref["forces"].clone()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    # (a) caches warm from the default stream, first use on the side stream
    with torch.cuda.stream(side):
        out = model(pos, *args)
        e1, f1 = out["energy"].clone(), out["forces"].clone()
    side.synchronize()
    assert _same(e1, f1, e_ref, f_ref)
    # (b) caches built on the side stream, next use on the default stream without a host sync in between
    _prepared.clear()
    from fasteq_b200.ops import uniform1d_jit
    uniform1d_jit._PLANS.clear()
    with torch.cuda.stream(side):
        out = model(pos, *args)
        e2, f2 = out["energy"].clone(), out["forces"].clone()
    out = model(pos, *args)
    e3, f3 = out["energy"].clone(), out["forces"].clone()
    torch.cuda.synchronize()
    assert _same(e2, f2, e_ref, f_ref)
    assert _same(e3, f3, e_ref, f_ref)


def test_operators_launch_on_the_current_stream():
    """A long kernel queued on the side stream first: an operator launched there afterwards must not have run
    ahead of it (it would if it went to the default stream), which shows in the value it reads."""
    from fasteq_b200.ops.dense import dense
    side = torch.cuda.Stream()
    x = torch.zeros(4096, 64, device="cuda")
    w = torch.eye(64, device="cuda")
    big = torch.randn(8192, 8192, device="cuda")
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        for _ in range(4):
            big = big @ big * 1e-4       # keeps the side stream busy
        x.fill_(3.0)                     # ordered behind the matmuls on the side stream
        y = dense(x, w)                  # must see the filled values
    side.synchronize()
    assert float(y.min()) == 3.0 and float(y.max()) == 3.0
