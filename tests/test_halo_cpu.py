"""Receiver-range partition + halo exchange on CPU ranks (gloo, world size 2 and 3): energies and
forces of a small differentiable message-passing stand-in must equal the single-process result."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _toy_energy(pos_owned, feat_owned, src, dst, shift, w1, w2, halo, n_layers=2, split=False):
    """Two rounds of h_i <- tanh(W h_i) + sum_j exp(-|r_ij|) * (W h_j); E_i = sum(h_i^2)."""
    pos_ext = halo(pos_owned) if halo is not None else pos_owned
    vec = pos_ext[src] + shift - pos_ext[dst]
    r = vec.norm(dim=-1, keepdim=True)
    h = feat_owned
    n = pos_owned.shape[0]
    for w in (w1, w2)[:n_layers]:
        up = h @ w
        if halo is not None and split:       # node-local work between begin and end
            t = halo.begin(up)
            _ = torch.tanh(up)
            ext = halo.end(t)
        else:
            ext = halo(up) if halo is not None else up
        msg = torch.zeros(n, up.shape[1], dtype=up.dtype).index_add(0, dst, torch.exp(-r) * ext[src])
        h = torch.tanh(up) + msg
    return (h * h).sum(dim=1)


def _problem():
    sys.path.insert(0, ROOT)
    from fasteq_b200.graph import make_boxes
    b = make_boxes(1, 60, 9.0, 3.5, 2, seed=7)
    g = torch.Generator().manual_seed(1)
    feat = torch.randn(b.n_nodes, 5, generator=g, dtype=torch.float64)
    w1 = torch.randn(5, 5, generator=g, dtype=torch.float64) * 0.4
    w2 = torch.randn(5, 5, generator=g, dtype=torch.float64) * 0.4
    return b, feat, w1, w2


def _worker(rank, world, port, q, mode="alltoall"):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fasteq_b200.parallel import HaloExchange, partition_by_receiver_range
    b, feat, w1, w2 = _problem()
    parts = partition_by_receiver_range(b.n_nodes, b.edge_src, b.edge_dst, world)
    lg = parts[rank]
    halo = HaloExchange(lg, "cpu", mode={"gather": "gather", "auto": "auto"}.get(mode, "alltoall"))
    pos = torch.from_numpy(b.positions[lg.start:lg.stop]).requires_grad_(True)
    shift = torch.from_numpy(b.edge_shift[lg.edge_ids])
    e = _toy_energy(pos, feat[lg.start:lg.stop], torch.from_numpy(lg.edge_src), torch.from_numpy(lg.edge_dst), shift, w1, w2, halo,
                    split=mode == "split")
    (g,) = torch.autograd.grad(e.sum(), pos)
    q.put((rank, lg.start, lg.stop, e.detach().numpy(), g.numpy(), len(lg.ghost_global), int(len(lg.edge_ids))))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,mode", [(2, "alltoall"), (3, "alltoall"), (3, "split"), (2, "gather"), (2, "auto")])
def test_partitioned_energy_and_forces_match_single_process(world, mode):
    b, feat, w1, w2 = _problem()
    pos = torch.from_numpy(b.positions).requires_grad_(True)
    e_ref = _toy_energy(pos, feat, torch.from_numpy(b.edge_src), torch.from_numpy(b.edge_dst), torch.from_numpy(b.edge_shift), w1, w2, None)
    (g_ref,) = torch.autograd.grad(e_ref.sum(), pos)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    e = np.zeros(b.n_nodes); g = np.zeros((b.n_nodes, 3)); edges = 0
    for rank, lo, hi, er, gr, n_ghost, n_edges in got:
        e[lo:hi] = er; g[lo:hi] = gr; edges += n_edges
        assert n_ghost > 0
    assert edges == b.n_edges                       # every edge has exactly one owner
    np.testing.assert_allclose(e, e_ref.detach().numpy(), rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(g, g_ref.numpy(), rtol=1e-10, atol=1e-12)


def test_partition_tables_are_consistent():
    sys.path.insert(0, ROOT)
    from fasteq_b200.parallel import node_ranges, partition_by_receiver_range
    b, *_ = _problem()
    parts = partition_by_receiver_range(b.n_nodes, b.edge_src, b.edge_dst, 4)
    bounds = node_ranges(b.n_nodes, 4, b.edge_dst)
    assert bounds[0] == 0 and bounds[-1] == b.n_nodes and all(a <= c for a, c in zip(bounds, bounds[1:]))
    counts = [len(p.edge_ids) for p in parts]
    assert sum(counts) == b.n_edges and max(counts) < 1.5 * b.n_edges / 4
    for p in parts:
        assert (np.diff(p.edge_dst) >= 0).all() and p.edge_dst.max() < p.n_owned
        assert p.edge_src.max() < p.n_local
        # per-peer tables of the neighbour-only exchange: what r sends q is what q expects from r, nothing to itself,
        # and the rows q receives, taken in rank order, are its ghosts in order
        assert p.send_counts[p.rank] == 0 and p.recv_counts[p.rank] == 0
        assert sum(p.recv_counts) == len(p.ghost_global) and sum(p.send_counts) == len(p.send_idx)
        for q in parts:
            assert p.send_counts[q.rank] == q.recv_counts[p.rank]
        got = np.concatenate([q.start + q.send_idx[sum(q.send_counts[:p.rank]):sum(q.send_counts[:p.rank + 1])] for q in parts])
        assert (got == p.ghost_global).all()
        # a ghost's slot points into its owner's slab
        for g, slot in zip(p.ghost_global, p.ghost_slot):
            owner = slot // p.max_export
            assert parts[owner].start <= g < parts[owner].stop
            assert parts[owner].export_local[slot % p.max_export] + parts[owner].start == g


class _FakeEngine:
    """Stands in for an MD engine's ghost communication: ghost row g is a copy of owned row owner[g]."""

    def __init__(self, nlocal, owner):
        self.nlocal, self.owner = nlocal, torch.as_tensor(owner)
        self.ntotal = nlocal + len(owner)
        self.calls = []

    def forward_exchange(self, src, dst, width):
        assert src.shape == dst.shape == (self.ntotal, width)
        dst.copy_(src)
        dst[self.nlocal:] = src[self.owner]
        self.calls.append("fwd")

    def reverse_exchange(self, grad, dst, width):
        assert grad.shape == dst.shape == (self.ntotal, width)
        dst.copy_(grad)
        dst.index_add_(0, self.owner, grad[self.nlocal:])
        self.calls.append("rev")


def test_engine_ghost_exchange_matches_plain_indexing():
    from fasteq_b200.parallel import EngineGhostExchange
    torch.manual_seed(0)
    nlocal, owner = 7, [2, 2, 5, 0]
    eng = _FakeEngine(nlocal, owner)
    halo = EngineGhostExchange(eng)
    x = torch.randn(nlocal, 3, 4, dtype=torch.float64, requires_grad=True)
    ext = halo(x)
    ref = torch.cat([x, x[torch.tensor(owner)]], 0)
    assert ext.shape == (11, 3, 4) and torch.equal(ext, ref)
    r = torch.randn_like(ext)
    (g,) = torch.autograd.grad(ext, x, r)
    (g_ref,) = torch.autograd.grad(ref, x, r)
    assert torch.allclose(g, g_ref, atol=1e-14, rtol=0) and eng.calls == ["fwd", "rev"]
    # no ghosts: the owned tensor passes through untouched
    assert EngineGhostExchange(_FakeEngine(nlocal, [])) (x) is x
