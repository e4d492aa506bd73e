"""World-size-2 gloo run of the whole-structure split: every rank builds its own share, the summed
edge counts and a checksum of the per-structure work agree with the single-process result."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fasteq_b200.graph import make_boxes, split_structures
    atoms = [24, 40, 32, 48, 28, 36]
    ref = [make_boxes(1, a, 8.0, 4.0, 2, seed=100 + i) for i, a in enumerate(atoms)]
    edges = np.array([b.n_edges for b in ref])
    mine = split_structures(edges, world)[rank]
    local = torch.tensor([float(sum(edges[i] for i in mine)), float(sum(ref[i].edge_vec.sum() for i in mine))], dtype=torch.float64)
    dist.all_reduce(local, op=dist.ReduceOp.SUM)
    tmax = torch.tensor([float(len(mine))]); dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    if rank == 0:
        out.put((local.tolist(), float(edges.sum()), float(sum(b.edge_vec.sum() for b in ref)), tmax.item()))
    dist.destroy_process_group()


def test_whole_structure_split_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (tot_edges, checksum), ref_edges, ref_checksum, tmax = got
    assert tot_edges == ref_edges
    assert abs(checksum - ref_checksum) < 1e-9 * max(1.0, abs(ref_checksum))
    assert tmax == 3
