"""The MD-engine ghost-exchange hook on the GPU: the MACE-style model driven through ``EngineGhostExchange`` with CUDA
tensors and a stand-in engine that follows the LAMMPS ML-IAP protocol (``nlocal``, ``ntotal``, ``forward_exchange``,
``reverse_exchange``; …/nequip/nn/_ghost_exchange_lmp_mliap.py:11-64).  As in an MD engine's domain decomposition, every
sender that is reached through a periodic image becomes a ghost atom (a copy of its owner); the result must equal the
plain evaluation of the periodic graph."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


class _Engine:
    """Ghost row g is a copy of owned row owner[g]; gradients of ghost rows are summed onto their owners."""

    def __init__(self, nlocal, owner, device):
        self.nlocal, self.owner = nlocal, torch.as_tensor(owner, device=device)
        self.ntotal = nlocal + len(owner)
        self.calls = []

    def forward_exchange(self, src, dst, width):
        assert src.is_cuda and src.shape == dst.shape == (self.ntotal, width)
        dst.copy_(src)
        dst[self.nlocal:] = src[self.owner]
        self.calls.append("fwd")

    def reverse_exchange(self, grad, dst, width):
        assert grad.is_cuda and grad.shape == dst.shape == (self.ntotal, width)
        dst.copy_(grad)
        dst.index_add_(0, self.owner, grad[self.nlocal:])
        self.calls.append("rev")


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-10), (torch.float32, 1e-5)])
def test_model_through_engine_exchange_matches_periodic_graph(dtype, tol):
    from fasteq_b200.graph import make_boxes
    from fasteq_b200.nn.mace_style import MACEStyleModel
    from fasteq_b200.parallel import EngineGhostExchange
    torch.manual_seed(0)
    b = make_boxes(1, 60, 8.0, 3.5, 3, seed=4)
    model = MACEStyleModel(num_species=3, channels=32, r_max=3.5, avg_num_neighbors=12.0).to(dtype).cuda()
    for p in model.parameters():
        p.requires_grad_(False)
    n = b.n_nodes
    # ghost atoms: one per distinct (sender, image) pair with a non-zero image shift
    key = {}
    src_local = b.edge_src.copy()
    for e in np.nonzero(np.abs(b.edge_shift).sum(1) > 0)[0]:
        k = (int(b.edge_src[e]),) + tuple(np.round(b.edge_shift[e], 6))
        src_local[e] = key.setdefault(k, n + len(key))
    owner = [k[0] for k in key]
    assert len(owner) > 20
    eng = _Engine(n, owner, "cuda")
    t = lambda a, dt=None: torch.from_numpy(a).cuda() if dt is None else torch.from_numpy(a).to(dt).cuda()
    pos, spec, shift = t(b.positions, dtype), t(b.species), t(b.edge_shift, dtype)
    ref = model(pos, spec, t(b.edge_src), t(b.edge_dst), shift)
    out = model(pos, spec, t(src_local), t(b.edge_dst), shift, halo=EngineGhostExchange(eng))
    # forward: the positions and one exchange per layer; reverse: the same minus the first layer's features, which do
    # not depend on the positions and so receive no gradient
    assert eng.calls.count("fwd") == 1 + len(model.layers) and eng.calls.count("rev") == len(model.layers)
    assert (out["energy"] - ref["energy"]).abs().max() <= tol * ref["energy"].abs().max()
    assert (out["forces"] - ref["forces"]).abs().max() <= tol * ref["forces"].abs().max()
