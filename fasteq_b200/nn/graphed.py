"""CUDA-graph replay of an energy + forces evaluation for a fixed neighbour list.

Between neighbour-list rebuilds a molecular-dynamics step evaluates the same graph with new
positions.  ``GraphedEnergyForces`` captures one evaluation (forward and the autograd force
backward, a few hundred kernel launches) into a CUDA graph and replays it, so the per-step host
cost is one copy of the positions and one graph launch instead of the Python / launch overhead of
every operator.  Capture needs the operator plans and generated modules to exist already, which the
warm-up evaluations ensure.  The model's weights are taken as frozen for the life of the graph: the
prepared (TF32-split) weight forms cached during the warm-up are captured as they are.  Collectives a ``halo=``
exchange makes (NCCL) are captured with the kernels; the capture uses the thread-local error mode so that the
process group's watchdog thread may keep polling its events meanwhile.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import _prepared
from ..ops import uniform1d_jit as _u1d


class GraphedEnergyForces:
    def __init__(self, model, pos: torch.Tensor, *static_args, warmup: int = 3, **static_kwargs):
        if not pos.is_cuda:
            raise RuntimeError("CUDA graphs need CUDA tensors")
        self.model = model
        self.static_pos = pos.detach().clone()
        self.args, self.kwargs = static_args, static_kwargs
        side = torch.cuda.Stream(device=pos.device)
        side.wait_stream(torch.cuda.current_stream(pos.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                model(self.static_pos, *static_args, **static_kwargs)
        torch.cuda.current_stream(pos.device).wait_stream(side)
        torch.cuda.synchronize(pos.device)
        self.graph = torch.cuda.CUDAGraph()
        with _prepared.frozen_weights(), _u1d.record_plans() as plans, torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            self.static_out = model(self.static_pos, *static_args, **static_kwargs)
        self._prepared = _prepared.snapshot()      # the captured kernels read these buffers
        # ... and the CSR offsets / permutations / partitions of these plans: the plan cache is a bounded LRU
        # and would hand their memory back to the allocator after enough other graphs
        self._plans = list(plans)

    def __call__(self, pos: torch.Tensor) -> Dict[str, torch.Tensor]:
        """Results live in static buffers that the next call overwrites; clone what must be kept."""
        self.static_pos.copy_(pos, non_blocking=True)
        self.graph.replay()
        return self.static_out
