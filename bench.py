#!/usr/bin/env python
"""Benchmark of the ChannelwiseTensorProduct hot path (forward + force backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one forward + one backward (grad_w, grad_x, grad_y) of the fused
gather / tensor-product / scatter operator over one synthetic batch.  Default
workload: the interaction of benchmark configuration 1 -- 64 periodic boxes x 192 atoms
(cutoff 5 A, ~52 neighbours), hidden 128x0e+128x1o (x) SH l<=3 -> all paths l<=3,
FP32, per-edge weights materialised.  With N > 1 every rank processes its own
batch of whole structures (no data-path collective): weak scaling.

Prints ONE JSON line (rank 0).  ``value`` is edges/s with inputs resident in HBM,
``e2e`` the same through the public operator with pinned-host inputs copied in
and a scalar result copied out every step, ``roofline`` the dominant kernel's
algorithmic bytes / CUDA-event time against the measured copy bandwidth,
``cpu_baseline`` the CPU oracle (e3nn algorithm, torch CPU, all host threads)
on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np
import torch

WORKLOADS = {
    # name: (irreps_in1, SH lmax, lmax_out, boxes per GPU, dtype)
    "config1_cwtp": ("128x0e+128x1o", 3, 3, 64, torch.float32),
    "config0_layout_cwtp": ("128x0e+128x1o+128x2e", 3, 3, 64, torch.float32),
    # the interaction of configuration 3's NequIP-style layers (64 channels, six irreps, SH l <= 2: 30 weight / 102 output segments)
    "config3_layer_cwtp": ("64x0e+64x0o+64x1e+64x1o+64x2e+64x2o", 2, 2, 64, torch.float32),
}
METRIC = "ChannelwiseTP edges/s (fwd+force bwd)"
CPU_NOTE = ("port of e3nn's uvu TensorProduct + scatter (oracle/e3nn_uvu_ref.py, pinned to e3nn 0.5.6 golden vectors at 1e-12), "
            "torch CPU kernels, no einsum-order optimisation (e3nn's opt_einsum_fx pass is not applied)")
# DRAM bytes (dram__bytes_read + dram__bytes_write) over algorithmic bytes, from one ncu capture per kernel
# on a 16-box case of the same workload; traffic grows in proportion to the edge count (every term
# is per edge or per node and the generator fixes edges per node), so the ratio carries to a full launch.
TRAFFIC_RATIO = {"config1_cwtp": {"fwd": 1.009, "bwd": 1.040}, "config0_layout_cwtp": {"fwd": 1.063, "bwd": 1.131},
                 "config3_layer_cwtp": {"fwd": 1.039, "bwd": 1.134}}


def algorithmic_bytes(N, E, d, s):
    """Each logical tensor once (unique node rows, per-edge tensors, outputs, indices)."""
    U = d.u_dim
    fwd = s * (N * d.x_seg_num * U + E * d.w_seg_num * U + E * d.y_seg_num + N * d.out_seg_num * U) + 8 * E
    bwd = s * (2 * E * d.w_seg_num * U + 2 * N * d.x_seg_num * U + 2 * E * d.y_seg_num + N * d.out_seg_num * U) + 8 * E
    return fwd, bwd


def fp32_floor(spec, tun, direction, needs, E, U, launch_s, dev, sm_mhz=None, lanes=128, tag="fp32"):
    """Arithmetic-pipe view of a CWTP kernel: arithmetic instructions per (edge, channel) counted in the generated source,
    the time they need at ``lanes`` per SM per clock (128 for FP32, 64 for FP64), and the share of that rate the launch
    reached."""
    from fasteq_b200.codegen import u1d as gen
    ops = gen.arith_ops(spec, tun, direction, needs)
    n = ops["fma"] + ops["mul"] + ops["add"]
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    if sm_mhz is None:
        try:
            sm_mhz = float(torch.cuda.clock_rate())
        except Exception:
            sm_mhz = 1965.0
    floor_s = float(E) * U * n / (sms * lanes * sm_mhz * 1e6)
    return {f"{tag}_ops_per_edge_channel": n, "fma": ops["fma"], "mul": ops["mul"], f"{tag}_floor_ms": floor_s * 1e3,
            f"{tag}_pipe_utilisation": floor_s / launch_s, "sm_mhz": sm_mhz}


def _go_home(tun):
    """Where a backward layout keeps the receiver's grad_out row."""
    return "shared memory" if tun.go_smem else ("tensor memory" if tun.go_tmem else "global memory through L1")


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, pw, reasons = [], [], [], set()
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            try:
                pw.append(float(f[2]))
            except ValueError:
                pass
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_min_mhz": float(min(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": (float(max(pw)) if pw else None)}


def build_inputs(workload: str, seed: int, n_boxes=None):
    from fasteq_b200.descriptors import channelwise_tensor_product, full_channelwise_instructions
    from fasteq_b200.graph import config1_batch
    from fasteq_b200.irreps import Irreps
    in1, lsh, lout, boxes, dtype = WORKLOADS[workload]
    sh = Irreps.spherical_harmonics(lsh)
    io, ins = full_channelwise_instructions(in1, sh, lout)
    d = channelwise_tensor_product(in1, sh, io, ins)
    batch = config1_batch(n_boxes or boxes, seed=seed)
    g = torch.Generator().manual_seed(seed)
    N, E, U = batch.n_nodes, batch.n_edges, d.u_dim
    vec = torch.from_numpy(batch.edge_vec)
    return dict(d=d, ins=ins, irreps=(in1, str(sh), str(io)), batch=batch, N=N, E=E, dtype=dtype, vec=vec, n_boxes=n_boxes or boxes,
                x=torch.randn(N, d.x_seg_num * U, generator=g, dtype=dtype),
                w=torch.randn(E, d.w_seg_num * U, generator=g, dtype=dtype),
                r=torch.randn(N, d.out_seg_num * U, generator=g, dtype=dtype),
                src=torch.from_numpy(batch.edge_src).int(), dst=torch.from_numpy(batch.edge_dst).int())


def cpu_reference_run(inp, steps: int, warmup: int, threads: int):
    """e3nn-algorithm CPU oracle: scatter(tp(x[src], sh, w), dst) forward + autograd backward (mul_ir layout)."""
    from fasteq_b200.irreps import Irreps, ir_mul_to_mul_ir
    from oracle import e3nn_uvu_ref, sh_ref
    torch.set_num_threads(threads)
    d = inp["d"]
    in1, in2, io = inp["irreps"]
    dt = inp["dtype"]
    tp = e3nn_uvu_ref.TensorProductUVU(in1, in2, io, inp["ins"], dtype=dt)
    x = ir_mul_to_mul_ir(inp["x"], Irreps(in1)).requires_grad_(True)
    y = sh_ref.spherical_harmonics(Irreps(in2).lmax, inp["vec"].to(dt), normalize=True).requires_grad_(True)
    w = inp["w"].clone().requires_grad_(True)
    r = ir_mul_to_mul_ir(inp["r"], Irreps(io))
    src, dst = inp["src"].long(), inp["dst"].long()
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        out = e3nn_uvu_ref.tp_scatter(tp, x, y, w, dst, src, inp["N"])
        torch.autograd.grad((out * r).sum(), (w, x, y))
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return inp["E"] * len(times) / sum(times), float(np.mean(times))


def model_inputs(n_boxes: int, seed: int, dtype, device):
    from fasteq_b200.graph import config1_batch
    b = config1_batch(n_boxes, seed=seed)
    t = lambda a, dt=None: torch.from_numpy(a).to(dt) if dt is not None else torch.from_numpy(a)
    host = dict(pos=t(b.positions, dtype), species=t(b.species), src=t(b.edge_src), dst=t(b.edge_dst), shift=t(b.edge_shift, dtype),
                graph=t(b.node_graph))
    return b, {k: v.to(device) for k, v in host.items()}


def halo_model_bench(args, dev, rank, world, dist):
    """benchmark configuration 3: NequIP-style network (64 x {0e,0o,1e,1o,2e,2o}, SH l <= 2, 4 gated interaction
    layers, FP32) on one periodic cube of 20,000 atoms (cutoff 4 A), partitioned by receiver range
    with a halo exchange per layer: strong scaling."""
    from fasteq_b200.graph import large_box
    from fasteq_b200.nn.nequip_style import NequIPStyleModel
    from fasteq_b200.parallel import HaloExchange, partition_by_receiver_range
    torch.manual_seed(0)
    model = NequIPStyleModel(num_species=2, channels=64, lmax=2, sh_lmax=2, num_layers=4, r_max=4.0, avg_num_neighbors=27.0).to(dev)
    for prm in model.parameters():
        prm.requires_grad_(False)
    b = large_box(seed=0)
    lg = partition_by_receiver_range(b.n_nodes, b.edge_src, b.edge_dst, world)[rank]
    halo = HaloExchange(lg, dev) if world > 1 else None
    t = lambda a, dt=None: torch.from_numpy(a).to(dev) if dt is None else torch.from_numpy(a).to(dt).to(dev)
    pos, spec = t(b.positions[lg.start:lg.stop], torch.float32), t(b.species[lg.start:lg.stop])
    src, dst, shift = t(lg.edge_src), t(lg.edge_dst), t(b.edge_shift[lg.edge_ids], torch.float32)
    run = lambda: model(pos, spec, src, dst, shift, halo=halo)
    for _ in range(3):
        out = run()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    k = max(3, min(args.steps, 10))
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(k):
        out = run()
    ev1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
    # the same graph, model seed and weights at every world size: the summed energy and the force checksums
    # must agree between N = 1 and N = 8 to FP32 round-off
    def checksums(o):
        f64 = o["forces"].detach().double()
        c = torch.stack([o["energy"].detach().double().sum(), (f64 * f64).sum(), f64.abs().sum()])
        if dist is not None:
            dist.all_reduce(c, op=dist.ReduceOp.SUM)
        return {"energy": float(c[0]), "force_l2": float(c[1].sqrt()), "force_l1": float(c[2])}
    chk = checksums(out)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    # the same step replayed from a CUDA graph (fixed neighbour list and partition, the halo collectives captured with the
    # kernels): at 2,500 atoms per rank the eager step is bound by the host's launch rate, the replay is not
    replay = None
    try:
        from fasteq_b200.nn.graphed import GraphedEnergyForces
        ge = GraphedEnergyForces(model, pos, spec, src, dst, shift, halo=halo)
        ok, why = 1, ""
    except Exception as exc:
        ok, why = 0, f"{type(exc).__name__}: {str(exc)[:200]}"
    okt = torch.tensor([ok], device=dev)
    if dist is not None:
        dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    if int(okt[0]) == 1:
        ge(pos); torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        ev0.record()
        for _ in range(k):
            o2 = ge(pos)
        ev1.record(); torch.cuda.synchronize()
        msr = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(msr, op=dist.ReduceOp.MAX)
        replay = dict(checksums(o2), ms_per_step=float(msr[0]) / k, value=b.n_nodes * k / (float(msr[0]) * 1e-3), unit="atom-steps/s")
    else:
        replay = {"failed": why or "capture failed on another rank"}
    breakdown = None
    if getattr(args, "breakdown", False):
        # rank 0's device time of an eager step by kernel family (every rank profiles, so that all stay in step)
        from torch.profiler import ProfilerActivity, profile
        n_prof = 5
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(n_prof):
                run()
            torch.cuda.synchronize()
        fam = {"tensor product (fasteq_u1d_*)": 0.0, "NCCL": 0.0, "tcgen05 GEMMs + radial chain": 0.0, "gate": 0.0, "edge geometry": 0.0,
               "framework kernels (pack / unpack, adds, fills, reductions)": 0.0}
        launches = 0
        for e in prof.key_averages():
            if e.device_type.name != "CUDA" or e.device_time_total <= 0:
                continue
            name, t_us = e.key, e.device_time_total / n_prof
            launches += e.count
            key = ("tensor product (fasteq_u1d_*)" if "fasteq_u1d" in name else "NCCL" if "nccl" in name.lower() else
                   "tcgen05 GEMMs + radial chain" if ("gemm_tf32x3" in name or "radial_chain" in name or "eqlinear" in name or "pack_weights" in name) else
                   "gate" if "gate" in name else "edge geometry" if "edge_geometry" in name else
                   "framework kernels (pack / unpack, adds, fills, reductions)")
            fam[key] += t_us
        breakdown = {"device_us_per_step": {k_: round(v, 1) for k_, v in fam.items()}, "device_us_total": round(sum(fam.values()), 1),
                     "launches_per_step": launches / n_prof, "rank": rank, "note": "eager step, torch profiler (CUPTI kernel records)"}
    eager_ms = float(ms[0]) / k
    # the block's figure: the replayed step where the capture succeeded and reproduces the eager checksums (a molecular-dynamics
    # run replays between neighbour-list rebuilds), else the eager step; both are printed
    replay_ok = "ms_per_step" in replay and abs(replay["energy"] - chk["energy"]) <= 1e-5 * abs(chk["energy"]) \
        and abs(replay["force_l2"] - chk["force_l2"]) <= 1e-5 * chk["force_l2"]
    best_ms = min(eager_ms, replay["ms_per_step"]) if replay_ok else eager_ms
    return {"metric": "NequIP-style atom-steps/s, one 20,000-atom graph, receiver-range partition + halo", "scaling": "strong",
            "value": b.n_nodes / (best_ms * 1e-3), "unit": "atom-steps/s", "ms_per_step": best_ms,
            "mode": "cuda_graph_replay" if (replay_ok and replay["ms_per_step"] < eager_ms) else "eager",
            "breakdown": breakdown, "eager_ms_per_step": eager_ms, "eager_exchange": "all-gather of padded export slabs (least host work)" if world > 1 else None,
            "energy": chk["energy"], "force_l2": chk["force_l2"], "force_l1": chk["force_l1"], "cuda_graph_replay": replay,
            "replay_exchange": ("per layer one variable-size all-to-all to the ranks that read this rank's rows (forward) and back "
                                "(force pass), captured with the kernels") if world > 1 else None,
            "atoms": b.n_nodes, "edges": b.n_edges, "owned": lg.n_owned, "ghosts": int(len(lg.ghost_global)),
            "config": "config 3: 4 gated layers, 64x0e+64x0o+64x1e+64x1o+64x2e+64x2o, SH l<=2, cutoff 4 A, FP32"}


def model_bench(args, dev, rank, dist, n_boxes: int, quick: bool = False):
    """Energy + forces of the synthetic MACE-style model of benchmark configuration 1 (FP32): atom-steps/s.
    ``quick``: the eager steps only (no graph replay, no end-to-end legs), for profiling."""
    from fasteq_b200.nn.mace_style import MACEStyleModel
    torch.manual_seed(0)
    model = MACEStyleModel().to(dev)
    for prm in model.parameters():          # inference + forces: no weight gradients
        prm.requires_grad_(False)
    b, d = model_inputs(n_boxes, rank, torch.float32, dev)
    run = lambda: model(d["pos"], d["species"], d["src"], d["dst"], d["shift"], d["graph"], b.n_graphs)
    for _ in range(3):
        out = run()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    k = max(3, min(args.steps, 10))
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(k):
        out = run()
    ev1.record()
    torch.cuda.synchronize()
    t = torch.tensor([ev0.elapsed_time(ev1), float(b.n_nodes)], dtype=torch.float64, device=dev)
    ms, atoms = float(t[0]), float(t[1])
    if dist is not None:
        tm = t.clone(); dist.all_reduce(tm, op=dist.ReduceOp.MAX); ms = float(tm[0])
        ts = t.clone(); dist.all_reduce(ts, op=dist.ReduceOp.SUM); atoms = float(ts[1])
    if quick:
        return {"metric": "MACE atom-steps/s (energy + forces)", "value": atoms * k / (ms * 1e-3), "unit": "atom-steps/s",
                "ms_per_step": ms / k, "steps": k, "atoms": int(atoms), "edges_per_gpu": b.n_edges}
    # the same evaluation replayed from a CUDA graph (fixed neighbour list, new positions each step)
    graphed_ms = None
    try:
        from fasteq_b200.nn.graphed import GraphedEnergyForces
        ge = GraphedEnergyForces(model, d["pos"], d["species"], d["src"], d["dst"], d["shift"], d["graph"], b.n_graphs)
        ge(d["pos"]); torch.cuda.synchronize()
        ev0.record()
        for _ in range(k):
            ge(d["pos"])
        ev1.record(); torch.cuda.synchronize()
        tg = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        graphed_ms = float(tg[0]) / k
    except Exception as exc:   # report, never fail the benchmark over the optional replay path
        graphed_ms = f"capture failed: {type(exc).__name__}: {str(exc)[:120]}"
    # end to end through the model call: pinned host positions / species / edge lists in, energies and forces out
    hb = model_inputs(n_boxes, rank, torch.float32, "cpu")[1]
    hp = {kk: v.pin_memory() for kk, v in hb.items()}
    def e2e_step():
        dd = {kk: v.to(dev, non_blocking=True) for kk, v in hp.items()}
        o = model(dd["pos"], dd["species"], dd["src"], dd["dst"], dd["shift"], dd["graph"], b.n_graphs)
        return o["energy"].cpu(), o["forces"].cpu()
    for _ in range(3):
        e2e_step()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(k):
        en, fo = e2e_step()
    torch.cuda.synchronize()
    te = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    h2d = sum(v.numel() * v.element_size() for v in hp.values())
    e2e_host_graph = {"value": atoms * k / float(te[0]), "unit": "atom-steps/s", "h2d_bytes_per_step": h2d,
                      "d2h_bytes_per_step": int(en.numel() * 4 + fo.numel() * 4),
                      "note": "edge lists built on the host beforehand and copied in with the positions every step"}
    # the same call with the neighbour list built on the GPU every step: positions / species in, energies / forces out
    from fasteq_b200.neighbors import radius_graph
    pos64 = torch.from_numpy(b.positions).pin_memory()
    boxes = np.full((b.n_graphs, 3), 12.4)
    def e2e_gpu_graph_step():
        p64 = pos64.to(dev, non_blocking=True)
        sp, gr = hp["species"].to(dev, non_blocking=True), hp["graph"].to(dev, non_blocking=True)
        g = radius_graph(p64, gr, boxes, 5.0)
        o = model(p64.to(torch.float32), sp, g.edge_src, g.edge_dst, g.edge_shift.to(torch.float32), gr, b.n_graphs)
        return o["energy"].cpu(), o["forces"].cpu()
    for _ in range(3):
        en2, fo2 = e2e_gpu_graph_step()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(k):
        en2, fo2 = e2e_gpu_graph_step()
    torch.cuda.synchronize()
    te2 = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(te2, op=dist.ReduceOp.MAX)
    e2e = {"value": atoms * k / float(te2[0]), "unit": "atom-steps/s",
           "h2d_bytes_per_step": int(pos64.numel() * 8 + hp["species"].numel() * hp["species"].element_size()
                                     + hp["graph"].numel() * hp["graph"].element_size()),
           "d2h_bytes_per_step": int(en2.numel() * 4 + fo2.numel() * 4 + 8),
           "note": "pinned host positions / species in, periodic radius graph rebuilt on the GPU every step, energies and forces out",
           "max_force_difference_to_host_graph": float((fo2 - fo).abs().max())}
    return {"metric": "MACE atom-steps/s (energy + forces)", "value": atoms * k / (ms * 1e-3), "unit": "atom-steps/s", "e2e": e2e, "e2e_host_graph": e2e_host_graph,
            "cuda_graph_replay": ({"ms_per_step": graphed_ms, "value": atoms / (graphed_ms * 1e-3), "unit": "atom-steps/s"}
                                  if isinstance(graphed_ms, float) else graphed_ms),
            "ms_per_step": ms / k, "steps": k, "atoms": int(atoms), "edges_per_gpu": b.n_edges,
            "config": "config 1: 2 layers, 128x0e+128x1o, SH l<=3, correlation 3, 8 Bessel x p=5 envelope, 64-64-64 SiLU radial MLP, FP32",
            "energy_finite": bool(torch.isfinite(out["energy"]).all()), "forces_finite": bool(torch.isfinite(out["forces"]).all())}


def operator_extras(args, dev):
    """Standalone timings of the other two operators of the path (benchmark configuration 4 asks for the
    SymmetricContraction on 200k nodes; SO3Linear at config 1's node count)."""
    from fasteq_b200.descriptors import linear, symmetric_contraction
    from fasteq_b200.ops import fast_equi_linear, fast_stc_uniform1d_jit
    g = torch.Generator().manual_seed(0)
    out = {}

    def timed(fn, k=10):
        fn(); fn(); torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(k):
            fn()
        b.record(); torch.cuda.synchronize()
        return a.elapsed_time(b) / k * 1e-3

    # SymmetricContraction, correlation 3, 128 channels, 10 species, 200k nodes
    d = symmetric_contraction("128x0e+128x1o+128x2e+128x3o", "128x0e+128x1o")
    B, U = 200000, d.u_dim
    x1 = (torch.randn(B, d.x1_segs, U, generator=g) * 0.3).to(dev).requires_grad_(True)
    x0 = (torch.randn(10, d.x0_segs, U, generator=g) * 0.1).to(dev)
    i0 = torch.randint(0, 10, (B,), generator=g).to(dev)
    r = torch.randn(B, d.out_segs * U, generator=g).to(dev)
    coeffs, paths, idx = d.tensors(torch.float32, dev)
    with torch.no_grad():
        t_f = timed(lambda: fast_stc_uniform1d_jit(x1, x0, i0, coeffs, paths, idx, d.out_segs))
    def fb():
        o = fast_stc_uniform1d_jit(x1, x0, i0, coeffs, paths, idx, d.out_segs)
        torch.autograd.grad(o, x1, r)
    t_fb = timed(fb)
    byts = 4.0 * (B * d.x1_segs * U + B * d.out_segs * U + 10 * d.x0_segs * U) + 4 * B
    # executed arithmetic: FMA / multiply instructions per (node, channel) thread, counted in the generated kernel source
    from fasteq_b200.codegen import stc as stc_gen
    from fasteq_b200.prebuild import stc_spec
    ops = stc_gen.arith_ops(stc_spec("128x0e+128x1o+128x2e+128x3o", "128x0e+128x1o", "f32"), "fwd")
    sm = torch.cuda.get_device_properties(dev).multi_processor_count
    try:
        clk_hz = float(torch.cuda.clock_rate()) * 1e6      # current SM clock (MHz, through NVML)
    except Exception:
        clk_hz = 1.965e9                                   # the part's maximum SM clock
    issue_peak = sm * 128 * clk_hz                           # FP32 lanes x clock: one FMA or multiply per lane per cycle
    with torch.no_grad():
        t_f_dev = _graph_replay_ms(lambda: fast_stc_uniform1d_jit(x1, x0, i0, coeffs, paths, idx, d.out_segs), k=5) * 1e-3
    out["stc_200k"] = {"nodes": B, "paths": d.num_paths, "fwd_ms": t_f * 1e3, "fwd_ms_device": t_f_dev * 1e3, "fwd_bwd_ms": t_fb * 1e3,
                       "nodes_per_s_fwd": B / t_f, "fwd_hbm_gbs": byts / t_f / 1e9,
                       "bound": "fp32 issue", "fma_per_thread": ops["fma"], "mul_per_thread": ops["mul"],
                       "fp32_issue_utilisation": float(B) * U * (ops["fma"] + ops["mul"]) / t_f_dev / issue_peak,
                       "issue_peak_note": f"{sm} SMs x 128 lanes x {clk_hz / 1e6:.0f} MHz (clock as sampled when the block ran)"}
    # SO3Linear after the tensor product of config 1: 55 -> 16 rows, 128 channels, 12,288 nodes
    from fasteq_b200.descriptors import full_channelwise_instructions
    from fasteq_b200.irreps import Irreps
    irr_tp, _ = full_channelwise_instructions("128x0e+128x1o", Irreps.spherical_harmonics(3), 3)
    dl = linear(irr_tp, "128x0e+128x1o+128x2e+128x3o")
    N = 12288
    x = torch.randn(N, irr_tp.dim, generator=g).to(dev).requires_grad_(True)
    w = torch.randn(dl.num_weights, generator=g).to(dev)
    ro = torch.randn(N, 16 * 128, generator=g).to(dev)
    with torch.no_grad():
        t_l = timed(lambda: fast_equi_linear(dl, w, x))
    def lb():
        o = fast_equi_linear(dl, w, x)
        torch.autograd.grad(o, x, ro)
    t_lb = timed(lb)
    # the two launches alone, replayed from a CUDA graph (no host work per launch): kernel time of the forward and of grad_x
    from fasteq_b200.ops import eqlinear as eql
    geom = eql._descriptor_problem(dl)
    plan = eql._Plan(geom, eql._resolve_precision(x, w, None), N, w.shape)
    xd = x.detach()
    t_fk = _graph_replay_ms(lambda: plan.forward(w, xd)) * 1e-3
    t_dk = _graph_replay_ms(lambda: plan.dgrad(w, ro)) * 1e-3
    rows = sum(p_rows for p_rows in [irr_tp[p.indices[1]].ir.dim for p in dl.paths])
    lbytes = 4.0 * (N * irr_tp.dim + N * 16 * 128 + dl.num_weights)
    peak, _ = measured_peak()
    out["so3linear_after_tp"] = {"nodes": N, "paths": len(dl.paths), "fwd_ms": t_l * 1e3, "fwd_bwd_ms": t_lb * 1e3,
                                 "fwd_kernel_ms": t_fk * 1e3, "dgrad_kernel_ms": t_dk * 1e3,
                                 "fwd_kernel_hbm_gbs": lbytes / t_fk / 1e9, "dgrad_kernel_hbm_gbs": lbytes / t_dk / 1e9,
                                 "fwd_kernel_frac_of_hbm": lbytes / t_fk / 1e9 / peak, "dgrad_kernel_frac_of_hbm": lbytes / t_dk / 1e9 / peak,
                                 "host_ms_per_fwd_bwd_pair": max(0.0, (t_lb - t_fk - t_dk) * 1e3),
                                 "fwd_hbm_gbs": lbytes / t_l / 1e9, "fwd_tflops": 2.0 * N * 128 * 128 * rows / t_fk / 1e12,
                                 "precision": "3xTF32 on tcgen05",
                                 "note": "*_kernel_*: launches replayed from a CUDA graph; fwd_ms / fwd_bwd_ms: through the public operator and autograd"}
    return out



def _events_ms(fn, k):
    """Mean milliseconds of ``fn`` over ``k`` back-to-back calls, CUDA events on the current stream."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(k):
        fn()
    b.record(); torch.cuda.synchronize()
    return a.elapsed_time(b) / k


def _graph_replay_ms(fn, k=10, reps=5):
    """Device time of ``fn``: ``k`` calls captured into one CUDA graph, the graph replayed ``reps`` times.  Replay has
    no per-launch host work, so this is kernel time even where the Python front-end is slower than the kernel."""
    from fasteq_b200.ops import _prepared
    fn(); fn(); torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    with torch.no_grad(), _prepared.frozen_weights(), torch.cuda.graph(g):
        for _ in range(k):
            fn()
    g.replay(); torch.cuda.synchronize()
    return _events_ms(g.replay, reps) / k


def cwtp_kernel_block(workload: str, dev, seed: int = 0):
    """Forward / backward kernels of one CWTP workload timed alone (bursts of 10 launches, as the copy the peak comes
    from) against the HBM roofline."""
    from fasteq_b200.ops import uniform1d_jit as u1d
    from fasteq_b200.sh import spherical_harmonics_host
    inp = build_inputs(workload, seed=seed)
    d, N, E, dtype = inp["d"], inp["N"], inp["E"], inp["dtype"]
    s = 4 if dtype == torch.float32 else 8
    y = torch.from_numpy(spherical_harmonics_host(WORKLOADS[workload][1], inp["vec"].numpy(), normalize=True)).to(dtype).contiguous().to(dev)
    w, x, r = inp["w"].to(dev), inp["x"].to(dev), inp["r"].to(dev)
    src, dst = inp["src"].to(dev), inp["dst"].to(dev)
    meta = d.meta(dtype, dev)
    call = u1d._Call(w, x, y, {1: src}, {0: dst}, meta)
    with torch.no_grad():
        for _ in range(3):
            u1d._run_fwd(call, w, x, y); u1d._run_bwd(call, r, w, x, y, (True, True, True))
        torch.cuda.synchronize()
        t_f = _events_ms(lambda: u1d._run_fwd(call, w, x, y), 10) * 1e-3
        t_b = _events_ms(lambda: u1d._run_bwd(call, r, w, x, y, (True, True, True)), 10) * 1e-3
    bf, bb = algorithmic_bytes(N, E, d, s)
    peak, kind = measured_peak()
    tun = {"fwd": u1d._tuning_for(call.spec, "fwd", (w, x, y)), "bwd": u1d._tuning_for(call.spec, "bwd", (w, x, y), (True, True, True))}
    pipe = {"fwd": fp32_floor(call.spec, tun["fwd"], "fwd", (False, False, False), E, d.u_dim, t_f, dev),
            "bwd": fp32_floor(call.spec, tun["bwd"], "bwd", (True, True, True), E, d.u_dim, t_b, dev)}
    return {"workload": workload, "fp32_pipe": pipe, "w_segs": d.w_seg_num, "out_segs": d.out_seg_num, "cg_paths": d.num_paths, "atoms": N, "edges": E,
            "fwd": {"launch_ms": t_f * 1e3, "achieved": bf / t_f / 1e9, "frac": bf / t_f / 1e9 / peak, "algorithmic_bytes_per_launch": bf,
                    "traffic": TRAFFIC_RATIO[workload]["fwd"] * bf},
            "bwd": {"launch_ms": t_b * 1e3, "achieved": bb / t_b / 1e9, "frac": bb / t_b / 1e9 / peak, "algorithmic_bytes_per_launch": bb,
                    "traffic": TRAFFIC_RATIO[workload]["bwd"] * bb},
            "fwd_bwd": {"achieved": (bf + bb) / (t_f + t_b) / 1e9, "frac": (bf + bb) / (t_f + t_b) / 1e9 / peak,
                        "frac_of_nominal_8TBs": (bf + bb) / (t_f + t_b) / 8e12, "edges_per_s": E / (t_f + t_b)},
            "unit": "GB/s", "peak": peak, "peak_kind": kind, "bound": "hbm",
            "tuning": {dr: {"pipes": t.pipes, "groups": t.groups, "stages": t.stages, "vec": t.vec, "ctas_per_sm": t.min_blocks,
                            "two_pass": t.two_pass, "grad_out_row": _go_home(t)} for dr, t in tun.items()}}


def config2_bench(dev, boxes=None):
    """benchmark configuration 2 at its stated size (``boxes`` shrinks it for a profiler capture): 32 periodic boxes x 384 atoms (side 15.6 A, cutoff 5 A), hidden
    256x0e+256x1o+256x2e, SH l <= 3, correlation 3, 2 layers, FP64, energy + forces.  Also the FP64 tensor-product
    kernels of the second interaction layer alone against the HBM roofline."""
    from fasteq_b200.graph import make_boxes
    from fasteq_b200.nn.mace_style import MACEStyleModel
    from fasteq_b200.ops import uniform1d_jit as u1d
    from fasteq_b200.sh import spherical_harmonics_host
    torch.manual_seed(0)
    model = MACEStyleModel(channels=256, hidden_lmax=2).double().to(dev)
    for prm in model.parameters():
        prm.requires_grad_(False)
    b = make_boxes(boxes or 32, 384, 15.6, 5.0, 4, seed=0)
    t = lambda a: torch.from_numpy(a).to(dev)
    args = (t(b.positions), t(b.species), t(b.edge_src), t(b.edge_dst), t(b.edge_shift), t(b.node_graph), b.n_graphs)
    run = lambda: model(*args)
    for _ in range(2):
        out = run()
    torch.cuda.synchronize()
    k = 3
    ms = _events_ms(run, k)
    res = {"metric": "MACE atom-steps/s (energy + forces), FP64", "value": b.n_nodes / (ms * 1e-3), "unit": "atom-steps/s",
           "ms_per_step": ms, "steps": k, "atoms": b.n_nodes, "edges": b.n_edges, "dtype": "f64",
           "config": f"config 2: {boxes or 32} boxes x 384 atoms, side 15.6 A, 2 layers, 256x0e+256x1o+256x2e, SH l<=3, correlation 3, FP64",
           "energy_finite": bool(torch.isfinite(out["energy"]).all()), "forces_finite": bool(torch.isfinite(out["forces"]).all())}
    del out
    # the layer-2 tensor product (17 weight / 71 output segments, 256 channels) in FP64, kernels alone
    d = model.layers[1].conv_tp.descriptor
    N, E, U = b.n_nodes, b.n_edges, d.u_dim
    g = torch.Generator().manual_seed(0)
    y = torch.from_numpy(spherical_harmonics_host(3, b.edge_vec, normalize=True)).contiguous().to(dev)
    x = torch.randn(N, d.x_seg_num * U, generator=g, dtype=torch.float64).to(dev)
    r = torch.randn(N, d.out_seg_num * U, generator=g, dtype=torch.float64).to(dev)
    w = torch.randn(E, d.w_seg_num * U, dtype=torch.float64, device=dev)
    meta = d.meta(torch.float64, dev)
    call = u1d._Call(w, x, y, {1: args[2].int()}, {0: args[3].int()}, meta)
    with torch.no_grad():
        u1d._run_fwd(call, w, x, y); u1d._run_bwd(call, r, w, x, y, (True, True, True)); torch.cuda.synchronize()
        t_f = _events_ms(lambda: u1d._run_fwd(call, w, x, y), 5) * 1e-3
        t_b = _events_ms(lambda: u1d._run_bwd(call, r, w, x, y, (True, True, True)), 5) * 1e-3
    bf, bb = algorithmic_bytes(N, E, d, 8)
    peak, kind = measured_peak()
    needs = (True, True, True)
    tun_f = u1d._tuning_for(call.spec, "fwd", (w, x, y, r))
    tun_b = u1d._tuning_for(call.spec, "bwd", (r, w, x, y), needs)
    res["cwtp_layer2_f64"] = {"w_segs": d.w_seg_num, "out_segs": d.out_seg_num, "u": U, "bound": "fp64 pipe (64 lanes per SM per clock)",
                              "unit": "GB/s", "peak": peak, "peak_kind": kind,
                              "fwd": {"launch_ms": t_f * 1e3, "achieved": bf / t_f / 1e9, "frac": bf / t_f / 1e9 / peak,
                                      **fp32_floor(call.spec, tun_f, "fwd", None, E, U, t_f, dev, lanes=64, tag="fp64")},
                              "bwd": {"launch_ms": t_b * 1e3, "achieved": bb / t_b / 1e9, "frac": bb / t_b / 1e9 / peak,
                                      **fp32_floor(call.spec, tun_b, "bwd", needs, E, U, t_b, dev, lanes=64, tag="fp64")}}
    return res


def config4_structures(n_structs: int = 1024, seed: int = 0):
    """benchmark configuration 4: atom counts uniform in 32..256, density 0.1 atoms / A^3 (cubic box side (n / 0.1)^(1/3))."""
    rng = np.random.default_rng(seed)
    atoms = rng.integers(32, 257, size=n_structs)
    side = (atoms / 0.1) ** (1.0 / 3.0)
    return atoms, side


def config4_sweep(args, dev, rank, world, dist, group_size: int = 128):
    """benchmark configuration 4: ONE fixed batch of 1024 independent periodic structures through the configuration-1
    MACE-style model (FP32, energy + forces), split by whole structure over the ranks (greedy bin packing by edge
    count) with no communication in the layer loop: strong scaling.  Every rank walks its structures in groups of at
    most ``group_size`` (one model call per group); the radius graphs are built on the GPU beforehand (timed apart)."""
    from fasteq_b200.graph import split_structures
    from fasteq_b200.neighbors import radius_graph
    from fasteq_b200.nn.mace_style import MACEStyleModel
    atoms, side = config4_structures()
    est_edges = atoms * (0.1 * 4.0 / 3.0 * np.pi * 125.0)
    mine = split_structures(est_edges, world)[rank]
    torch.manual_seed(0)
    model = MACEStyleModel().to(dev)
    for prm in model.parameters():
        prm.requires_grad_(False)
    groups = []
    t0 = time.perf_counter()
    for g0 in range(0, len(mine), group_size):
        ids = mine[g0:g0 + group_size]
        pos, spec, gid, boxes = [], [], [], []
        for local, sid in enumerate(ids):
            rng = np.random.default_rng(100000 + sid)          # a structure is the same whatever rank holds it
            n = int(atoms[sid])
            pos.append(rng.uniform(0.0, side[sid], size=(n, 3))); spec.append(rng.integers(0, 4, size=n))
            gid.append(np.full(n, local)); boxes.append(side[sid])
        p64 = torch.from_numpy(np.concatenate(pos)).to(dev)
        gr = torch.from_numpy(np.concatenate(gid)).to(dev)
        rg = radius_graph(p64, gr, np.asarray(boxes), 5.0, register_plan=False)
        groups.append(dict(pos=p64.float(), species=torch.from_numpy(np.concatenate(spec)).to(dev), src=rg.edge_src, dst=rg.edge_dst,
                           shift=rg.edge_shift.float(), graph=gr, n_graphs=len(ids)))
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0

    def one_pass():
        e_sum = torch.zeros((), dtype=torch.float64, device=dev)
        f_sq = torch.zeros((), dtype=torch.float64, device=dev)
        for gdat in groups:
            o = model(gdat["pos"], gdat["species"], gdat["src"], gdat["dst"], gdat["shift"], gdat["graph"], gdat["n_graphs"])
            e_sum = e_sum + o["energy"].double().sum()
            f_sq = f_sq + (o["forces"].double() ** 2).sum()
        return e_sum, f_sq
    for _ in range(2):
        one_pass()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    k = 3
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(k):
        e_sum, f_sq = one_pass()
    ev1.record(); torch.cuda.synchronize()
    n_atoms = sum(int(g["pos"].shape[0]) for g in groups)
    n_edges = sum(int(g["src"].numel()) for g in groups)
    tm = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
    tot = torch.stack([torch.tensor(float(n_atoms), dtype=torch.float64, device=dev),
                       torch.tensor(float(n_edges), dtype=torch.float64, device=dev), e_sum, f_sq])
    loads = torch.tensor([float(n_edges)], dtype=torch.float64, device=dev)
    lmax = loads.clone()
    if dist is not None:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        dist.all_reduce(lmax, op=dist.ReduceOp.MAX)
    ms = float(tm[0]) / k
    return {"metric": "MACE atom-steps/s (energy + forces), fixed batch of 1024 structures", "scaling": "strong",
            "value": float(tot[0]) / (ms * 1e-3), "unit": "atom-steps/s", "ms_per_step": ms, "steps": k, "n_gpus": world,
            "structures": 1024, "atoms": int(tot[0]), "edges": int(tot[1]), "max_edges_on_a_rank": int(lmax[0]),
            "structures_on_rank0": len(mine), "model_calls_per_step_on_rank0": len(groups),
            "energy_sum": float(tot[2]), "force_l2": float(tot[3].sqrt()), "graph_build_s_rank0": build_s,
            "config": "config 4: atoms uniform in 32..256 per structure, density 0.1 / A^3, cutoff 5 A, config-1 model, FP32; "
                      f"whole-structure split over {world} rank(s), groups of <= {group_size} structures per model call"}


def model_reference_cpu(threads: int):
    """The MACE-style model of configuration 1 evaluated by the CPU oracle (float64 torch, autograd forces) on ONE box of
    192 atoms: the CPU figure that stands beside the model's atom-steps/s."""
    from fasteq_b200.graph import config1_batch
    from fasteq_b200.nn.mace_style import MACEStyleModel
    from oracle import mace_style_ref
    torch.set_num_threads(threads)
    torch.manual_seed(0)
    model = MACEStyleModel()
    b = config1_batch(1, seed=0)
    a = (torch.from_numpy(b.positions), torch.from_numpy(b.species), torch.from_numpy(b.edge_src), torch.from_numpy(b.edge_dst),
         torch.from_numpy(b.edge_shift))
    mace_style_ref.energy_and_forces(model, *a)      # warm-up
    times = []
    for _ in range(2):
        t0 = time.perf_counter()
        mace_style_ref.energy_and_forces(model, *a)
        times.append(time.perf_counter() - t0)
    sec = float(np.mean(times))
    return {"value": b.n_nodes / sec, "unit": "atom-steps/s", "s_per_step": sec, "cores": threads, "kind": "port",
            "sample": f"1 box of 64 ({b.n_nodes} atoms, {b.n_edges} edges), 2 timed energy + forces evaluations, float64",
            "note": "dense torch restatement of the model's path formulas on the CPU (oracle/mace_style_ref.py); the e3nn package "
                    "itself cannot travel to the GPU box"}


def reference_arm(args):
    """The reference's CPU path (e3nn algorithm, restated in oracle/) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = len(os.sched_getaffinity(0))
    inp = build_inputs(args.workload, seed=0, n_boxes=1)
    eps, sec = cpu_reference_run(inp, max(1, args.steps), max(0, args.warmup), threads)
    in1, lsh, lout, boxes, dtype = WORKLOADS[args.workload]
    sample = f"1 of {boxes} boxes per step ({inp['N']} atoms, {inp['E']} edges), forward + autograd backward"
    from fasteq_b200.graph import config1_batch
    full = config1_batch(args.boxes or boxes, seed=0)          # the GPU arm's graph (rank 0), for the identical config entry
    line = {
        "impl": "reference", "metric": METRIC, "value": eps, "unit": "edges/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if dtype == torch.float32 else "f64", "data": "synthetic",
        # the arm's config is the GPU arm's, key for key (same workload); what was actually timed is described in `sample`
        "config": dict(config_dict(args.workload, dict(inp, n_boxes=args.boxes or boxes), args.gpus),
                       atoms_per_gpu=full.n_nodes, edges_per_gpu=full.n_edges),
        "cpu_baseline": {"value": eps, "unit": "edges/s", "cores": threads, "kind": "port", "sample": sample,
                         "torch_threads": torch.get_num_threads(), "os_cpu_count": os.cpu_count(), "note": CPU_NOTE},
        "e2e": {"value": eps, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def config_dict(workload, inp, n_gpus):
    in1, lsh, lout, boxes, dtype = WORKLOADS[workload]
    boxes = inp.get("n_boxes", boxes)
    d = inp["d"]
    return {"workload": workload, "irreps_in1": in1, "sh_lmax": lsh, "lmax_out": lout, "u": d.u_dim,
            "w_segs": d.w_seg_num, "out_segs": d.out_seg_num, "cg_paths": d.num_paths,
            "boxes_per_gpu": boxes, "atoms_per_box": 192, "box_side_A": 12.4, "cutoff_A": 5.0,
            "parallelism": f"whole-structure split, {n_gpus} rank(s), no data-path collective",
            "l2_policy": "inputs larger than L2 (per-edge weights alone are several GB)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="config1_cwtp", choices=sorted(WORKLOADS))
    ap.add_argument("--boxes", type=int, default=None, help="boxes per GPU (default: the workload's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-model", action="store_true")
    ap.add_argument("--no-halo", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the fixed batch of 1024 structures (configuration 4)")
    ap.add_argument("--no-sustained", action="store_true", help="skip the > 1 s repeat of the headline loop")
    ap.add_argument("--breakdown", action="store_true",
                    help="with --only single_graph: rank 0's device time per step by kernel family (torch profiler, CUPTI)")
    ap.add_argument("--only", default=None, choices=["operators", "other_signature", "config2", "fixed_batch", "single_graph", "model"],
                    help="run one of the side blocks alone and print its JSON (for profiling a block under ncu)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))

    from fasteq_b200.ops import fast_uniform1d_jit
    from fasteq_b200.ops import uniform1d_jit as u1d
    from fasteq_b200.sh import spherical_harmonics_host

    if args.only:
        block = {"operators": lambda: operator_extras(args, dev),
                 "other_signature": lambda: cwtp_kernel_block("config0_layout_cwtp" if args.workload == "config1_cwtp" else "config1_cwtp", dev),
                 "config2": lambda: config2_bench(dev, args.boxes),
                 "model": lambda: model_bench(args, dev, rank, dist, args.boxes or WORKLOADS[args.workload][3], quick=True),
                 "fixed_batch": lambda: config4_sweep(args, dev, rank, world, dist),
                 "single_graph": lambda: halo_model_bench(args, dev, rank, world, dist)}[args.only]()
        if rank == 0:
            print(json.dumps({"only": args.only, "n_gpus": world, "result": block}), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    inp = build_inputs(args.workload, seed=rank, n_boxes=args.boxes)
    d, N, E, dtype = inp["d"], inp["N"], inp["E"], inp["dtype"]
    s = 4 if dtype == torch.float32 else 8
    y_host = torch.from_numpy(spherical_harmonics_host(WORKLOADS[args.workload][1], inp["vec"].numpy(), normalize=True)).to(dtype).contiguous()
    meta = d.meta(dtype, dev)
    host = {k: inp[k].contiguous().pin_memory() for k in ("w", "x", "r", "src", "dst")}
    host["y"] = y_host.pin_memory()
    devt = {k: v.to(dev) for k, v in host.items()}
    w, x, y = (devt[k].requires_grad_(True) for k in ("w", "x", "y"))
    inp_idx, out_idx = {1: devt["src"]}, {0: devt["dst"]}

    def step():
        out = fast_uniform1d_jit(w, x, y, inp_idx, out_idx, meta)
        return torch.autograd.grad(out, (w, x, y), devt["r"])

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:   # sampled from the warm-up on, so that short runs still see the clocks under load
        for _ in range(max(3, args.warmup)):
            step()
        barrier()
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1)
    t = torch.tensor([ms, float(E)], dtype=torch.float64, device=dev)
    if dist is not None:
        tmax = t.clone(); dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone(); dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        ms, total_edges = float(tmax[0]), float(tsum[1])
    else:
        total_edges = float(E)
    value = total_edges * args.steps / (ms * 1e-3)

    # ---- per-kernel timing for the roofline (rank 0's kernels, CUDA events on the launch stream)
    call = u1d._Call(w, x, y, inp_idx, out_idx, meta)
    k = min(max(3, args.steps), 10)     # each kernel timed alone, a short burst (the peak it is compared with is a burst figure)
    def timed(fn):
        fn(); torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(k):
            fn()
        b.record(); torch.cuda.synchronize()
        return a.elapsed_time(b) / k * 1e-3
    with torch.no_grad():
        t_fwd = timed(lambda: u1d._run_fwd(call, w, x, y))
        t_bwd = timed(lambda: u1d._run_bwd(call, devt["r"], w, x, y, (True, True, True)))
    bytes_fwd, bytes_bwd = algorithmic_bytes(N, E, d, s)
    peak, peak_kind = measured_peak()
    roof = {"bound": "hbm", "kernel": "fasteq_u1d_bwd_kernel", "achieved": bytes_bwd / t_bwd / 1e9, "peak": peak,
            "unit": "GB/s", "frac": bytes_bwd / t_bwd / 1e9 / peak,
            "traffic": TRAFFIC_RATIO[args.workload]["bwd"] * bytes_bwd, "traffic_source": "ncu capture of a 16-box case, scaled by edges",
            "peak_kind": peak_kind,
            "algorithmic_bytes_per_launch": bytes_bwd, "launch_ms": t_bwd * 1e3}
    roof_fwd = {"bound": "hbm", "kernel": "fasteq_u1d_fwd_kernel", "achieved": bytes_fwd / t_fwd / 1e9, "peak": peak,
                "unit": "GB/s", "frac": bytes_fwd / t_fwd / 1e9 / peak, "traffic": TRAFFIC_RATIO[args.workload]["fwd"] * bytes_fwd,
                "algorithmic_bytes_per_launch": bytes_fwd,
                "launch_ms": t_fwd * 1e3}
    tun_f = u1d._tuning_for(call.spec, "fwd", (w, x, y))
    tun_b = u1d._tuning_for(call.spec, "bwd", (w, x, y), (True, True, True))
    roof["fp32_pipe"] = fp32_floor(call.spec, tun_b, "bwd", (True, True, True), E, d.u_dim, t_bwd, dev)
    roof_fwd["fp32_pipe"] = fp32_floor(call.spec, tun_f, "fwd", (False, False, False), E, d.u_dim, t_fwd, dev)
    roof["tuning"] = {k_: getattr(tun_b, k_) for k_ in ("pipes", "groups", "stages", "min_blocks", "two_pass")}
    roof["tuning"]["grad_out_row"] = _go_home(tun_b)
    roof_fwd["tuning"] = {k_: getattr(tun_f, k_) for k_ in ("pipes", "groups", "stages", "min_blocks", "two_pass")}
    roof_both = {"achieved": (bytes_fwd + bytes_bwd) / (t_fwd + t_bwd) / 1e9,
                 "frac": (bytes_fwd + bytes_bwd) / (t_fwd + t_bwd) / 1e9 / peak,
                 "edges_per_s_kernels_only": E / (t_fwd + t_bwd)}

    # ---- end to end: pinned host inputs in, scalar out, through the public operator
    e2e = None
    if not args.no_e2e:
        ke = max(2, min(args.steps, 5))
        h2d = sum(host[n].numel() * host[n].element_size() for n in ("w", "x", "y", "r", "src", "dst"))
        def e2e_step():
            dv = {n: host[n].to(dev, non_blocking=True) for n in ("w", "x", "y", "r", "src", "dst")}
            ww, xx, yy = (dv[n].requires_grad_(True) for n in ("w", "x", "y"))
            out = fast_uniform1d_jit(ww, xx, yy, {1: dv["src"]}, {0: dv["dst"]}, meta)
            gw, gx, gy = torch.autograd.grad(out, (ww, xx, yy), dv["r"])
            return float((out.sum() + gw.sum() + gx.sum() + gy.sum()).item())
        e2e_step(); barrier()
        t0 = time.perf_counter()
        for _ in range(ke):
            e2e_step()
        barrier()
        te = time.perf_counter() - t0
        tt = torch.tensor([te], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e = {"value": total_edges * ke / float(tt[0]), "unit": "edges/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": 8, "steps": ke,
               "note": "pinned host w/x/y/grad_out/indices copied in each step (PCIe-bound: per-edge weights dominate)"}

    # ---- the same loop held for at least a second (the headline region above is the driver's K steps, a short burst)
    n_sus = args.steps if args.no_sustained else max(args.steps, int(1200.0 / max(ms / args.steps, 1e-3)) + 1)
    with ClockSampler(local) as clocks_sus:
        barrier()
        ev0.record()
        for _ in range(n_sus):
            step()
        ev1.record()
        barrier()
    ms_sus = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(ms_sus, op=dist.ReduceOp.MAX)
    sustained = {"value": total_edges * n_sus / (float(ms_sus[0]) * 1e-3), "unit": "edges/s", "steps": n_sus,
                 "ms_per_step": float(ms_sus[0]) / n_sus, "seconds": float(ms_sus[0]) * 1e-3, "clocks": clocks_sus.summary(),
                 "note": "the headline loop again, held for more than a second, after the per-kernel and end-to-end measurements"}


    status = {name: m.device_status() for name, m in (("fwd", u1d.get_module(call.spec, "fwd")),
                                                      ("bwd", u1d.get_module(call.spec, "bwd", (True, True, True))))}

    def guarded(fn, *a, **k):
        """Optional blocks never take the benchmark line down: a failure is reported in place of the block."""
        try:
            return fn(*a, **k)
        except Exception as exc:
            import traceback
            return {"failed": f"{type(exc).__name__}: {str(exc)[:300]}", "where": traceback.format_exc().strip().splitlines()[-3:]}
        finally:
            torch.cuda.empty_cache()

    model = None
    if not args.no_model:
        del devt, w, x, y            # the operator benchmark's 10+ GB of weights are not needed any more
        torch.cuda.empty_cache()
        model = model_bench(args, dev, rank, dist, args.boxes or WORKLOADS[args.workload][3])
        if not args.no_halo:
            model["single_graph"] = halo_model_bench(args, dev, rank, world, dist)
        torch.cuda.empty_cache()
        if not args.no_sweep:
            model["fixed_batch_1024"] = config4_sweep(args, dev, rank, world, dist)
        torch.cuda.empty_cache()

    # blocks that describe one GPU (other signatures, configuration 2, stand-alone operators, CPU figures): N = 1 runs only
    extras = other_sig = config2 = None
    if rank == 0 and world == 1 and not args.no_model:
        extras = guarded(operator_extras, args, dev)
        other = "config0_layout_cwtp" if args.workload == "config1_cwtp" else "config1_cwtp"
        other_sig = guarded(cwtp_kernel_block, other, dev)
        config2 = guarded(config2_bench, dev)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = len(os.sched_getaffinity(0))
        small = build_inputs(args.workload, seed=0, n_boxes=1)
        eps, sec = cpu_reference_run(small, steps=2, warmup=1, threads=threads)
        cpu = {"value": eps, "unit": "edges/s", "cores": threads, "kind": "port",
               "sample": f"1 box ({small['N']} atoms, {small['E']} edges), 2 timed forward+backward passes of the e3nn-algorithm oracle",
               "torch_threads": torch.get_num_threads(), "os_cpu_count": os.cpu_count(), "note": CPU_NOTE}
        if model is not None:
            model["cpu_baseline"] = guarded(model_reference_cpu, threads)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32" if dtype == torch.float32 else "f64", "data": "synthetic",
            "config": dict(config_dict(args.workload, inp, world), atoms_per_gpu=N, edges_per_gpu=E),
            "value_sustained": sustained,
            "roofline": roof, "roofline_fwd": roof_fwd, "roofline_fwd_bwd": roof_both, "cpu_baseline": cpu, "e2e": e2e, "model": model, "operators": extras,
            "other_signature": other_sig, "config2": config2,
            "gpu_launches": 2 * args.steps, "clocks": clocks.summary(), "device_status": status,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
