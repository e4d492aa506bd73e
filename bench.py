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
}
METRIC = "ChannelwiseTP edges/s (fwd+force bwd)"
# DRAM bytes (dram__bytes_read + dram__bytes_write) over algorithmic bytes, from one ncu capture per kernel
# on a 16-box case of the same workload; traffic grows in proportion to the edge count (every term
# is per edge or per node and the generator fixes edges per node), so the ratio carries to a full launch.
TRAFFIC_RATIO = {"config1_cwtp": {"fwd": 1.013, "bwd": 1.035}, "config0_layout_cwtp": {"fwd": 1.060, "bwd": 1.176}}


def algorithmic_bytes(N, E, d, s):
    """Each logical tensor once (unique node rows, per-edge tensors, outputs, indices)."""
    U = d.u_dim
    fwd = s * (N * d.x_seg_num * U + E * d.w_seg_num * U + E * d.y_seg_num + N * d.out_seg_num * U) + 8 * E
    bwd = s * (2 * E * d.w_seg_num * U + 2 * N * d.x_seg_num * U + 2 * E * d.y_seg_num + N * d.out_seg_num * U) + 8 * E
    return fwd, bwd


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
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


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
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return {"metric": "NequIP-style atom-steps/s, one 20,000-atom graph, receiver-range partition + halo", "scaling": "strong",
            "value": b.n_nodes * k / (float(ms[0]) * 1e-3), "unit": "atom-steps/s", "ms_per_step": float(ms[0]) / k,
            "atoms": b.n_nodes, "edges": b.n_edges, "owned": lg.n_owned, "ghosts": int(len(lg.ghost_global)),
            "config": "config 3: 4 gated layers, 64x0e+64x0o+64x1e+64x1o+64x2e+64x2o, SH l<=2, cutoff 4 A, FP32"}


def model_bench(args, dev, rank, dist, n_boxes: int):
    """Energy + forces of the synthetic MACE-style model of benchmark configuration 1 (FP32): atom-steps/s."""
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
    lens = (d.paths != -1).sum(1) - 1                       # multiplications + add per path: flops = B * U * sum of path lengths
    flops = float(B) * U * float(lens.sum())
    byts = 4.0 * (B * d.x1_segs * U + B * d.out_segs * U + 10 * d.x0_segs * U) + 4 * B
    out["stc_200k"] = {"nodes": B, "paths": d.num_paths, "fwd_ms": t_f * 1e3, "fwd_bwd_ms": t_fb * 1e3, "nodes_per_s_fwd": B / t_f,
                       "fwd_gflops_path_count": flops / t_f / 1e9, "fwd_hbm_gbs": byts / t_f / 1e9}
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
    rows = sum(p_rows for p_rows in [irr_tp[p.indices[1]].ir.dim for p in dl.paths])
    lbytes = 4.0 * (N * irr_tp.dim + N * 16 * 128 + dl.num_weights)
    out["so3linear_after_tp"] = {"nodes": N, "paths": len(dl.paths), "fwd_ms": t_l * 1e3, "fwd_bwd_ms": t_lb * 1e3,
                                 "fwd_hbm_gbs": lbytes / t_l / 1e9, "fwd_tflops": 2.0 * N * 128 * 128 * rows / t_l / 1e12,
                                 "precision": "3xTF32 on tcgen05"}
    return out


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
    line = {
        "impl": "reference", "metric": METRIC, "value": eps, "unit": "edges/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if dtype == torch.float32 else "f64", "data": "synthetic",
        # the arm's config is the GPU arm's (same workload); what was actually timed is described in `sample`
        "config": config_dict(args.workload, dict(inp, n_boxes=args.boxes or boxes), args.gpus),
        "cpu_baseline": {"value": eps, "unit": "edges/s", "cores": threads, "kind": "port", "sample": sample,
                         "torch_threads": torch.get_num_threads(), "os_cpu_count": os.cpu_count()},
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
        dist.init_process_group("nccl", device_id=dev)

    from fasteq_b200.ops import fast_uniform1d_jit
    from fasteq_b200.ops import uniform1d_jit as u1d
    from fasteq_b200.sh import spherical_harmonics_host

    inp = build_inputs(args.workload, seed=rank, n_boxes=args.boxes)
    d, N, E, dtype = inp["d"], inp["N"], inp["E"], inp["dtype"]
    s = 4 if dtype == torch.float32 else 8
    y_host = torch.from_numpy(spherical_harmonics_host(3, inp["vec"].numpy(), normalize=True)).to(dtype).contiguous()
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

    model = None
    if not args.no_model:
        del devt, w, x, y            # the operator benchmark's 10+ GB of weights are not needed any more
        torch.cuda.empty_cache()
        model = model_bench(args, dev, rank, dist, args.boxes or WORKLOADS[args.workload][3])
        if not args.no_halo:
            model["single_graph"] = halo_model_bench(args, dev, rank, world, dist)

    extras = None
    if rank == 0 and not args.no_model:
        extras = operator_extras(args, dev)

    status = {name: m.device_status() for name, m in (("fwd", u1d.get_module(call.spec, "fwd")),
                                                      ("bwd", u1d.get_module(call.spec, "bwd", (True, True, True))))}

    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        threads = len(os.sched_getaffinity(0))
        small = build_inputs(args.workload, seed=0, n_boxes=1)
        eps, sec = cpu_reference_run(small, steps=2, warmup=1, threads=threads)
        cpu = {"value": eps, "unit": "edges/s", "cores": threads, "kind": "port",
               "sample": f"1 box ({small['N']} atoms, {small['E']} edges), 2 timed forward+backward passes of the e3nn-algorithm oracle",
               "torch_threads": torch.get_num_threads(), "os_cpu_count": os.cpu_count()}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32" if dtype == torch.float32 else "f64", "data": "synthetic",
            "config": dict(config_dict(args.workload, inp, world), atoms_per_gpu=N, edges_per_gpu=E),
            "roofline": roof, "roofline_fwd": roof_fwd, "roofline_fwd_bwd": roof_both, "cpu_baseline": cpu, "e2e": e2e, "model": model, "operators": extras,
            "gpu_launches": 2 * args.steps, "clocks": clocks.summary(), "device_status": status,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
