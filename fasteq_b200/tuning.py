"""Measured launch configurations of the generated Uniform1D kernels, kept per operator signature.

The reference compiles a handful of candidates per signature, derives warps per block from the registers ptxas reports,
times them at several sizes and stores the winner on disk (fasteq/ops/uniform1d_jit.py:549-580, :975-1069; sizes in
fasteq/ops/auto_schedule/multi_size_tuning.py:9-21).  Here the knobs are those of the pipelined kernels -- pipelines
per CTA, thread groups, ring depth, resident CTAs, one or two passes in the backward, where the backward keeps the
receiver's grad_out row (shared memory, L1, tensor memory) -- and the procedure is:

* ``candidates(spec, direction)``: the configurations that fit one SM's shared memory and tensor memory;
* ``sweep(spec, direction, needs)`` (needs a GPU): compile every candidate, time its kernel alone on a synthetic
  receiver-sorted graph of the benchmark's density, then time the fastest and the heuristic default again in five
  alternating bursts; the challenger replaces the default only if it wins that alternation by more than the margin;
* the winners live in ``tuning_db.json`` beside this file (tracked, so that a fresh checkout starts tuned); the
  operator front-end asks ``lookup`` before it falls back to the heuristic ``codegen.u1d.default_tuning``.

``python -m fasteq_b200.tuning`` sweeps the standard signatures and rewrites the file.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Dict, List, Optional, Tuple

from .codegen import u1d as _emit
from .codegen.u1d_common import U1DSpec

DB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tuning_db.json")
_FIELDS = ("ct", "groups", "stages", "min_blocks", "vec", "two_pass", "pipes", "go_smem", "prefetch", "go_tmem")
_db: Optional[Dict[str, dict]] = None


def _key(spec: U1DSpec, direction: str, needs) -> str:
    return spec.key(f"tuning|{direction}|{tuple(bool(n) for n in needs)}")


def load_db() -> Dict[str, dict]:
    global _db
    if _db is None:
        try:
            with open(DB_PATH) as f:
                _db = json.load(f)
        except (OSError, ValueError):
            _db = {}
    return _db


_LOOKUPS: Dict[Tuple, Optional[_emit.Tuning]] = {}


def lookup(spec: U1DSpec, direction: str, needs=(False, False, False)) -> Optional[_emit.Tuning]:
    """The stored winner of this signature, or ``None``.  A signature with in-kernel spherical harmonics shares the
    entry of the same signature without them (the consumer code is identical).  Answers are memoised: the database
    key hashes the whole path table, which must not happen on every operator call."""
    memo = (spec, direction, tuple(bool(n) for n in needs))
    if memo in _LOOKUPS:
        return _LOOKUPS[memo]
    out = _LOOKUPS[memo] = _lookup(spec, direction, needs)
    return out


def _lookup(spec: U1DSpec, direction: str, needs) -> Optional[_emit.Tuning]:
    db = load_db()
    for sp in (spec, dataclasses.replace(spec, y_sh=()) if spec.y_sh else None):
        if sp is None:
            continue
        hit = db.get(_key(sp, direction, needs))
        if hit is not None:
            try:
                return _emit.Tuning(**{k: hit["tuning"][k] for k in _FIELDS if k in hit["tuning"]})
            except (KeyError, TypeError):
                return None
    return None


def smem_bytes(spec: U1DSpec, tun: _emit.Tuning, direction: str, need_gy: bool = True) -> int:
    """Dynamic shared memory of one CTA (mirrors the layout constants of the generated source)."""
    e = spec.elem_bytes
    tpg = tun.ct // tun.vec
    if direction == "fwd":
        return tun.pipes * (256 + tun.stages * _emit._stage_bytes(spec, tun.ct, 0))
    warps = tun.groups * tpg // 32
    extra = (warps * spec.y_segs * e + 15) // 16 * 16 if (need_gy and not spec.y_vec) else 0
    go = ((spec.out_segs * tun.ct * e + 127) // 128 * 128) if tun.go_smem else 0
    return tun.pipes * (256 + tun.stages * _emit._stage_bytes(spec, tun.ct, extra) + go)


def candidates(spec: U1DSpec, direction: str, needs=(True, True, True)) -> List[_emit.Tuning]:
    """Launch configurations worth timing: the heuristic default and its neighbours in (two to six pipelines, thread
    groups, ring depth, resident CTAs, passes; backward: the grad_out row staged in shared memory, read through L1 or
    parked in tensor memory; L2 prefetch distance) that fit 227 KB of shared memory, 1024 threads per CTA and 512
    columns of tensor memory."""
    base = _emit.default_tuning(spec, direction)
    out: List[_emit.Tuning] = [base]
    wpg = base.ct // (32 * base.vec)
    two_groups_ok = direction == "fwd" or not (spec.w_shared or spec.y_vec or spec.y_indexed or not spec.x_indexed)

    def add(pipes, groups, mb, two_pass, depths, go_smem=True, go_tmem=False):
        probe = dataclasses.replace(base, pipes=pipes, groups=groups, min_blocks=mb, two_pass=two_pass, stages=2, go_smem=go_smem,
                                    go_tmem=go_tmem)
        if go_tmem:
            try:
                _emit._check_tuning(spec, probe)
            except ValueError:
                return
        if pipes * groups * wpg > 16 or pipes * (groups * (probe.ct // probe.vec) + 32) > 1024:
            return
        per_stage = (smem_bytes(spec, dataclasses.replace(probe, stages=3), direction, needs[2]) -
                     smem_bytes(spec, probe, direction, needs[2]))
        room = 227 * 1024 // mb - smem_bytes(spec, probe, direction, needs[2])
        if room < 0:
            return
        fit = min(2 + room // max(per_stage, 1), 12 if direction == "fwd" else 6)
        for stages in sorted({max(2, min(d, fit)) for d in depths(fit)}):
            tun = dataclasses.replace(probe, stages=stages)
            if tun not in out:
                out.append(tun)

    for pipes in sorted({2, 3, 4, 5, 6, base.pipes}):
        for groups in ((1, 2) if two_groups_ok else (1,)):
            for mb in (1, 2):
                add(pipes, groups, mb, False, lambda fit: (fit, base.stages))          # deepest ring that fits, and the default depth
                if direction == "bwd":
                    # without the staged grad_out row (read through L1 instead) deeper rings and more pipelines fit
                    add(pipes, groups, mb, False, lambda fit: (fit, base.stages), go_smem=False)
                    if groups == 1 and mb == 1:
                        # ... or parked in tensor memory (one lane per consumer thread): the same room, no L1 traffic
                        add(pipes, groups, mb, False, lambda fit: (fit, max(2, fit - 1), base.stages), go_smem=False, go_tmem=True)
    if direction == "bwd":
        for groups in ((1, 2) if two_groups_ok else (1,)):
            add(base.pipes, groups, base.min_blocks, True, lambda fit: (fit,))         # two passes over a block: fewer live registers
    # L2 prefetch one and two ring-fuls ahead, on top of the default and of the deepest-ring variants of its shape
    for tun in [t for t in out if (t.pipes, t.groups, t.min_blocks, t.two_pass) == (base.pipes, base.groups, base.min_blocks, False)]:
        for pf in (1, 2):
            out.append(dataclasses.replace(tun, prefetch=pf))
    return out


def _inputs(spec: U1DSpec, n_boxes: int, device):
    """Synthetic receiver-sorted graph of the benchmark's density (192 atoms per 12.4 A box, cutoff 5 A) and random
    operands of this signature."""
    import torch
    b = _graph(n_boxes)
    g = torch.Generator(device=device).manual_seed(0)            # operands are drawn on the device: gigabytes at full size
    dt = torch.float32 if spec.dtype == "f32" else torch.float64
    N, E, U = b.n_nodes, b.n_edges, spec.u
    x = torch.randn(N, spec.x_segs * U, generator=g, dtype=dt, device=device)
    w = torch.randn(1 if spec.w_shared else E, spec.w_segs * U, generator=g, dtype=dt, device=device)
    ycols = 3 if spec.y_sh else spec.y_segs * (U if spec.y_vec else 1)
    y = torch.randn(E, ycols, generator=g, dtype=dt, device=device)
    r = torch.randn(N, spec.out_segs * U, generator=g, dtype=dt, device=device)
    src = torch.from_numpy(b.edge_src).int().to(device)
    dst = torch.from_numpy(b.edge_dst).int().to(device)
    return N, E, w, x, y, r, src, dst


_GRAPHS: Dict[int, object] = {}


def _graph(n_boxes: int):
    if n_boxes not in _GRAPHS:
        from .graph import config1_batch
        _GRAPHS[n_boxes] = config1_batch(n_boxes, seed=0)
    return _GRAPHS[n_boxes]


def sweep(spec: U1DSpec, direction: str, needs=(True, True, True), n_boxes: int = 64, launches: int = 8, repeats: int = 3,
          margin: float = 0.03, verbose: bool = False) -> dict:
    """Time every candidate's kernel alone (CUDA events around ``launches`` back-to-back launches after two warm-up
    launches; the best of ``repeats`` such bursts) and return the database entry of the fastest.  The heuristic default
    keeps its place unless a candidate beats it by more than ``margin`` in five alternating bursts of the two
    (run-to-run noise is a few per cent)."""
    import torch
    from . import _cabi
    from .ops import uniform1d_jit as u1d
    if not (spec.scattered and spec.x_indexed and not spec.y_indexed):
        raise ValueError("the sweep covers the gather / scatter signatures (x gathered, output scattered)")
    dev = torch.device("cuda", torch.cuda.current_device())
    N, E, w, x, y, r, src, dst = _inputs(spec, n_boxes, dev)
    plan = u1d.graph_plan(dst, N)
    results = []
    runners = {}
    bufs: Dict[str, object] = {}       # outputs shared by all candidates

    def burst(run):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(launches):
            run()
        b.record(); torch.cuda.synchronize()
        return a.elapsed_time(b) / launches

    for tun in candidates(spec, direction, needs):
        try:
            mod = u1d.get_module(spec, direction, needs if direction == "bwd" else (False, False, False), tuning=tun)
        except Exception as exc:                       # a candidate that does not compile (registers, shared memory) is skipped
            results.append({"tuning": dataclasses.asdict(tun), "failed": str(exc)[-200:]})
            continue
        gph = _cabi.U1DGraph()
        gph.n_edges, gph.n_out_rows, gph.x_rows, gph.y_rows = E, N, N, E
        gph.x_index, gph.y_index, gph.seg_ptr, gph.perm = src.data_ptr(), None, plan.seg_ptr.data_ptr(), None
        n_parts = max(1, min(u1d._sm_count(dev) * int(mod.desc.ctas_per_sm), N))
        gph.part_ptr, gph.n_parts = plan.partition(n_parts).data_ptr(), n_parts
        stream = torch.cuda.current_stream(dev).cuda_stream
        # (the closures bind this candidate's module and graph record: they are called again in the confirmation phase)
        if direction == "fwd":
            out = bufs.setdefault("out", torch.empty(N, spec.out_segs * spec.u, dtype=x.dtype, device=dev))
            run = lambda mod=mod, gph=gph: mod.forward(gph, w.data_ptr(), x.data_ptr(), y.data_ptr(), out.data_ptr(), stream)
        else:
            gw = bufs.setdefault("gw", torch.empty_like(w)) if needs[0] else None
            gx = bufs.setdefault("gx", torch.empty_like(x)) if needs[1] else None
            gy = bufs.setdefault("gy", torch.empty_like(y)) if needs[2] else None
            ptr = lambda t: t.data_ptr() if t is not None else None
            run = lambda mod=mod, gph=gph: mod.backward(gph, r.data_ptr(), w.data_ptr(), x.data_ptr(), y.data_ptr(), ptr(gw), ptr(gx), ptr(gy), stream)
        try:
            run(); run(); torch.cuda.synchronize()
            ms = min(burst(run) for _ in range(repeats))
            status = mod.device_status()
            runners[tun] = run
        except Exception as exc:
            results.append({"tuning": dataclasses.asdict(tun), "failed": str(exc)[-200:]})
            continue
        results.append({"tuning": dataclasses.asdict(tun), "ms": ms, "device_status": status})
        if verbose:
            print(f"  {direction} pipes={tun.pipes} groups={tun.groups} stages={tun.stages} ctas={tun.min_blocks} two_pass={tun.two_pass} prefetch={tun.prefetch} go={'smem' if tun.go_smem else ('tmem' if tun.go_tmem else 'l1')}: {ms:.4f} ms",
                  flush=True)
    good = [r_ for r_ in results if "ms" in r_ and r_["device_status"] == 0]
    if not good:
        raise RuntimeError("no candidate ran")
    best = min(good, key=lambda r_: r_["ms"])
    default_ms = results[0].get("ms")
    default_ok = default_ms is not None and results[0].get("device_status") == 0
    if default_ok and best is not results[0]:
        # confirmation: the GPU's clocks and temperature drift over a sweep, so the challenger and the default are timed
        # again in alternation; the default keeps its place unless it loses by more than the margin here too
        tb, td = _emit.Tuning(**best["tuning"]), _emit.Tuning(**results[0]["tuning"])
        b_ms = d_ms = float("inf")
        for _ in range(5):
            d_ms = min(d_ms, burst(runners[td])); b_ms = min(b_ms, burst(runners[tb]))
        best = dict(best, ms=b_ms, confirmed_against_default_ms=d_ms)
        if verbose:
            print(f"  confirmation: challenger {b_ms:.4f} ms, default {d_ms:.4f} ms (first pass {default_ms:.4f} ms)", flush=True)
        # the verdict rests on the alternation alone: both were timed in the same thermal state there, while the first
        # pass timed the default on a cooler GPU than the candidates after it
        if b_ms > d_ms * (1.0 - margin):
            best = dict(results[0], ms=min(default_ms, d_ms))
        default_ms = min(default_ms, d_ms)
    return {"tuning": best["tuning"], "ms": best["ms"], "default_ms": default_ms, "confirmed_against_default_ms": best.get("confirmed_against_default_ms"),
            "edges": E, "atoms": N,
            "gpu": torch.cuda.get_device_name(dev), "direction": direction, "needs": [bool(n) for n in needs],
            "signature": {"u": spec.u, "dtype": spec.dtype, "w_segs": spec.w_segs, "x_segs": spec.x_segs, "y_segs": spec.y_segs,
                          "out_segs": spec.out_segs, "paths": len(spec.paths)},
            "timed": [{"ms": r_.get("ms"), **{k: r_["tuning"][k] for k in ("pipes", "groups", "stages", "min_blocks", "two_pass", "prefetch")}}
                      for r_ in results]}


def standard_signatures() -> List[Tuple[str, U1DSpec]]:
    """The signatures of the benchmark configurations and the two synthetic models (without in-kernel harmonics)."""
    from .codegen.u1d_common import make_spec
    from .prebuild import cwtp_spec
    out = [("config0: 128x0e+128x1o+128x2e, all couplings l<=3", cwtp_spec("128x0e+128x1o+128x2e", 3, 3, "f32")),
           ("config1 operator: 128x0e+128x1o, all couplings l<=3", cwtp_spec("128x0e+128x1o", 3, 3, "f32"))]

    def of_model(tag, model, dtype):
        seen = set()
        for li, layer in enumerate(model.layers):
            d = layer.conv_tp.descriptor
            spec = make_spec(d.i_list, d.j_list, d.k_list, d.v_list, d.coeff_list, w_segs=d.w_seg_num, x_segs=d.x_seg_num,
                             y_segs=d.y_seg_num, out_segs=d.out_seg_num, u=d.u_dim, dtype=dtype)
            if spec not in seen:
                seen.add(spec)
                out.append((f"{tag} layer {li + 1}: {d.w_seg_num} weight / {d.out_seg_num} output segments, u = {d.u_dim}", spec))
    from .nn.mace_style import MACEStyleModel
    from .nn.nequip_style import NequIPStyleModel
    of_model("config1 model", MACEStyleModel(), "f32")
    of_model("config3 model", NequIPStyleModel(num_species=2, channels=64, lmax=2, sh_lmax=2, num_layers=4, r_max=4.0), "f32")
    of_model("config2 model", MACEStyleModel(channels=256, hidden_lmax=2), "f64")
    return out


def sweep_jobs(signatures=None):
    """(label, spec, direction, needs) of everything ``python -m fasteq_b200.tuning`` times."""
    jobs = []
    for label, spec in (signatures or standard_signatures()):
        jobs.append((label, spec, "fwd", (False, False, False)))
        jobs.append((label, spec, "bwd", (True, True, True)))
        if spec.x_segs == 1:
            jobs.append((label, spec, "bwd", (True, False, True)))     # first layer: the senders' features need no gradient
    return jobs


def main(argv=None) -> None:
    import argparse
    ap = argparse.ArgumentParser(description="time the launch configurations of the standard signatures on this GPU")
    ap.add_argument("--boxes", type=int, default=64, help="boxes of 192 atoms in the timing graph (64 = the benchmark's size)")
    ap.add_argument("--compile-only", action="store_true", help="build every candidate (no GPU needed), time nothing")
    ap.add_argument("--match", default=None, help="only signatures whose label contains this text")
    ap.add_argument("--direction", default=None, choices=["fwd", "bwd"], help="only this direction")
    args = ap.parse_args(argv)
    jobs = [j for j in sweep_jobs() if (args.match is None or args.match in j[0]) and args.direction in (None, j[2])]
    if args.compile_only:
        from concurrent.futures import ThreadPoolExecutor
        from .ops.uniform1d_jit import get_module
        todo = [(spec, d, needs if d == "bwd" else (False, False, False), tun) for _, spec, d, needs in jobs for tun in candidates(spec, d, needs)]
        def build(t):
            try:
                get_module(t[0], t[1], t[2], tuning=t[3])
                return 1
            except Exception as exc:
                print("skipped", t[3], str(exc)[-160:].replace("\n", " "), flush=True)
                return 0
        with ThreadPoolExecutor(max_workers=max(4, min(32, os.cpu_count() or 8))) as ex:
            n = sum(ex.map(build, todo))
        print(f"built {n} of {len(todo)} candidate modules")
        return
    db = dict(load_db())
    for label, spec, direction, needs in jobs:
        print(f"{label} [{direction} {needs}]", flush=True)
        entry = sweep(spec, direction, needs, n_boxes=args.boxes, verbose=True)
        entry["label"] = label
        db[_key(spec, direction, needs)] = entry
        print(f"  -> {entry['tuning']}  {entry['ms']:.4f} ms (heuristic default {entry['default_ms']})", flush=True)
    with open(DB_PATH, "w") as f:
        json.dump(db, f, indent=1, sort_keys=True)
    print("wrote", DB_PATH)


if __name__ == "__main__":
    main()
