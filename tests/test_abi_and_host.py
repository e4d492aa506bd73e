"""CPU-only checks: the C-ABI libraries load and export every symbol the header declares,
the code generator's table analysis, the synthetic graph generator, structure splitting."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "fasteq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fasteq_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    from fasteq_b200 import _build
    from fasteq_b200.prebuild import cwtp_spec
    from fasteq_b200.ops.uniform1d_jit import get_module
    core = ctypes.CDLL(_build.build_core())
    spec = cwtp_spec("32x0e+32x1o", 2, 2, "f32")
    fwd = ctypes.CDLL(get_module(spec, "fwd").path)
    bwd = ctypes.CDLL(get_module(spec, "bwd", (True, True, True)).path)
    from fasteq_b200.ops import spherical_harmonics as shmod, stc_uniform1d_jit as stcmod
    from fasteq_b200.prebuild import stc_spec
    import torch
    sh = shmod._module((0, 1, 2), torch.float32, True, "component")
    sspec = stc_spec("4x0e+4x1o", "4x0e", "f32")
    stc_fwd = ctypes.CDLL(stcmod.get_module(sspec, "fwd").path)
    stc_bwd = ctypes.CDLL(stcmod.get_module(sspec, "bwd", False).path)
    names = _declared_functions()
    assert len(names) >= 20
    for n in names:
        if n.startswith("fasteq_sh_"):
            assert hasattr(sh, n), n
            continue
        if n.startswith("fasteq_stc_"):
            assert hasattr(stc_fwd, n) and hasattr(stc_bwd, n), n
            continue
        if n.startswith("fasteq_u1d_"):
            assert hasattr(fwd, n) or hasattr(bwd, n), n
            if n != "fasteq_u1d_forward_noalloc":
                assert hasattr(fwd, n) and hasattr(bwd, n), n
        else:
            assert hasattr(core, n), n
    core.fasteq_status_string.restype = ctypes.c_char_p
    assert core.fasteq_status_string(0) == b"ok"
    assert core.fasteq_core_abi_version() == 1


def test_describe_reports_the_signature():
    from fasteq_b200.prebuild import cwtp_spec
    from fasteq_b200.ops.uniform1d_jit import get_module
    spec = cwtp_spec("32x0e+32x1o", 2, 2, "f64")
    d = get_module(spec, "bwd", (True, True, True)).desc
    assert (d.dtype, d.u, d.w_segs, d.x_segs, d.y_segs, d.out_segs) == (1, 32, spec.w_segs, 4, 9, spec.out_segs)
    assert d.direction == 1 and d.need_gw == d.need_gx == d.need_gy == 1 and d.scattered == 1


def test_blocks_cover_every_path_once():
    from fasteq_b200.codegen.u1d_common import build_blocks, split_out_segments
    from fasteq_b200.prebuild import cwtp_spec
    spec = cwtp_spec("128x0e+128x1o+128x2e", 3, 3, "f32")
    blocks = build_blocks(spec)
    assert 12 <= len(blocks) <= 144               # connected components of product sharing, inside (l1, l2) pairs
    items = [(t.i, j, k, t.v) for b in blocks for t in b.terms for (j, k, c) in t.items]
    assert sorted(items) == sorted((i, j, k, v) for (i, j, k, v, c) in spec.paths)
    assert sum(len(b.products) for b in blocks) == 9 * 16
    owners = split_out_segments(blocks, spec.out_segs, 2)
    assert sorted(owners[0] + owners[1]) == list(range(spec.out_segs))


def test_generated_source_has_no_cpu_path_and_bounded_waits():
    from fasteq_b200.codegen import u1d
    from fasteq_b200.prebuild import cwtp_spec
    spec = cwtp_spec("32x0e+32x1o", 2, 2, "f32")
    src = u1d.emit_forward(spec, u1d.default_tuning(spec, "fwd"))
    assert "fasteq_u1d_fwd_kernel<<<" in src and "extern \"C\" int fasteq_u1d_forward(" in src
    dev = open(os.path.join(ROOT, "fasteq_b200", "csrc", "fasteq_device.cuh")).read()
    assert "2000000000ull" in dev and "kDevWaitTimeout" in dev      # every mbarrier wait gives up
    # no wait's verdict is dropped: consumers derive global addresses from the stage record a completed wait
    # publishes, so a wait that gave up must end the loop (and stop the producer) instead of falling through
    bwd = u1d.emit_backward(spec, u1d.default_tuning(spec, "bwd"), True, True, True)
    pipe = open(os.path.join(ROOT, "fasteq_b200", "csrc", "u1d_pipeline.cuh")).read()
    for text in (src, bwd, pipe):
        for line in text.splitlines():
            if "mbar_wait(" in line and not line.lstrip().startswith("//"):
                assert "if (" in line and ("!mbar_wait(" in line or "if (mbar_wait(" in line), line


def test_config1_graph_generator():
    from fasteq_b200.graph import config1_batch, split_structures
    b = config1_batch(2, seed=0)
    assert b.n_nodes == 384 and (np.diff(b.edge_dst) >= 0).all()
    assert 45 < b.n_edges / b.n_nodes < 60                  # ~52 neighbours at cutoff 5 A
    r = np.linalg.norm(b.edge_vec, axis=1)
    assert r.max() < 5.0 and r.min() > 0.0
    # both directions present
    pairs = set(zip(b.edge_src.tolist(), b.edge_dst.tolist()))
    assert all((d, s) in pairs for s, d in list(pairs)[:200])
    parts = split_structures(np.array([5, 9, 1, 7, 3, 8]), 2)
    assert sorted(parts[0] + parts[1]) == list(range(6))
    loads = [sum([5, 9, 1, 7, 3, 8][i] for i in p) for p in parts]
    assert abs(loads[0] - loads[1]) <= 3


def test_op_rejects_cpu_tensors_without_a_gpu():
    import torch
    from fasteq_b200.ops import fast_uniform1d_jit
    from fasteq_b200.descriptors import channelwise_tensor_product, full_channelwise_instructions
    from fasteq_b200.irreps import Irreps
    io, ins = full_channelwise_instructions("4x0e", Irreps.spherical_harmonics(1), 1)
    d = channelwise_tensor_product("4x0e", Irreps.spherical_harmonics(1), io, ins)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fast_uniform1d_jit(torch.zeros(3, d.w_seg_num * 4), torch.zeros(2, 4), torch.zeros(3, 4), {1: torch.zeros(3, dtype=torch.int32)},
                           {0: torch.zeros(3, dtype=torch.int32)}, d.meta())


def test_fixed_batch_of_benchmark_configuration_4_splits_evenly():
    """1024 structures, 32..256 atoms each at density 0.1 / A^3; the whole-structure split over 1 / 2 / 4 / 8 ranks keeps
    every structure exactly once and balances the estimated edge counts to a few per cent."""
    import importlib.util
    from fasteq_b200.graph import split_structures
    spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec); spec.loader.exec_module(bench)
    atoms, side = bench.config4_structures()
    assert atoms.shape == (1024,) and atoms.min() >= 32 and atoms.max() <= 256
    np.testing.assert_allclose(atoms / side ** 3, 0.1, rtol=1e-12)
    a2, _ = bench.config4_structures()
    assert (a2 == atoms).all()                                   # the same batch at every world size
    for world in (1, 2, 4, 8):
        parts = split_structures(atoms * 52.0, world)
        assert sorted(i for p in parts for i in p) == list(range(1024))
        loads = np.array([atoms[p].sum() for p in parts], dtype=float)
        assert loads.max() / loads.mean() < 1.02


def test_device_status_helper_needs_no_gpu():
    """``fasteq_b200.status.device_status`` reads every loaded kernel family's status word; without CUDA it reports nothing."""
    import torch
    from fasteq_b200.status import device_status
    if not torch.cuda.is_available():
        assert device_status() == {}
