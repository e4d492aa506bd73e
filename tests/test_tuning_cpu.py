"""The per-signature tuning layer on the CPU: candidate generation respects one SM's shared memory and thread limits, the
tracked database decodes, names only standard signatures, and the operator front-end picks its entries up."""
import dataclasses

import pytest

from fasteq_b200 import tuning
from fasteq_b200.codegen import u1d as gen
from fasteq_b200.prebuild import cwtp_spec


@pytest.mark.parametrize("in1,lmax,dtype", [("128x0e+128x1o+128x2e", 3, "f32"), ("128x0e+128x1o", 3, "f32"), ("64x0e+64x1o", 3, "f64"),
                                            ("33x0e+33x1o", 2, "f32")])
def test_candidates_fit_one_sm(in1, lmax, dtype):
    spec = cwtp_spec(in1, lmax, lmax, dtype)
    for direction, needs in (("fwd", (False, False, False)), ("bwd", (True, True, True))):
        cands = tuning.candidates(spec, direction, needs)
        assert cands[0] == gen.default_tuning(spec, direction)              # the heuristic default is always timed first
        assert len(cands) == len(set(cands)) and 1 <= len(cands) <= 96
        for t in cands:
            assert tuning.smem_bytes(spec, t, direction, needs[2]) * t.min_blocks <= 227 * 1024 or t == cands[0]
            assert t.pipes * (t.groups * (t.ct // t.vec) + 32) <= 1024
            if direction == "bwd" and t.groups == 2:
                gen.emit_backward(spec, t, *needs)                           # the generator accepts what the tuner proposes


def test_smem_model_matches_the_generated_constants():
    """``tuning.smem_bytes`` mirrors the SMEM_BYTES expression of the generated source (checked by evaluating it)."""
    import re
    spec = cwtp_spec("128x0e+128x1o", 3, 3, "f32")
    for direction in ("fwd", "bwd"):
        t = gen.default_tuning(spec, direction)
        src = gen.emit_forward(spec, t) if direction == "fwd" else gen.emit_backward(spec, t, True, True, True)
        assert "constexpr int SMEM_BYTES = cfg::PIPES * PIPE_BYTES;" in src
        stage = gen._stage_bytes(spec, t.ct, 0 if direction == "fwd" else (2 * 16 * 4 + 15) // 16 * 16)
        want = t.pipes * (256 + t.stages * stage + (0 if direction == "fwd" else (spec.out_segs * t.ct * 4 + 127) // 128 * 128))
        assert tuning.smem_bytes(spec, t, direction, True) == want


def test_database_entries_decode_and_are_used():
    db = tuning.load_db()
    if not db:
        pytest.skip("no tuning database in this checkout")
    keys = {tuning._key(spec, d, needs): (spec, d, needs) for _, spec, d, needs in tuning.sweep_jobs()}
    for k, entry in db.items():
        assert k in keys, f"entry {entry.get('label')} belongs to no standard signature"
        spec, d, needs = keys[k]
        t = tuning.lookup(spec, d, needs)
        assert isinstance(t, gen.Tuning) and t in tuning.candidates(spec, d, needs)
        # the winner is never slower than the default it was timed against: in alternation with it when it was a
        # challenger (the first pass times the default on a cooler GPU than the candidates after it)
        against = entry.get("confirmed_against_default_ms") or entry["default_ms"]
        assert entry["ms"] <= against * 1.0001
        # the front-end resolves the same configuration, also for the variant with in-kernel harmonics
        from fasteq_b200.ops import uniform1d_jit as u1d
        assert u1d._tuning_for(spec, d, (), needs) == t
        if spec.y_segs == 16 and not spec.y_vec:
            fused = dataclasses.replace(spec, y_sh=((0, 1, 2, 3), True, "component"))
            assert tuning.lookup(fused, d, needs) == t


def test_tensor_memory_layout_limits():
    """The backward layout that parks the grad_out row in tensor memory: column budget (512 per SM, shared by the resident
    CTAs), no shared-memory tile beside it, whole channel tiles only."""
    import dataclasses
    spec = cwtp_spec("128x0e+128x1o", 3, 3, "f32")
    base = gen.default_tuning(spec, "bwd")
    ok = dataclasses.replace(base, go_smem=False, go_tmem=True, stages=5)
    gen._check_tuning(spec, ok)
    assert gen.tmem_columns(spec, ok) == 256                      # 8 consumer warps: 2 per lane quarter x 110 columns -> 256
    assert "scratch_tmem_alloc" in gen.emit_backward(spec, ok, True, True, True)
    for bad in (dataclasses.replace(ok, go_smem=True), dataclasses.replace(ok, groups=2), dataclasses.replace(ok, min_blocks=3)):
        with pytest.raises(ValueError):
            gen._check_tuning(spec, bad)
    wide = cwtp_spec("128x0e+128x1o+128x2e", 3, 3, "f64")          # 106 segments x 2 columns: 4 pipelines of 2 warps do not fit
    with pytest.raises(ValueError):
        gen._check_tuning(wide, dataclasses.replace(gen.default_tuning(wide, "bwd"), pipes=6, go_smem=False, go_tmem=True))
    tail = cwtp_spec("33x0e+33x1o", 2, 2, "f32")                   # a channel tail would make the warp-collective loads diverge
    with pytest.raises(ValueError):
        gen._check_tuning(tail, dataclasses.replace(gen.default_tuning(tail, "bwd"), go_smem=False, go_tmem=True))


def test_instruction_counts_of_the_standard_signatures():
    """Multiply / FMA instructions per (edge, channel) in the generated source: the figures the bench line's arithmetic
    floors rest on.  One-product couplings (l1 = 0 or l2 = 0) cost 2n + 3 instructions for n output components in the
    backward (sum over the components first, then the shared operand), not 5n."""
    for in1, fwd, bwd in (("128x0e+128x1o", 220, 490), ("128x0e+128x1o+128x2e", 562, 1244)):
        spec = cwtp_spec(in1, 3, 3, "f32")
        f = gen.arith_ops(spec, gen.default_tuning(spec, "fwd"), "fwd", (False, False, False))
        b = gen.arith_ops(spec, gen.default_tuning(spec, "bwd"), "bwd", (True, True, True))
        assert (sum(f.values()), sum(b.values())) == (fwd, bwd)
    # a single l1 = 0 coupling with n = 7 components: 2 * 7 + 3 backward instructions
    from fasteq_b200.codegen.u1d_common import make_spec
    n = 7
    spec = make_spec([0] * n, [0] * n, list(range(n)), list(range(n)), [1.0] * n, w_segs=1, x_segs=1, y_segs=n, out_segs=n, u=64, dtype="f32")
    b = gen.arith_ops(spec, gen.default_tuning(spec, "bwd"), "bwd", (True, True, True))
    assert sum(b.values()) == 2 * n + 3
    # ... and an l2 = 0 coupling (the components differ in x, share y)
    spec = make_spec([0] * n, list(range(n)), [0] * n, list(range(n)), [1.0] * n, w_segs=1, x_segs=n, y_segs=1, out_segs=n, u=64, dtype="f32")
    b = gen.arith_ops(spec, gen.default_tuning(spec, "bwd"), "bwd", (True, True, True))
    assert sum(b.values()) == 2 * n + 3


def test_tensor_memory_columns_are_returned_on_every_consumer_exit():
    """Source check (no GPU fault is provoked to test this): in the tensor-memory layout the consumers leave their loop only
    through ``break`` - also when a bounded wait gave up - and the code after the loop holds the consumers' barrier and the
    release of the columns; the producers, which never touch tensor memory, are the only warps that return early."""
    import dataclasses
    spec = cwtp_spec("128x0e+128x1o", 3, 3, "f32")
    tun = dataclasses.replace(gen.default_tuning(spec, "bwd"), go_smem=False, go_tmem=True, stages=5)
    src = gen.emit_backward(spec, tun, True, True, True)
    kernel = src[src.index("fasteq_u1d_bwd_kernel("):]
    kernel = kernel[:kernel.index("__device__ int g_status_word")]
    consumer = kernel[kernel.index("p.run(flush, begin);"):]
    consumer = consumer[consumer.index("return;") + len("return;"):]          # past the producers' exit
    import re
    assert re.search(r"\breturn\b", consumer) is None
    loop_end = consumer.rindex("if (m.flags & F_DONE) break;")
    tail = consumer[loop_end:]
    assert tail.index("bar.sync 1") < tail.index("scratch_tmem_free(")
    assert kernel.index("scratch_tmem_alloc(") < kernel.index("p.run(flush, begin);")
    assert consumer.count("if (!mbar_wait(") >= 1 and "break;" in consumer
