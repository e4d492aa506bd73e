"""Compile the generated modules of the standard signatures ahead of time (no GPU needed)."""
from __future__ import annotations

import time
from concurrent.futures import ThreadPoolExecutor

from .codegen.u1d_common import make_spec
from .descriptors import channelwise_tensor_product, full_channelwise_instructions
from .irreps import Irreps

# (irreps_in1, SH lmax, lmax_out, dtypes): benchmark configurations and the test / smoke signatures
STANDARD_CWTP = [
    ("128x0e+128x1o+128x2e", 3, 3, ("f32", "f64")),   # config 0
    ("128x0e+128x1o", 3, 3, ("f32",)),                # config 1 interaction
    ("64x0e+64x1o", 3, 3, ("f32", "f64")),
    ("32x0e+32x1o", 2, 2, ("f32", "f64")),
    ("33x0e+33x1o", 2, 2, ("f32",)),                  # a channel tail (u not a multiple of the tile)
]


def cwtp_spec(in1: str, lmax_sh: int, lmax_out: int, dtype: str):
    sh = Irreps.spherical_harmonics(lmax_sh)
    io, ins = full_channelwise_instructions(in1, sh, lmax_out)
    d = channelwise_tensor_product(in1, sh, io, ins)
    return make_spec(d.i_list, d.j_list, d.k_list, d.v_list, d.coeff_list, w_segs=d.w_seg_num, x_segs=d.x_seg_num,
                     y_segs=d.y_seg_num, out_segs=d.out_seg_num, u=d.u_dim, dtype=dtype)


# (irreps_in, irreps_out, dtypes) for the symmetric contraction
STANDARD_STC = [
    ("128x0e+128x1o+128x2e+128x3o", "128x0e+128x1o", ("f32", "f64")),   # config 1 product basis
]


def stc_spec(irreps_in: str, irreps_out: str, dtype: str):
    from .codegen.stc import make_stc_spec
    from .descriptors import symmetric_contraction
    d = symmetric_contraction(irreps_in, irreps_out)
    return make_stc_spec(d.paths, d.coeffs, x1_segs=d.x1_segs, x0_segs=d.x0_segs, out_segs=d.out_segs, u=d.u_dim, dtype=dtype)


def model_jobs(dtype: str = "f32", kind: str = "mace", **model_kwargs):
    """Module signatures a synthetic model needs at run time (forward, force backward)."""
    from .codegen.stc import make_stc_spec
    if kind == "mace":
        from .nn.mace_style import MACEStyleModel as Model
    else:
        from .nn.nequip_style import NequIPStyleModel as Model
    model = Model(**model_kwargs)
    u1d, stcj = [], []
    for layer in model.layers:
        d = layer.conv_tp.descriptor
        spec = make_spec(d.i_list, d.j_list, d.k_list, d.v_list, d.coeff_list, w_segs=d.w_seg_num, x_segs=d.x_seg_num,
                         y_segs=d.y_seg_num, out_segs=d.out_seg_num, u=d.u_dim, dtype=dtype)
        u1d += [(spec, "fwd", (False, False, False)), (spec, "bwd", (True, True, True)), (spec, "bwd", (True, False, True))]
        if getattr(model, "fuse_sh", False):      # the variants that evaluate the edge harmonics in the kernel
            import dataclasses
            fused = dataclasses.replace(spec, y_sh=(layer.conv_tp.sh_degrees(), True, "component"))
            u1d += [(fused, "fwd", (False, False, False)), (fused, "bwd", (True, True, True)), (fused, "bwd", (True, False, True))]
        if hasattr(layer, "product"):
            s = layer.product.descriptor
            sp = make_stc_spec(s.paths, s.coeffs, x1_segs=s.x1_segs, x0_segs=s.x0_segs, out_segs=s.out_segs, u=s.u_dim, dtype=dtype)
            stcj += [(sp, "fwd", False), (sp, "bwd", False)]
    return u1d, stcj, tuple(model.sh._ls)


def build_standard_modules(verbose: bool = False) -> None:
    from .ops.uniform1d_jit import get_module
    from .ops import stc_uniform1d_jit as stc
    jobs = []
    for in1, lsh, lout, dtypes in STANDARD_CWTP:
        for dt in dtypes:
            spec = cwtp_spec(in1, lsh, lout, dt)
            jobs.append((spec, "fwd", (False, False, False)))
            jobs.append((spec, "bwd", (True, True, True)))
    # the 128-channel signatures of the wide-layout parity tests, with and without in-kernel harmonics
    import dataclasses
    for in1, parity in (("128x0e+128x1o", None), ("128x0e+128x1o", "natural"), ("128x0e", "natural")):
        sh = Irreps.spherical_harmonics(3)
        io, ins = full_channelwise_instructions(in1, sh, 3, parity_filter=parity)
        d = channelwise_tensor_product(in1, sh, io, ins)
        spec = make_spec(d.i_list, d.j_list, d.k_list, d.v_list, d.coeff_list, w_segs=d.w_seg_num, x_segs=d.x_seg_num,
                         y_segs=d.y_seg_num, out_segs=d.out_seg_num, u=d.u_dim, dtype="f32")
        for sp in (spec, dataclasses.replace(spec, y_sh=((0, 1, 2, 3), True, "component"))):
            jobs += [(sp, "fwd", (False, False, False)), (sp, "bwd", (True, True, True))]
            # ... and on the heuristic four-pipeline layout, which those tests force next to the tuned one
            from .codegen.u1d import default_tuning
            jobs += [(sp, "fwd", (False, False, False), default_tuning(sp, "fwd")), (sp, "bwd", (True, True, True), default_tuning(sp, "bwd"))]
            # ... and on the backward layout that parks the grad_out row in tensor memory
            jobs.append((sp, "bwd", (True, True, True), dataclasses.replace(default_tuning(sp, "bwd"), go_smem=False, go_tmem=True, stages=6)))
    stc_jobs = []
    for a, b, dtypes in STANDARD_STC:
        for dt in dtypes:
            sp = stc_spec(a, b, dt)
            stc_jobs += [(sp, "fwd", False), (sp, "bwd", False), (sp, "bwd", True)]
    import torch
    from .ops import spherical_harmonics as shmod
    sh_jobs = []
    for dt, kind, kw in (("f32", "mace", {}), ("f64", "mace", dict(num_species=3, channels=32, r_max=3.5)),
                         ("f64", "mace", dict(channels=256, hidden_lmax=2)),       # benchmark configuration 2
                         ("f32", "mace", dict(num_species=3, channels=32, r_max=3.5)),
                         ("f32", "mace", dict(num_species=4, channels=128, r_max=4.0)),
                         ("f32", "nequip", dict(num_species=2, channels=64, lmax=2, sh_lmax=2, num_layers=4, r_max=4.0))):
        a, b, ls = model_jobs(dt, kind, **kw)
        jobs += a
        stc_jobs += b
        sh_jobs.append((ls, torch.float32 if dt == "f32" else torch.float64, True, "component"))
    jobs = list(dict.fromkeys(jobs)); stc_jobs = list(dict.fromkeys(stc_jobs)); sh_jobs = list(dict.fromkeys(sh_jobs))
    t0 = time.time()
    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(lambda j: shmod._module(*j), sh_jobs))
        list(ex.map(lambda j: get_module(*j), jobs))
        list(ex.map(lambda j: stc.get_module(*j), stc_jobs))
    if verbose:
        print(f"built {len(jobs)} Uniform1D and {len(stc_jobs)} symmetric-contraction modules in {time.time() - t0:.1f} s")
