"""The SO3Linear backend-interface table (``fasteq_eqlinear_<precision>_api``: create / run / destroy function pointers in
the layout of the reference's ``EqLinearBackendApi``, fasteq/cuda/src/eqlinear/common/eqlinear_backend_api.h:12-27)
driven through ctypes the way a dispatcher would drive it, against the numpy oracle: the dense run-length layout
(``i_dims``), the explicit path mapping with permuted weight blocks, all three precisions, forward and grad_x."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import eqlinear_ref

pytestmark = pytest.mark.gpu


class PathC(C.Structure):
    _fields_ = [("input_row", C.c_int32), ("output_row", C.c_int32), ("weight_path", C.c_int32), ("rows", C.c_int32)]


class ProblemC(C.Structure):
    _fields_ = [("B", C.c_int32), ("I", C.c_int32), ("U", C.c_int32), ("P", C.c_int32), ("V", C.c_int32), ("J", C.c_int32),
                ("i_dims", C.POINTER(C.c_int32)), ("paths", C.POINTER(PathC))]


class PlanInfo(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("precision", "forward_impl", "dgrad_impl", "a_view", "j_rows")]


CREATE = C.CFUNCTYPE(C.c_int, C.POINTER(ProblemC), C.c_void_p, C.POINTER(C.c_double), C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(PlanInfo))
RUN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p)
DESTROY = C.CFUNCTYPE(None, C.c_void_p)
STATUS = C.CFUNCTYPE(C.c_char_p, C.c_int)


class Api(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("precision", C.c_int32), ("forward_create", CREATE), ("forward_run", RUN),
                ("forward_destroy", DESTROY), ("dgrad_create", CREATE), ("dgrad_run", RUN), ("dgrad_destroy", DESTROY),
                ("status_string", STATUS)]


def _api(name):
    from fasteq_b200 import _cabi
    lib = _cabi.core()
    fn = getattr(lib, f"fasteq_eqlinear_{name}_api")
    fn.restype = C.POINTER(Api)
    return fn().contents


def _rel(a, b):
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


@pytest.mark.parametrize("name,code,dtype,tol", [("fp64", 2, torch.float64, 1e-12), ("fp32", 1, torch.float32, 2e-6), ("tf32", 0, torch.float32, 1e-5)])
@pytest.mark.parametrize("layout", ["i_dims", "paths"])
def test_backend_table_runs_forward_and_dgrad(name, code, dtype, tol, layout):
    api = _api(name)
    assert api.abi_version == 2 and api.precision == code and api.status_string(0) == b"ok"
    g = torch.Generator().manual_seed(3)
    B, U, V = 517, 64, 96
    if layout == "i_dims":
        i_dims = [1, 1, 3, 3, 3, 5]                                   # runs (1,1) (3,3,3) (5): J = 9 output rows
        mapping = eqlinear_ref.mapping_from_i_dims(i_dims)
        I, J, P = sum(i_dims), eqlinear_ref.out_rows(i_dims), len(i_dims)
        arr = (C.c_int32 * P)(*i_dims)
        prob = ProblemC(B, I, U, P, V, J, arr, None)
    else:
        # explicit mapping, weight blocks in another order than the paths, one input block nobody reads
        mapping = [(0, 3, 2, 3), (3, 0, 0, 1), (4, 3, 1, 3), (10, 6, 3, 5)]      # (in_row, out_row, weight block, rows)
        I, J, P = 15, 11, 4
        arr = (PathC * P)(*[PathC(*m) for m in mapping])
        prob = ProblemC(B, I, U, P, V, J, None, arr)
    cg = [0.01 + 0.001 * q for q in range(P)]
    x = torch.randn(B, I, U, generator=g, dtype=torch.float64)
    w = torch.randn(P, U, V, generator=g, dtype=torch.float64)
    r = torch.randn(B, J, V, generator=g, dtype=torch.float64)
    ref = eqlinear_ref.eqlinear_forward(x.numpy(), w.numpy(), mapping, cg, J)
    ref_gx = eqlinear_ref.eqlinear_dgrad(r.numpy(), w.numpy(), mapping, cg, I)
    xd, wd, rd = x.to(dtype).cuda(), w.to(dtype).cuda(), r.to(dtype).cuda()
    out = torch.full((B, J, V), float("nan"), dtype=dtype, device="cuda")
    gx = torch.full((B, I, U), float("nan"), dtype=dtype, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    cgarr = (C.c_double * P)(*cg)
    plan, info = C.c_void_p(), PlanInfo()
    assert api.forward_create(C.byref(prob), wd.data_ptr(), cgarr, stream, C.byref(plan), C.byref(info)) == 0
    assert info.precision == code and info.j_rows == J and info.forward_impl == (2 if name == "tf32" else 1)
    wd_saved = wd.clone()
    wd.zero_()                       # the plan owns its weights: the caller's tensor may change after create
    for _ in range(2):
        assert api.forward_run(plan, xd.data_ptr(), out.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    api.forward_destroy(plan)
    assert _rel(out.cpu().double().numpy(), ref) <= tol
    plan2 = C.c_void_p()
    assert api.dgrad_create(C.byref(prob), wd_saved.data_ptr(), cgarr, stream, C.byref(plan2), None) == 0
    assert api.dgrad_run(plan2, rd.data_ptr(), gx.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    api.dgrad_destroy(plan2)
    assert _rel(gx.cpu().double().numpy(), ref_gx) <= tol
    if layout == "paths":
        assert np.count_nonzero(gx.cpu().numpy()[:, 7:10]) == 0          # the input rows no path reads


def test_backend_table_rejects_bad_problems():
    api = _api("fp32")
    w = torch.zeros(4, device="cuda")
    plan = C.c_void_p()
    bad = ProblemC(8, 1, 2, 1, 2, 1, None, None)             # neither i_dims nor paths
    cg = (C.c_double * 1)(1.0)
    assert api.forward_create(C.byref(bad), w.data_ptr(), cg, None, C.byref(plan), None) == 2      # invalid argument
    assert api.status_string(2) == b"invalid argument"
