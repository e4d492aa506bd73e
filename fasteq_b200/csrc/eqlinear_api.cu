// The SO3Linear entry points in the SHAPE of the reference's per-precision backend interface: a table of function
// pointers { forward_create, forward_run, forward_destroy, dgrad_create, dgrad_run, dgrad_destroy, status_string }
// returned by an extern "C" fasteq_eqlinear_<precision>_api()
// (fasteq/cuda/src/eqlinear/common/eqlinear_backend_api.h:12-27; problem and plan-info layouts
// eqlinear_common.h:30-62; the dispatcher that consumes the table: dispatch/eqlinear_dispatch.cpp:215-312).
// A dispatcher built against that interface can load this library in place of a backend DSO.
//
// A plan copies the path tables (the caller's arrays are borrowed only during create, as in the reference), owns a
// device copy of the weights in the form its kernel multiplies with (tensor-core precision: the pre-scaled, K-major
// TF32-split blocks of fasteq_eqlinear_pack; otherwise the raw blocks), and is bound to the batch size of its
// problem.  create allocates (cudaMalloc) and enqueues the weight preparation on `stream`; run enqueues one launch;
// destroy frees (which waits for the device, the reference's behaviour: device_lifetime.h:48-73).
#include <cstdint>
#include <cstring>
#include <new>
#include <vector>
#include <cuda_runtime.h>
#include "fasteq_b200.h"
#include "core_common.h"

using namespace fasteq;

namespace {

struct Plan {
  fasteq_eqlinear_problem prob{};
  std::vector<int32_t> in_row, out_row, rows;
  std::vector<double> coeff;
  void* weights = nullptr;     // device: packed (tensor-core path) or a clone of the caller's blocks
  bool packed = false;
  bool dgrad = false;
  int device = 0;
};

size_t elem_bytes(int precision) { return precision == FASTEQ_EQLIN_FP64 ? 8 : 4; }

// Path tables from the interface's problem: the explicit (input_row, output_row, weight_path, rows) mapping when given,
// else the historical dense layout (consecutive paths with equal i share their output rows; eqlinear_group_table.cpp:7-47).
int fill_tables(const fasteq_eqlinear_problem_c* pc, const double* cg, Plan* pl) {
  const int P = pc->P;
  if (P < 1 || P > 64 || pc->U < 1 || pc->V < 1 || pc->B < 0 || pc->I < 1 || pc->J < 1) return FASTEQ_INVALID;
  if (!cg || (!pc->paths && !pc->i_dims)) return FASTEQ_INVALID;
  pl->in_row.resize(P); pl->out_row.resize(P); pl->rows.resize(P); pl->coeff.resize(P);
  if (pc->paths) {
    for (int q = 0; q < P; ++q) {
      const fasteq_eqlinear_path_c& a = pc->paths[q];
      if (a.weight_path < 0 || a.weight_path >= P) return FASTEQ_INVALID;
      // kernels index weight block q for table entry q: entries are stored in weight-block order
      const int w = a.weight_path;
      pl->in_row[w] = a.input_row; pl->out_row[w] = a.output_row; pl->rows[w] = a.rows; pl->coeff[w] = cg[q];
    }
  } else {
    int in_row = 0, out_row = 0, prev = -1;
    for (int q = 0; q < P; ++q) {
      const int i = pc->i_dims[q];
      if (i < 1) return FASTEQ_INVALID;
      if (prev >= 0 && prev != i) out_row += prev;
      pl->in_row[q] = in_row; pl->out_row[q] = out_row; pl->rows[q] = i; pl->coeff[q] = cg[q];
      in_row += i; prev = i;
    }
    if (in_row > pc->I || out_row + prev > pc->J) return FASTEQ_INVALID;
  }
  return FASTEQ_OK;
}

int create(int precision, bool dgrad, const fasteq_eqlinear_problem_c* pc, const void* w, const double* cg, cudaStream_t stream,
           void** plan, fasteq_eqlinear_plan_info* info) {
  if (!pc || !w || !plan) return FASTEQ_INVALID;
  Plan* pl = new (std::nothrow) Plan();
  if (!pl) return FASTEQ_INTERNAL;
  int rc = fill_tables(pc, cg, pl);
  if (rc != FASTEQ_OK) { delete pl; return rc; }
  pl->dgrad = dgrad;
  pl->prob.precision = precision; pl->prob.u = pc->U; pl->prob.v = pc->V; pl->prob.in_rows = pc->I; pl->prob.out_rows = pc->J;
  pl->prob.num_paths = pc->P; pl->prob.batch = pc->B;
  pl->prob.in_row = pl->in_row.data(); pl->prob.out_row = pl->out_row.data(); pl->prob.rows = pl->rows.data(); pl->prob.coeff = pl->coeff.data();
  cudaError_t e = cudaGetDevice(&pl->device);
  if (e != cudaSuccess) { delete pl; return cuda_fail(e); }
  const size_t n = (size_t)pc->P * pc->U * pc->V;
  int impl = 1;     // 1 = FMA tile kernel on the raw weight blocks, 2 = tcgen05 3xTF32 kernel on prepared blocks
  if (precision == FASTEQ_EQLIN_TF32X3) {
    e = cudaMalloc(&pl->weights, 2 * n * sizeof(float));
    if (e != cudaSuccess) { delete pl; return cuda_fail(e); }
    rc = fasteq_eqlinear_pack(&pl->prob, dgrad ? 1 : 0, w, pl->weights, (fasteq_stream_t)stream);
    if (rc == FASTEQ_OK) { pl->packed = true; impl = 2; }
    else { cudaFree(pl->weights); pl->weights = nullptr; if (rc != FASTEQ_UNSUPPORTED) { delete pl; return rc; } }
  }
  if (!pl->weights) {
    e = cudaMalloc(&pl->weights, n * elem_bytes(precision));
    if (e != cudaSuccess) { delete pl; return cuda_fail(e); }
    e = cudaMemcpyAsync(pl->weights, w, n * elem_bytes(precision), cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) { cudaFree(pl->weights); delete pl; return cuda_fail(e); }
  }
  if (info) {
    info->precision = precision; info->a_view = 1; info->j_rows = pc->J;
    info->forward_impl = dgrad ? -1 : impl; info->dgrad_impl = dgrad ? impl : -1;
  }
  *plan = pl;
  return FASTEQ_OK;
}

int run(void* plan, const void* a, void* c, cudaStream_t stream) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl || !a || !c) return pl && pl->prob.batch == 0 ? FASTEQ_OK : FASTEQ_INVALID;
  fasteq_stream_t s = (fasteq_stream_t)stream;
  if (pl->packed) {
    int rc = pl->dgrad ? fasteq_eqlinear_dgrad_packed(&pl->prob, pl->weights, a, c, s) : fasteq_eqlinear_forward_packed(&pl->prob, pl->weights, a, c, s);
    return rc;      // FASTEQ_UNSUPPORTED here means operands the tensor-core kernel refuses (alignment): the caller's error
  }
  return pl->dgrad ? fasteq_eqlinear_dgrad(&pl->prob, pl->weights, a, c, s) : fasteq_eqlinear_forward(&pl->prob, pl->weights, a, c, s);
}

void destroy(void* plan) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl) return;
  int cur = 0;
  const bool sw = cudaGetDevice(&cur) == cudaSuccess && cur != pl->device && cudaSetDevice(pl->device) == cudaSuccess;
  if (pl->weights) cudaFree(pl->weights);      // waits for work that may still read the buffer
  if (sw) cudaSetDevice(cur);
  delete pl;
}

template <int PREC> int fwd_create(const fasteq_eqlinear_problem_c* p, const void* w, const double* cg, void* s, void** plan,
                                   fasteq_eqlinear_plan_info* info) { return create(PREC, false, p, w, cg, (cudaStream_t)s, plan, info); }
template <int PREC> int dg_create(const fasteq_eqlinear_problem_c* p, const void* w, const double* cg, void* s, void** plan,
                                  fasteq_eqlinear_plan_info* info) { return create(PREC, true, p, w, cg, (cudaStream_t)s, plan, info); }
int any_run(void* plan, const void* a, void* c, void* s) { return run(plan, a, c, (cudaStream_t)s); }

template <int PREC> const fasteq_eqlinear_backend_api* table() {
  static const fasteq_eqlinear_backend_api api = {2u, PREC, &fwd_create<PREC>, &any_run, &destroy, &dg_create<PREC>, &any_run, &destroy,
                                                  &fasteq_status_string};
  return &api;
}

}  // namespace

extern "C" const fasteq_eqlinear_backend_api* fasteq_eqlinear_tf32_api(void) { return table<FASTEQ_EQLIN_TF32X3>(); }
extern "C" const fasteq_eqlinear_backend_api* fasteq_eqlinear_fp32_api(void) { return table<FASTEQ_EQLIN_FP32>(); }
extern "C" const fasteq_eqlinear_backend_api* fasteq_eqlinear_fp64_api(void) { return table<FASTEQ_EQLIN_FP64>(); }
