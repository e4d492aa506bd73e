// Equivariant gate non-linearity (e3nn ``nn.Gate``) on ir_mul tensors, forward and backward.
//
//   out = [ c_i * act_i(scalar_i) ] (+) [ c_j * act_j(gate_j) * gated_j ]
//
// Input row layout [segments, u]: the scalar segments, then one gate segment per gated irrep block,
// then the gated irreps ((2l+1) segments each).  Output: scalar segments, then the gated irreps.
// The reference treats the gate as a neighbour of the hot path and ships it among its e3nn shims
// (fasteq/e3nn/triton/nn/_gate.py:17-39, fasteq/triton/fused_equivariant_gate.py).
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "fasteq_b200.h"
#include "core_common.h"

using namespace fasteq;

namespace {
constexpr int kMaxSeg = 96;

struct GateTable {
  int n_in, n_out, n_scalar, n_gate;
  int act[kMaxSeg];        // per scalar / gate segment (index = input segment): activation code
  double cst[kMaxSeg];     // second-moment normalisation constant of that activation
  int gate_of[kMaxSeg];    // per gated INPUT segment: its gate's input segment; -1 for scalars / gates
  int first_gated[kMaxSeg];// per gate segment: first gated input segment of its block
  int n_gated[kMaxSeg];    // per gate segment: 2l+1
};

template <typename T> __device__ __forceinline__ T act_f(int code, T x) {
  switch (code) {
    case 1: return x / (T(1) + exp(-x));               // silu
    case 2: return tanh(x);
    case 3: return T(1) / (T(1) + exp(-x));             // sigmoid
    case 4: return fabs(x);
    default: return x;
  }
}
template <typename T> __device__ __forceinline__ T act_d(int code, T x) {
  switch (code) {
    case 1: { const T s = T(1) / (T(1) + exp(-x)); return s * (T(1) + x * (T(1) - s)); }
    case 2: { const T t = tanh(x); return T(1) - t * t; }
    case 3: { const T s = T(1) / (T(1) + exp(-x)); return s * (T(1) - s); }
    case 4: return x >= T(0) ? T(1) : T(-1);
    default: return T(1);
  }
}

// One thread per (node, channel): it walks the row's segments, so the index arithmetic (one 64-bit division) and each
// gate's activation are paid once per thread instead of once per element, and every element is touched exactly once.
// Consecutive threads hold consecutive channels: each segment access of a warp is one contiguous 128-byte line.
template <typename T>
__global__ void __launch_bounds__(256) gate_fwd_kernel(const T* __restrict__ x, T* __restrict__ out, long long batch, int u,
                                                       const __grid_constant__ GateTable t) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch * u) return;
  const long long b = i / u;
  const int c = (int)(i - b * u);
  const T* row = x + (size_t)b * t.n_in * u + c;
  T* orow = out + (size_t)b * t.n_out * u + c;
  for (int s = 0; s < t.n_scalar; ++s) orow[(size_t)s * u] = T(t.cst[s]) * act_f<T>(t.act[s], row[(size_t)s * u]);
  for (int k = 0; k < t.n_gate; ++k) {
    const int g = t.n_scalar + k;
    const T a = T(t.cst[g]) * act_f<T>(t.act[g], row[(size_t)g * u]);
    const int s0 = t.first_gated[g];
    for (int m = 0; m < t.n_gated[g]; ++m) orow[(size_t)(s0 + m - t.n_gate) * u] = a * row[(size_t)(s0 + m) * u];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gate_bwd_kernel(const T* __restrict__ x, const T* __restrict__ go, T* __restrict__ gx,
                                                       long long batch, int u, const __grid_constant__ GateTable t) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch * u) return;
  const long long b = i / u;
  const int c = (int)(i - b * u);
  const T* row = x + (size_t)b * t.n_in * u + c;
  const T* grow = go + (size_t)b * t.n_out * u + c;
  T* gxr = gx + (size_t)b * t.n_in * u + c;
  for (int s = 0; s < t.n_scalar; ++s)
    gxr[(size_t)s * u] = grow[(size_t)s * u] * T(t.cst[s]) * act_d<T>(t.act[s], row[(size_t)s * u]);
  for (int k = 0; k < t.n_gate; ++k) {
    const int g = t.n_scalar + k;
    const T xg = row[(size_t)g * u];
    const T a = T(t.cst[g]) * act_f<T>(t.act[g], xg);
    const int s0 = t.first_gated[g];
    T acc = T(0);
    for (int m = 0; m < t.n_gated[g]; ++m) {
      const T gv = grow[(size_t)(s0 + m - t.n_gate) * u];
      acc += gv * row[(size_t)(s0 + m) * u];
      gxr[(size_t)(s0 + m) * u] = gv * a;
    }
    gxr[(size_t)g * u] = acc * T(t.cst[g]) * act_d<T>(t.act[g], xg);
  }
}

template <typename T> __device__ __forceinline__ T act_dd(int code, T x) {
  switch (code) {
    case 1: { const T s = T(1) / (T(1) + exp(-x)); return s * (T(1) - s) * (T(2) + x * (T(1) - T(2) * s)); }
    case 2: { const T t = tanh(x); return T(-2) * t * (T(1) - t * t); }
    case 3: { const T s = T(1) / (T(1) + exp(-x)); return s * (T(1) - s) * (T(1) - T(2) * s); }
    default: return T(0);
  }
}

// Second order: t = cotangent of grad_x.  d_go over the output elements, d_x over the input elements.
template <typename T>
__global__ void gate_dbwd_go_kernel(const T* __restrict__ x, const T* __restrict__ t_, T* __restrict__ d_go, long long batch, int u,
                                    const __grid_constant__ GateTable t) {
  const long long total = batch * t.n_out * u;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % u);
    const int so = (int)((i / u) % t.n_out);
    const long long b = i / ((long long)u * t.n_out);
    const T* row = x + (size_t)b * t.n_in * u;
    const T* trow = t_ + (size_t)b * t.n_in * u;
    if (so < t.n_scalar) {
      d_go[i] = trow[(size_t)so * u + c] * T(t.cst[so]) * act_d<T>(t.act[so], row[(size_t)so * u + c]);
    } else {
      const int si = so + t.n_gate, g = t.gate_of[si];
      const T xg = row[(size_t)g * u + c];
      // grad_x[gate] = c a'(x_g) sum_m go_m x_m  and  grad_x[gated m] = go_m c a(x_g)
      d_go[i] = T(t.cst[g]) * (trow[(size_t)g * u + c] * act_d<T>(t.act[g], xg) * row[(size_t)si * u + c] +
                               trow[(size_t)si * u + c] * act_f<T>(t.act[g], xg));
    }
  }
}

template <typename T>
__global__ void gate_dbwd_x_kernel(const T* __restrict__ x, const T* __restrict__ go, const T* __restrict__ t_, T* __restrict__ d_x,
                                   long long batch, int u, const __grid_constant__ GateTable t) {
  const long long total = batch * t.n_in * u;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % u);
    const int si = (int)((i / u) % t.n_in);
    const long long b = i / ((long long)u * t.n_in);
    const T* row = x + (size_t)b * t.n_in * u;
    const T* trow = t_ + (size_t)b * t.n_in * u;
    const T* grow = go + (size_t)b * t.n_out * u;
    if (si < t.n_scalar) {
      d_x[i] = trow[(size_t)si * u + c] * grow[(size_t)si * u + c] * T(t.cst[si]) * act_dd<T>(t.act[si], row[(size_t)si * u + c]);
    } else if (si < t.n_scalar + t.n_gate) {
      const T xg = row[(size_t)si * u + c];
      T dot = T(0), tdot = T(0);
      for (int m = 0; m < t.n_gated[si]; ++m) {
        const int sg = t.first_gated[si] + m;
        const T gm = grow[(size_t)(sg - t.n_gate) * u + c];
        dot += gm * row[(size_t)sg * u + c];
        tdot += gm * trow[(size_t)sg * u + c];
      }
      d_x[i] = T(t.cst[si]) * (trow[(size_t)si * u + c] * act_dd<T>(t.act[si], xg) * dot + act_d<T>(t.act[si], xg) * tdot);
    } else {
      const int g = t.gate_of[si];
      d_x[i] = trow[(size_t)g * u + c] * T(t.cst[g]) * act_d<T>(t.act[g], row[(size_t)g * u + c]) * grow[(size_t)(si - t.n_gate) * u + c];
    }
  }
}

int build(const fasteq_gate_problem* p, GateTable* t) {
  if (!p || p->n_scalar < 0 || p->n_gate < 0 || p->u < 1 || p->batch < 0) return FASTEQ_INVALID;
  if ((p->n_scalar + p->n_gate) > 0 && (!p->act || !p->cst)) return FASTEQ_INVALID;
  if (p->n_gate > 0 && !p->gated_dims) return FASTEQ_INVALID;
  int gated = 0;
  for (int k = 0; k < p->n_gate; ++k) gated += p->gated_dims[k];
  t->n_scalar = p->n_scalar; t->n_gate = p->n_gate;
  t->n_in = p->n_scalar + p->n_gate + gated; t->n_out = p->n_scalar + gated;
  if (t->n_in > kMaxSeg) return FASTEQ_UNSUPPORTED;
  for (int s = 0; s < t->n_in; ++s) { t->act[s] = 0; t->cst[s] = 1.0; t->gate_of[s] = -1; t->first_gated[s] = 0; t->n_gated[s] = 0; }
  for (int s = 0; s < p->n_scalar + p->n_gate; ++s) { t->act[s] = p->act[s]; t->cst[s] = p->cst[s]; }
  int pos = p->n_scalar + p->n_gate;
  for (int k = 0; k < p->n_gate; ++k) {
    const int g = p->n_scalar + k;
    t->first_gated[g] = pos; t->n_gated[g] = p->gated_dims[k];
    for (int m = 0; m < p->gated_dims[k]; ++m) t->gate_of[pos++] = g;
  }
  return FASTEQ_OK;
}
}  // namespace

extern "C" int fasteq_gate_forward(const fasteq_gate_problem* p, const void* x, void* out, fasteq_stream_t stream) {
  GateTable t; int rc = build(p, &t);
  if (rc != FASTEQ_OK) return rc;
  if (p->batch == 0) return FASTEQ_OK;
  if (!x || !out) return FASTEQ_INVALID;
  const long long total = p->batch * p->u;                     // one thread per (node, channel)
  if ((total + 255) / 256 > 0x7fffffffLL) return FASTEQ_UNSUPPORTED;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (p->dtype == FASTEQ_F32) gate_fwd_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)out, p->batch, p->u, t);
  else gate_fwd_kernel<double><<<blocks, 256, 0, (cudaStream_t)stream>>>((const double*)x, (double*)out, p->batch, p->u, t);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

extern "C" int fasteq_gate_backward(const fasteq_gate_problem* p, const void* x, const void* grad_out, void* grad_x,
                                    fasteq_stream_t stream) {
  GateTable t; int rc = build(p, &t);
  if (rc != FASTEQ_OK) return rc;
  if (p->batch == 0) return FASTEQ_OK;
  if (!x || !grad_out || !grad_x) return FASTEQ_INVALID;
  const long long total = p->batch * p->u;                     // one thread per (node, channel)
  if ((total + 255) / 256 > 0x7fffffffLL) return FASTEQ_UNSUPPORTED;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (p->dtype == FASTEQ_F32) gate_bwd_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((const float*)x, (const float*)grad_out, (float*)grad_x, p->batch, p->u, t);
  else gate_bwd_kernel<double><<<blocks, 256, 0, (cudaStream_t)stream>>>((const double*)x, (const double*)grad_out, (double*)grad_x, p->batch, p->u, t);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

extern "C" int fasteq_gate_double_backward(const fasteq_gate_problem* p, const void* x, const void* grad_out, const void* ggx,
                                           void* d_grad_out, void* d_x, fasteq_stream_t stream) {
  GateTable t; int rc = build(p, &t);
  if (rc != FASTEQ_OK) return rc;
  if (p->batch == 0) return FASTEQ_OK;
  if (!x || !grad_out || !ggx || !d_grad_out || !d_x) return FASTEQ_INVALID;
  auto blocks_for = [](long long total) { return (unsigned)((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32); };
  const long long n_out = p->batch * t.n_out * p->u, n_in = p->batch * t.n_in * p->u;
  cudaStream_t s = (cudaStream_t)stream;
  if (p->dtype == FASTEQ_F32) {
    gate_dbwd_go_kernel<float><<<blocks_for(n_out), 256, 0, s>>>((const float*)x, (const float*)ggx, (float*)d_grad_out, p->batch, p->u, t);
    gate_dbwd_x_kernel<float><<<blocks_for(n_in), 256, 0, s>>>((const float*)x, (const float*)grad_out, (const float*)ggx, (float*)d_x, p->batch, p->u, t);
  } else {
    gate_dbwd_go_kernel<double><<<blocks_for(n_out), 256, 0, s>>>((const double*)x, (const double*)ggx, (double*)d_grad_out, p->batch, p->u, t);
    gate_dbwd_x_kernel<double><<<blocks_for(n_in), 256, 0, s>>>((const double*)x, (const double*)grad_out, (const double*)ggx, (double*)d_x, p->batch, p->u, t);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}
