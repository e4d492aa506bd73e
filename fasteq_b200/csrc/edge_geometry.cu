// Edge geometry of a radius graph in one kernel per direction: edge vector, length and the radial basis
// (Bessel functions times a polynomial cutoff envelope) that feeds the radial MLP.
//
//   vec[e]    = (pos[src[e]] + shift[e]) - pos[dst[e]]
//   basis[e,n] = sqrt(2 / r_max) * sin((n + 1) pi r / r_max) / r * env(r / r_max)        n < n_basis
//   env(x)    = 1 - (p+1)(p+2)/2 x^p + p(p+2) x^(p+1) - p(p+1)/2 x^(p+2)   for x < 1, else 0
//
// (the basis of NequIP / MACE models, .../nequip/nn/embedding/_edge.py:174-189 and
// .../nequip/nn/embedding/cutoffs.py:17-27).  The backward takes dE/dvec and dE/dbasis, chains through
// the length and accumulates dE/dpos with red.global.add (senders and receivers).  These are the
// model-side elementwise steps around the hot path: about twenty framework launches otherwise.
#include <cstdint>
#include <cuda_runtime.h>
#include "fasteq_b200.h"
#include "core_common.h"
#include "fasteq_device.cuh"

using namespace fasteq;

namespace {

constexpr int kMaxBasis = 16;

template <typename T> struct Math;
template <> struct Math<float> {
  static __device__ __forceinline__ float sin_(float x) { return sinf(x); }
  static __device__ __forceinline__ float cos_(float x) { return cosf(x); }
  static __device__ __forceinline__ float sqrt_(float x) { return sqrtf(x); }
};
template <> struct Math<double> {
  static __device__ __forceinline__ double sin_(double x) { return sin(x); }
  static __device__ __forceinline__ double cos_(double x) { return cos(x); }
  static __device__ __forceinline__ double sqrt_(double x) { return sqrt(x); }
};

template <typename T>
__device__ __forceinline__ T ipow(T x, int n) {
  T r = T(1);
  for (int i = 0; i < n; ++i) r *= x;
  return r;
}

// envelope and its derivative with respect to x = r / r_max
template <typename T>
__device__ __forceinline__ void envelope(T x, int p, T& env, T& denv) {
  if (!(x < T(1))) { env = T(0); denv = T(0); return; }
  const T a = T(0.5) * (p + 1) * (p + 2), b = T(p) * (p + 2), c = T(0.5) * p * (p + 1);
  const T xp1 = ipow(x, p - 1), xp = xp1 * x;
  env = T(1) - a * xp + b * xp * x - c * xp * x * x;
  denv = -a * p * xp1 + b * (p + 1) * xp - c * (p + 2) * xp * x;
}

template <typename T>
__global__ void __launch_bounds__(256) edge_geometry_fwd_kernel(const T* __restrict__ pos, const int* __restrict__ src,
                                                                const int* __restrict__ dst, const T* __restrict__ shift,
                                                                long long n_edges, long long n_nodes, T r_max, int n_basis, int p,
                                                                T* __restrict__ vec, T* __restrict__ basis, int* status) {
  const T pi = T(3.14159265358979323846);
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n_edges; e += (long long)gridDim.x * blockDim.x) {
    const long long s = src[e], d = dst[e];
    if (s < 0 || s >= n_nodes || d < 0 || d >= n_nodes) {
      // an index outside the position array: record it, touch nothing through it, give the edge zero features
      atomicExch(status, 2);
      vec[3 * e] = vec[3 * e + 1] = vec[3 * e + 2] = T(0);
      for (int n = 0; n < n_basis; ++n) basis[e * n_basis + n] = T(0);
      continue;
    }
    T v[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) v[k] = (pos[3 * s + k] + shift[3 * e + k]) - pos[3 * d + k];
    vec[3 * e] = v[0]; vec[3 * e + 1] = v[1]; vec[3 * e + 2] = v[2];
    const T r = Math<T>::sqrt_(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
    T env, denv;
    envelope(r / r_max, p, env, denv);
    if (r > T(0)) {
      const T pref = Math<T>::sqrt_(T(2) / r_max) * env / r;
      for (int n = 0; n < n_basis; ++n) basis[e * n_basis + n] = pref * Math<T>::sin_((n + 1) * pi * r / r_max);
    } else {
      // coincident pair: the limit sin(k r) / r -> k (env(0) = 1); the gradient of that limit vanishes
      const T c0 = Math<T>::sqrt_(T(2) / r_max);
      for (int n = 0; n < n_basis; ++n) basis[e * n_basis + n] = c0 * (n + 1) * pi / r_max;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) edge_geometry_bwd_kernel(const T* __restrict__ pos, const int* __restrict__ src,
                                                                const int* __restrict__ dst, const T* __restrict__ shift,
                                                                const T* __restrict__ g_vec, const T* __restrict__ g_basis,
                                                                long long n_edges, long long n_nodes, T r_max, int n_basis, int p,
                                                                T* __restrict__ g_pos, int* status) {
  const T pi = T(3.14159265358979323846);
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n_edges; e += (long long)gridDim.x * blockDim.x) {
    const long long s = src[e], d = dst[e];
    if (s < 0 || s >= n_nodes || d < 0 || d >= n_nodes) { atomicExch(status, 2); continue; }
    T v[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) v[k] = (pos[3 * s + k] + shift[3 * e + k]) - pos[3 * d + k];
    T g[3] = {T(0), T(0), T(0)};
    if (g_vec) { g[0] = g_vec[3 * e]; g[1] = g_vec[3 * e + 1]; g[2] = g_vec[3 * e + 2]; }
    const T r = Math<T>::sqrt_(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
    if (g_basis && r > T(0)) {        // r == 0: the basis sits at its limit, whose gradient is zero
      T env, denv;
      envelope(r / r_max, p, env, denv);
      const T c0 = Math<T>::sqrt_(T(2) / r_max);
      // basis_n = c0 * sin(k_n r) * env / r ;  d/dr = c0 * [k_n cos(k_n r) env / r + sin(k_n r) (denv / r_max / r - env / r^2)]
      const T inv_r = T(1) / r;
      const T t1 = env * inv_r, t2 = denv / r_max * inv_r - env * inv_r * inv_r;
      T gr = T(0);
      for (int n = 0; n < n_basis; ++n) {
        const T k = (n + 1) * pi / r_max;
        gr += g_basis[e * n_basis + n] * c0 * (k * Math<T>::cos_(k * r) * t1 + Math<T>::sin_(k * r) * t2);
      }
      const T sc = gr * inv_r;
#pragma unroll
      for (int k = 0; k < 3; ++k) g[k] += sc * v[k];
    }
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      red_add(g_pos + 3 * s + k, g[k]);
      red_add(g_pos + 3 * d + k, -g[k]);
    }
  }
}

__device__ int g_geom_status;   // first fault of the edge-geometry kernels (2 = index outside the position array)

int* status_ptr() {
  int* p = nullptr;
  if (cudaGetSymbolAddress((void**)&p, g_geom_status) != cudaSuccess) return nullptr;
  return p;
}

long long grid_cap() {   // grid-stride loops: sixteen resident CTAs of 256 threads per SM
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 128;
  return (long long)sms * 16;
}

template <typename T>
int run_fwd(const void* pos, const int* src, const int* dst, const void* shift, long long E, long long N, double r_max, int nb, int p,
            void* vec, void* basis, cudaStream_t s) {
  int* st = status_ptr();
  if (!st) return FASTEQ_CUDA_ERROR;
  long long blocks = (E + 255) / 256; if (blocks > grid_cap()) blocks = grid_cap();
  edge_geometry_fwd_kernel<T><<<(unsigned)blocks, 256, 0, s>>>((const T*)pos, src, dst, (const T*)shift, E, N, (T)r_max, nb, p, (T*)vec,
                                                               (T*)basis, st);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

template <typename T>
int run_bwd(const void* pos, const int* src, const int* dst, const void* shift, const void* gv, const void* gb, long long E, long long N,
            double r_max, int nb, int p, void* gpos, cudaStream_t s) {
  cudaError_t e = cudaMemsetAsync(gpos, 0, (size_t)N * 3 * sizeof(T), s);
  if (e != cudaSuccess) return cuda_fail(e);
  if (E == 0) return FASTEQ_OK;
  int* st = status_ptr();
  if (!st) return FASTEQ_CUDA_ERROR;
  long long blocks = (E + 255) / 256; if (blocks > grid_cap()) blocks = grid_cap();
  edge_geometry_bwd_kernel<T><<<(unsigned)blocks, 256, 0, s>>>((const T*)pos, src, dst, (const T*)shift, (const T*)gv, (const T*)gb, E, N,
                                                               (T)r_max, nb, p, (T*)gpos, st);
  e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

}  // namespace

extern "C" int fasteq_edge_geometry_forward(int32_t dtype, const void* pos, const int32_t* src, const int32_t* dst, const void* shift,
                                            int64_t n_edges, int64_t n_nodes, double r_max, int32_t n_basis, int32_t envelope_p,
                                            void* vec, void* basis, fasteq_stream_t stream) {
  if (n_edges < 0 || n_nodes < 0 || n_basis < 1 || n_basis > kMaxBasis || envelope_p < 1 || !(r_max > 0.0)) return FASTEQ_INVALID;
  if (n_edges == 0) return FASTEQ_OK;
  if (!pos || !src || !dst || !shift || !vec || !basis) return FASTEQ_INVALID;
  if (dtype == FASTEQ_F32) return run_fwd<float>(pos, src, dst, shift, n_edges, n_nodes, r_max, n_basis, envelope_p, vec, basis, (cudaStream_t)stream);
  if (dtype == FASTEQ_F64) return run_fwd<double>(pos, src, dst, shift, n_edges, n_nodes, r_max, n_basis, envelope_p, vec, basis, (cudaStream_t)stream);
  return FASTEQ_INVALID;
}

extern "C" int fasteq_edge_geometry_backward(int32_t dtype, const void* pos, const int32_t* src, const int32_t* dst, const void* shift,
                                             const void* grad_vec, const void* grad_basis, int64_t n_edges, int64_t n_nodes,
                                             double r_max, int32_t n_basis, int32_t envelope_p, void* grad_pos,
                                             fasteq_stream_t stream) {
  if (n_edges < 0 || n_nodes < 0 || n_basis < 1 || n_basis > kMaxBasis || envelope_p < 1 || !(r_max > 0.0) || !grad_pos) return FASTEQ_INVALID;
  if (n_edges > 0 && (!pos || !src || !dst || !shift)) return FASTEQ_INVALID;
  if (dtype == FASTEQ_F32)
    return run_bwd<float>(pos, src, dst, shift, grad_vec, grad_basis, n_edges, n_nodes, r_max, n_basis, envelope_p, grad_pos, (cudaStream_t)stream);
  if (dtype == FASTEQ_F64)
    return run_bwd<double>(pos, src, dst, shift, grad_vec, grad_basis, n_edges, n_nodes, r_max, n_basis, envelope_p, grad_pos, (cudaStream_t)stream);
  return FASTEQ_INVALID;
}

extern "C" int fasteq_edge_geometry_device_status(int32_t* code) {
  if (!code) return FASTEQ_INVALID;
  int v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_geom_status, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaMemcpyToSymbol(g_geom_status, &zero, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  *code = v;
  return FASTEQ_OK;
}
