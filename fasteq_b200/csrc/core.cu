// libfasteq_b200_core: graph utilities and status reporting behind the C ABI of
// include/fasteq_b200.h.  (Spherical harmonics and SO3Linear entry points live in
// their own translation units of the same library.)
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "fasteq_b200.h"
#include "core_common.h"

namespace fasteq {
thread_local char g_cuda_err[256] = "";
int cuda_fail(cudaError_t e) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s", cudaGetErrorString(e));
  return FASTEQ_CUDA_ERROR;
}
}  // namespace fasteq
using namespace fasteq;

extern "C" const char* fasteq_status_string(int s) {
  switch (s) {
    case FASTEQ_OK: return "ok";
    case FASTEQ_UNSUPPORTED: return "unsupported shape or mode";
    case FASTEQ_INVALID: return "invalid argument";
    case FASTEQ_CUDA_ERROR: return "CUDA runtime error";
    case FASTEQ_INTERNAL: return "internal error";
    case FASTEQ_DEVICE_FAULT: return "device-side fault (wait timeout or index out of range)";
    default: return "unknown status";
  }
}
extern "C" const char* fasteq_last_cuda_error(void) { return g_cuda_err; }
extern "C" int fasteq_core_abi_version(void) { return FASTEQ_ABI_VERSION; }

// ---------------------------------------------------------------- sortedness
__global__ void check_sorted_kernel(const int* __restrict__ dst, long long n, int* flag) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  int bad = 0;
  for (; i + 1 < n; i += stride) bad |= (dst[i] > dst[i + 1]);
  if (bad) atomicExch(flag, 0);
}
__global__ void set_flag_kernel(int* flag, int v) { *flag = v; }

extern "C" int fasteq_graph_check_sorted(const int32_t* dst, int64_t n, int32_t* flag, fasteq_stream_t stream) {
  if (!flag || n < 0 || (n > 0 && !dst)) return FASTEQ_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  set_flag_kernel<<<1, 1, 0, s>>>(flag, 1);
  if (n > 1) {
    long long blocks = (n + 255) / 256;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
      sms = 128;
    if (blocks > (long long)sms * 8) blocks = (long long)sms * 8;     // grid-stride loop: eight resident CTAs per SM
    check_sorted_kernel<<<(int)blocks, 256, 0, s>>>(dst, n, flag);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

// ---------------------------------------------------------------- CSR offsets
// seg_ptr[r] = lower_bound(dst, r): one thread per row, binary search over the sorted index.
__global__ void build_csr_kernel(const int* __restrict__ dst, long long n_edges, long long n_rows, int* __restrict__ seg_ptr) {
  long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (r > n_rows) return;
  long long lo = 0, hi = n_edges;
  while (lo < hi) {
    long long mid = (lo + hi) >> 1;
    if ((long long)dst[mid] < r) lo = mid + 1; else hi = mid;
  }
  seg_ptr[r] = (int)lo;
}

extern "C" int fasteq_graph_build_csr(const int32_t* dst, int64_t n_edges, int64_t n_rows, int32_t* seg_ptr,
                                      fasteq_stream_t stream) {
  if (!seg_ptr || n_edges < 0 || n_rows < 0 || (n_edges > 0 && !dst)) return FASTEQ_INVALID;
  if (n_edges > 0x7fffffffLL || n_rows >= 0x7fffffffLL) return FASTEQ_UNSUPPORTED;
  const long long n = n_rows + 1;
  build_csr_kernel<<<(int)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(dst, n_edges, n_rows, seg_ptr);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

// ---------------------------------------------------------------- partition
__global__ void partition_kernel(const int* __restrict__ seg_ptr, long long n_rows, long long n_edges, int n_parts,
                                 int* __restrict__ part_ptr) {
  int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p > n_parts) return;
  if (p == n_parts) { part_ptr[p] = (int)n_rows; return; }
  // Work of a segment = its edges + 1 (an empty receiver still costs a row store).
  const long long total = n_edges + n_rows;
  const long long target = total * p / n_parts;
  long long lo = 0, hi = n_rows;
  while (lo < hi) {
    long long mid = (lo + hi) >> 1;
    if ((long long)seg_ptr[mid] + mid < target) lo = mid + 1; else hi = mid;
  }
  part_ptr[p] = (int)lo;
}

extern "C" int fasteq_graph_partition(const int32_t* seg_ptr, int64_t n_rows, int64_t n_edges, int32_t n_parts,
                                      int32_t* part_ptr, fasteq_stream_t stream) {
  if (!seg_ptr || !part_ptr || n_parts < 1 || n_rows < 0 || n_edges < 0) return FASTEQ_INVALID;
  partition_kernel<<<(n_parts + 1 + 255) / 256, 256, 0, (cudaStream_t)stream>>>(seg_ptr, n_rows, n_edges, n_parts, part_ptr);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}
