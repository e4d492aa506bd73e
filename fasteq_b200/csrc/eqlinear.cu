// SO3Linear (eqlinear) forward and grad_x as one grouped GEMM kernel: FP32 on the FMA pipe, FP64 on the tensor cores
// (DMMA) with the FMA kernel as the path for odd extents and unaligned operands.
//
//   C[b, c_row[g] + t, :] = sum_{q in group g} coeff[q] * A[b, a_row[q] + t, :] @ op(W[q])
//
// Forward: A = x, C = out, op = identity ([u, v]); paths are grouped by output row.
// grad_x : A = grad_out, C = grad_x, op = transpose; paths are grouped by input row.
// A "GEMM row" is one (batch entry, t) pair; the rows of a group are tiled 64 at a time, every
// CTA produces a 64 x 64 tile with 4 x 4 outputs per thread and walks K through shared memory.
// Reference semantics: test/test_eqlinear.py:38-69; problem / path layout
// fasteq/cuda/src/eqlinear/common/eqlinear_common.h:30-62.
#include <cstdio>
#include <cstdint>
#include <vector>
#include <algorithm>
#include <cuda_runtime.h>
#include "fasteq_b200.h"
#include "core_common.h"
#include "gemm_tf32x3.h"

using namespace fasteq;

namespace {

constexpr int kMaxPaths = 64;
constexpr int BM = 64, BN = 64, BK = 16, NT = 256;

struct GroupTable {
  int n_groups;
  int n_paths;
  int group_c_row[kMaxPaths];     // first row of C the group writes
  int group_rows[kMaxPaths];      // 2l+1
  int group_first[kMaxPaths + 1]; // paths of group g: [first[g], first[g+1])
  int path_a_row[kMaxPaths];
  int path_w[kMaxPaths];          // weight block
  float path_coeff_f[kMaxPaths];
  double path_coeff_d[kMaxPaths];
  long long tile_first[kMaxPaths + 1];  // prefix of row tiles per group
  long long wide_tile_first[kMaxPaths + 1];  // the same for the 128-row tiles of the FP64 tensor-core kernel
};

template <typename T> __device__ __forceinline__ T coeff_of(const GroupTable& t, int q);
template <> __device__ __forceinline__ float coeff_of<float>(const GroupTable& t, int q) { return t.path_coeff_f[q]; }
template <> __device__ __forceinline__ double coeff_of<double>(const GroupTable& t, int q) { return t.path_coeff_d[q]; }

// TRANS = false: W[q] is [K = u][N = v];  TRANS = true: W[q] is [N = u... stored [u][v]] used as [K = v][N = u]
template <typename T, bool TRANS>
__global__ void __launch_bounds__(NT) eqlinear_kernel(const __grid_constant__ GroupTable tab, const T* __restrict__ A,
                                                      const T* __restrict__ W, T* __restrict__ C, long long batch,
                                                      int a_rows_per_b, int c_rows_per_b, int K, int N, int u, int v) {
  __shared__ T sA[BK][BM + 4];
  __shared__ T sW[BK][BN + 4];
  // locate this CTA's (group, row tile)
  const long long tile = blockIdx.x;
  int g = 0;
  while (g + 1 < tab.n_groups && tile >= tab.tile_first[g + 1]) ++g;
  const long long row0 = (tile - tab.tile_first[g]) * BM;
  const int gi = tab.group_rows[g];
  const long long n_rows = batch * gi;
  const int n0 = blockIdx.y * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;   // 16 x 16 threads, 4 x 4 outputs each
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = T(0);

  // A tile [BM][BK]: thread loads elements (m = e*16 + tid/16, k = tid%16), 16 lanes along k (coalesced 64 B)
  const int lk = threadIdx.x % BK, lm0 = threadIdx.x / BK;
  size_t abase[4];
  bool avalid[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const long long r = row0 + e * (NT / BK) + lm0;
    avalid[e] = r < n_rows;
    const long long rb = avalid[e] ? r / gi : 0;
    const int rt = avalid[e] ? (int)(r % gi) : 0;
    abase[e] = ((size_t)rb * a_rows_per_b + rt) * (size_t)K;
  }

  for (int q = tab.group_first[g]; q < tab.group_first[g + 1]; ++q) {
    const T cq = coeff_of<T>(tab, q);
    const T* aq = A + (size_t)tab.path_a_row[q] * K;
    const T* wq = W + (size_t)tab.path_w[q] * u * v;
    T pacc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) pacc[i][j] = T(0);
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int k = k0 + lk;
        sA[lk][e * (NT / BK) + lm0] = (avalid[e] && k < K) ? aq[abase[e] + k] : T(0);
      }
      // W tile [BK][BN]: 1024 elements, 256 threads x 4
#pragma unroll
      for (int e = 0; e < (BK * BN) / NT; ++e) {
        const int idx = e * NT + threadIdx.x;
        const int k = idx / BN, n = idx % BN;
        T val = T(0);
        if (k0 + k < K && n0 + n < N)
          val = TRANS ? wq[(size_t)(n0 + n) * v + (k0 + k)] : wq[(size_t)(k0 + k) * v + (n0 + n)];
        sW[k][n] = val;
      }
      __syncthreads();
      // blocked summation: a chunk of BK products is summed on its own, then added to the path's
      // partial sum, which is scaled and added to the total -- the rounding error grows with the
      // square roots of the three lengths instead of with the full K * paths
      T part[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) part[i][j] = T(0);
#pragma unroll
      for (int k = 0; k < BK; ++k) {
        T a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = sA[k][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = sW[k][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) part[i][j] += a[i] * b[j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) pacc[i][j] += part[i][j];
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] += cq * pacc[i][j];
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long rr = row0 + ty * 4 + i;
    if (rr >= n_rows) continue;
    const long long b = rr / gi;
    const int t = (int)(rr % gi);
    T* crow = C + ((size_t)b * c_rows_per_b + tab.group_c_row[g] + t) * (size_t)N;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) crow[n] = acc[i][j];
    }
  }
}

// ------------------------------------------------------------------------------------------------
// FP64 on the tensor cores: the same grouped product with mma.sync m8n8k4 (DMMA), the FP64 tensor path of this part
// (tcgen05 has no FP64 kind; the reference's FP64 back-end is DMMA as well,
// fasteq/cuda/src/eqlinear/backends/fp64/direct_gemm_f64_tma.cu:204).  CTA tile 128 x 64, eight warps of 32 x 32
// (sixteen 8 x 8 accumulator tiles = 32 doubles per thread), two CTAs per SM so that one CTA's stores overlap the
// other's products.  Operands stream global -> shared memory through a DS-stage cp.async ring of DK-wide k-steps
// (16-byte copies, zero fill outside the problem), one barrier per step.
//
// A CTA owns one 128-row tile and a range of 64-column blocks.  When the tile's whole reduction (paths x K) is at most
// 64 wide, its A operand stays in shared memory across the column blocks ("stationary": the radial MLP's last layer
// multiplies [E, 64] by [64, 4352], so each row of A is read from HBM once instead of 68 times) and only W tiles (L2
// resident) move through the ring; otherwise A streams through the ring as well.
//
// Shared-memory pitches are 4 or 12 (mod 16) doubles, so the sixteen 8-byte fragment loads of a half warp hit sixteen
// different banks.  Fragment layout of m8n8k4.f64: a = A[lane / 4][lane % 4], b = B[lane % 4][lane / 4],
// c0, c1 = C[lane / 4][2 (lane % 4) + {0, 1}].  The path coefficient multiplies the A fragments, or the accumulators
// in the epilogue when all paths of the group share it.
constexpr int DM = 128, DN = 64;
constexpr int PW = DN + 4;                      // pitch of a W buffer [k][n]
constexpr int DMMA_MAX_STATIONARY_K = 64;

__device__ __forceinline__ void dmma_8x8x4(double (&c)[2], double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
               : "+d"(c[0]), "+d"(c[1]) : "d"(a), "d"(b));
}
// 16-byte asynchronous copy; `bytes` (0 or 16) of the source are read, the rest of the destination is zero
__device__ __forceinline__ void cp_async16(double* smem_dst, const double* gmem_src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

template <bool TRANS, int DK, int DS>
__global__ void __launch_bounds__(NT, 2) eqlinear_dmma_f64_kernel(const __grid_constant__ GroupTable tab, const double* __restrict__ A,
                                                                  const double* __restrict__ W, double* __restrict__ C, long long batch,
                                                                  int a_rows_per_b, int c_rows_per_b, int K, int N, int u, int v,
                                                                  int col_splits, int stationary) {
  constexpr int PA = DK + 4;                    // pitch of a streamed A buffer [row][k] and of a transposed W buffer [n][k]
  constexpr int W_BUF = DK * PW > DN * PA ? DK * PW : DN * PA;
  constexpr int CPR = DK / 2;                   // 16-byte chunks per row of a k-step
  extern __shared__ __align__(16) double dsm[];
  const long long tile = blockIdx.x / col_splits;
  const int split = blockIdx.x % col_splits;
  int g = 0;
  while (g + 1 < tab.n_groups && tile >= tab.wide_tile_first[g + 1]) ++g;
  const long long row0 = (tile - tab.wide_tile_first[g]) * DM;
  const int gi = tab.group_rows[g];
  const long long n_rows = batch * gi;
  const int q0 = tab.group_first[g], q1 = tab.group_first[g + 1];
  const int k_steps = (K + DK - 1) / DK;
  const int tile_steps = (q1 - q0) * k_steps;
  const int ncb = (N + DN - 1) / DN, per = (ncb + col_splits - 1) / col_splits;
  const int cb0 = split * per, cb1 = min(ncb, cb0 + per);
  if (cb0 >= cb1 || tile_steps == 0) return;
  const int total = (cb1 - cb0) * tile_steps;
  const int pitch_a = stationary ? tile_steps * DK + 4 : PA;
  double* sA = dsm;
  double* sW = dsm + (stationary ? DM * pitch_a : DS * DM * PA);

  bool uniform = true;
  for (int q = q0 + 1; q < q1; ++q) uniform = uniform && tab.path_coeff_d[q] == tab.path_coeff_d[q0];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = (warp & 3) * 32, wn = (warp >> 2) * 32;      // this warp's 32 x 32 corner of the tile
  const int fg = lane >> 2, ft = lane & 3;

  // copy roles.  A step: 128 rows x CPR chunks of two doubles; a thread copies chunk (tid % CPR) of rows tid / CPR + e * (NT / CPR).
  constexpr int A_PER = DM * CPR / NT, A_ROWS = NT / CPR;
  const int a_kc = (tid % CPR) * 2, a_r = tid / CPR;
  size_t a_off[A_PER];
  bool a_ok[A_PER];
#pragma unroll
  for (int e = 0; e < A_PER; ++e) {
    const long long ar = row0 + a_r + A_ROWS * e;
    a_ok[e] = ar < n_rows;
    a_off[e] = a_ok[e] ? ((size_t)(ar / gi) * a_rows_per_b + (size_t)(ar % gi)) * (size_t)K : 0;
  }
  // W step: DK x 64 doubles = DK * 32 chunks; [n][k] rows of the stored block when TRANS, else [k][n]
  constexpr int W_PER = DK * 32 / NT;
  const int w_r = TRANS ? (tid / CPR) : (tid >> 5);            // n (TRANS) or k
  const int w_c = TRANS ? (tid % CPR) * 2 : (tid & 31) * 2;    // k (TRANS) or n
  constexpr int W_RSTEP = TRANS ? NT / CPR : NT / 32;          // rows between a thread's chunks

  int i_cbl = 0, i_step = 0, i_q = q0, i_k0 = 0;            // the step the next issue() loads
  auto issue = [&](int flat) {
    if (flat < total) {
      if (!stationary || i_cbl == 0) {
        double* dst = stationary ? sA + i_step * DK : sA + (flat % DS) * (DM * PA);
        const double* aq = A + (size_t)tab.path_a_row[i_q] * K + i_k0 + a_kc;
        const bool kin = i_k0 + a_kc < K;
#pragma unroll
        for (int e = 0; e < A_PER; ++e) {
          const bool ok = a_ok[e] && kin;
          cp_async16(dst + (a_r + A_ROWS * e) * pitch_a + a_kc, ok ? aq + a_off[e] : A, ok ? 16 : 0);
        }
      }
      double* wd = sW + (flat % DS) * W_BUF;
      const double* wq = W + (size_t)tab.path_w[i_q] * u * v;
      const int n0 = (cb0 + i_cbl) * DN;
#pragma unroll
      for (int e = 0; e < W_PER; ++e) {
        const int r = w_r + W_RSTEP * e;
        if (TRANS) {
          const bool ok = n0 + r < N && i_k0 + w_c < K;
          cp_async16(wd + r * PA + w_c, ok ? wq + (size_t)(n0 + r) * v + i_k0 + w_c : W, ok ? 16 : 0);
        } else {
          const bool ok = i_k0 + r < K && n0 + w_c < N;
          cp_async16(wd + r * PW + w_c, ok ? wq + (size_t)(i_k0 + r) * v + n0 + w_c : W, ok ? 16 : 0);
        }
      }
      i_k0 += DK;
      if (i_k0 >= K) { i_k0 = 0; ++i_q; }
      if (++i_step == tile_steps) { i_step = 0; i_q = q0; ++i_cbl; }
    }
    cp_async_commit();
  };

  double acc[4][4][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

#pragma unroll
  for (int s = 0; s < DS - 1; ++s) issue(s);
  int cbl = 0, step = 0, q = q0, k0 = 0;
  for (int flat = 0; flat < total; ++flat) {
    cp_async_wait<DS - 2>();
    __syncthreads();                     // step `flat` has landed for every thread; the buffer of step flat - 1 is free
    issue(flat + DS - 1);
    const double* as = (stationary ? sA + step * DK : sA + (flat % DS) * (DM * PA)) + (wm + fg) * pitch_a + ft;
    const double* ws = sW + (flat % DS) * W_BUF + (TRANS ? (wn + fg) * PA + ft : ft * PW + wn + fg);
    const double cq = tab.path_coeff_d[q];
#pragma unroll
    for (int kk = 0; kk < DK; kk += 4) {
      double a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = as[8 * i * pitch_a + kk];
      if (!uniform) {
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] *= cq;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = TRANS ? ws[8 * j * PA + kk] : ws[kk * PW + 8 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) dmma_8x8x4(acc[i][j], a[i], b[j]);
    }
    k0 += DK;
    if (k0 >= K) { k0 = 0; ++q; }
    if (++step == tile_steps) {
      const double scale = uniform ? tab.path_coeff_d[q0] : 1.0;
      const int n0 = (cb0 + cbl) * DN;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const long long rr = row0 + wm + 8 * i + fg;
        double* crow = C + ((size_t)(rr / gi) * c_rows_per_b + tab.group_c_row[g] + (int)(rr % gi)) * (size_t)N;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n0 + wn + 8 * j + 2 * ft;      // even, and N is even: n < N covers n + 1
          if (rr < n_rows && n < N) *reinterpret_cast<double2*>(crow + n) = make_double2(scale * acc[i][j][0], scale * acc[i][j][1]);
          acc[i][j][0] = acc[i][j][1] = 0.0;
        }
      }
      step = 0; q = q0; ++cbl;
    }
  }
  cp_async_wait<0>();
}

// Launch geometry of the DMMA kernel: stationary A when every group's reduction fits, column blocks split over CTAs
// only as far as needed to fill the device twice over.
template <bool TRANS, int DK, int DS>
int launch_dmma(const GroupTable& tab, const fasteq_eqlinear_problem* p, const double* a, const double* w, double* c, int a_rows, int c_rows,
                int K, int N, cudaStream_t s) {
  const long long wt = tab.wide_tile_first[tab.n_groups];
  if (wt == 0) return FASTEQ_OK;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return cuda_fail(e);
  const int k_steps = (K + DK - 1) / DK, ncb = (N + DN - 1) / DN;
  int max_steps = 0;
  for (int g = 0; g < tab.n_groups; ++g) max_steps = std::max(max_steps, (tab.group_first[g + 1] - tab.group_first[g]) * k_steps);
  constexpr int PA = DK + 4, W_BUF = DK * PW > DN * PA ? DK * PW : DN * PA;
  const int stationary = max_steps * DK <= DMMA_MAX_STATIONARY_K ? 1 : 0;
  const long long want = (2LL * sms + wt - 1) / wt;
  const int col_splits = (int)std::min<long long>(ncb, std::max<long long>(1, want));
  if (wt * col_splits > 0x7fffffffLL) return FASTEQ_UNSUPPORTED;
  const size_t smem = sizeof(double) * ((stationary ? (size_t)DM * (max_steps * DK + 4) : (size_t)DS * DM * PA) + (size_t)DS * W_BUF);
  static bool raised[64] = {};
  if (dev < 64 && !raised[dev]) {
    const size_t most = std::max((size_t)DM * (DMMA_MAX_STATIONARY_K + 4), (size_t)DS * DM * PA) + (size_t)DS * W_BUF;
    e = cudaFuncSetAttribute(eqlinear_dmma_f64_kernel<TRANS, DK, DS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(double) * most));
    if (e != cudaSuccess) return cuda_fail(e);
    raised[dev] = true;
  } else if (dev >= 64) {
    return FASTEQ_UNSUPPORTED;
  }
  eqlinear_dmma_f64_kernel<TRANS, DK, DS><<<(unsigned)(wt * col_splits), NT, smem, s>>>(tab, a, w, c, p->batch, a_rows, c_rows, K, N, p->u, p->v,
                                                                               col_splits, stationary);
  e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

// Rows of C that no group writes must read as zero.  The uncovered rows form at most n_groups + 1 runs; every
// (batch entry, run) is one contiguous span of C, cleared with coalesced stores and no per-element index arithmetic.
struct GapTable {
  int n;
  int start[kMaxPaths + 1], len[kMaxPaths + 1];
};

template <typename T>
__global__ void __launch_bounds__(256) zero_gaps_kernel(T* __restrict__ C, long long batch, int c_rows_per_b, int N,
                                                        const __grid_constant__ GapTable gaps) {
  for (long long b = blockIdx.x; b < batch; b += gridDim.x)
    for (int g = 0; g < gaps.n; ++g) {
      T* p = C + ((size_t)b * c_rows_per_b + gaps.start[g]) * (size_t)N;
      const int n = gaps.len[g] * N;
      for (int i = threadIdx.x; i < n; i += blockDim.x) p[i] = T(0);
    }
}

template <typename T>
void zero_uncovered_rows(T* C, long long batch, int c_rows, int N, const GroupTable& tab, cudaStream_t s) {
  GapTable gaps; gaps.n = 0;
  int row = 0;                                      // groups are sorted by their first row and do not overlap
  for (int g = 0; g <= tab.n_groups; ++g) {
    const int next = g < tab.n_groups ? tab.group_c_row[g] : c_rows;
    if (next > row) { gaps.start[gaps.n] = row; gaps.len[gaps.n] = next - row; ++gaps.n; }
    if (g < tab.n_groups) row = tab.group_c_row[g] + tab.group_rows[g];
  }
  if (gaps.n == 0 || batch == 0) return;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 128;
  const long long blocks = batch < (long long)sms * 8 ? batch : (long long)sms * 8;
  zero_gaps_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(C, batch, c_rows, N, gaps);
}

int build_table(const fasteq_eqlinear_problem* p, bool dgrad, GroupTable* t, bool* covers_all) {
  if (!p || p->num_paths < 1 || p->num_paths > kMaxPaths || p->u < 1 || p->v < 1 || p->batch < 0) return FASTEQ_INVALID;
  if (!p->in_row || !p->out_row || !p->rows || !p->coeff) return FASTEQ_INVALID;
  const int P = p->num_paths;
  const int c_rows = dgrad ? p->in_rows : p->out_rows, a_rows = dgrad ? p->out_rows : p->in_rows;
  std::vector<int> order(P);
  for (int q = 0; q < P; ++q) order[q] = q;
  auto crow = [&](int q) { return dgrad ? p->in_row[q] : p->out_row[q]; };
  auto arow = [&](int q) { return dgrad ? p->out_row[q] : p->in_row[q]; };
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return crow(a) < crow(b); });
  t->n_groups = 0; t->n_paths = P;
  std::vector<char> covered(c_rows > 0 ? c_rows : 1, 0);
  for (int k = 0; k < P; ++k) {
    const int q = order[k];
    if (p->rows[q] < 1 || crow(q) < 0 || crow(q) + p->rows[q] > c_rows || arow(q) < 0 || arow(q) + p->rows[q] > a_rows)
      return FASTEQ_INVALID;
    if (t->n_groups == 0 || crow(q) != t->group_c_row[t->n_groups - 1]) {
      // groups must not overlap partially
      if (t->n_groups > 0 && crow(q) < t->group_c_row[t->n_groups - 1] + t->group_rows[t->n_groups - 1]) return FASTEQ_UNSUPPORTED;
      t->group_c_row[t->n_groups] = crow(q);
      t->group_rows[t->n_groups] = p->rows[q];
      t->group_first[t->n_groups] = k;
      ++t->n_groups;
      for (int r = 0; r < p->rows[q]; ++r) covered[crow(q) + r] = 1;
    } else if (p->rows[q] != t->group_rows[t->n_groups - 1]) {
      return FASTEQ_UNSUPPORTED;
    }
    t->path_a_row[k] = arow(q);
    t->path_w[k] = q;
    t->path_coeff_f[k] = (float)p->coeff[q];
    t->path_coeff_d[k] = p->coeff[q];
  }
  t->group_first[t->n_groups] = P;
  t->tile_first[0] = 0; t->wide_tile_first[0] = 0;
  for (int g = 0; g < t->n_groups; ++g) {
    t->tile_first[g + 1] = t->tile_first[g] + (p->batch * t->group_rows[g] + BM - 1) / BM;
    t->wide_tile_first[g + 1] = t->wide_tile_first[g] + (p->batch * t->group_rows[g] + 127) / 128;
  }
  *covers_all = true;
  for (int r = 0; r < c_rows; ++r) if (!covered[r]) *covers_all = false;
  return FASTEQ_OK;
}

template <typename T>
int launch(const fasteq_eqlinear_problem* p, bool dgrad, const void* w, const void* a, void* c, cudaStream_t s) {
  GroupTable tab; bool covers = true;
  int rc = build_table(p, dgrad, &tab, &covers);
  if (rc != FASTEQ_OK) return rc;
  if (p->batch == 0) return FASTEQ_OK;
  if (!w || !a || !c) return FASTEQ_INVALID;
  const int K = dgrad ? p->v : p->u, N = dgrad ? p->u : p->v;
  const int a_rows = dgrad ? p->out_rows : p->in_rows, c_rows = dgrad ? p->in_rows : p->out_rows;
  if (!covers) zero_uncovered_rows<T>((T*)c, p->batch, c_rows, N, tab, s);
  if (sizeof(T) == 8 && N >= 8 && (N % 2) == 0 && (K % 2) == 0 &&
      ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(c)) & 15u) == 0) {
    // FP64 on the tensor cores (DMMA); its 16-byte copies need even K and N and 16-byte aligned operands
    // k-steps of 8 through a four-deep ring; 16-wide steps and rings of two or three measured within 3 % of it
    return dgrad ? launch_dmma<true, 8, 4>(tab, p, (const double*)a, (const double*)w, (double*)c, a_rows, c_rows, K, N, s)
                 : launch_dmma<false, 8, 4>(tab, p, (const double*)a, (const double*)w, (double*)c, a_rows, c_rows, K, N, s);
  }
  const long long tiles = tab.tile_first[tab.n_groups];
  if (tiles > 0x7fffffffLL) return FASTEQ_UNSUPPORTED;
  dim3 grid((unsigned)tiles, (unsigned)((N + BN - 1) / BN));
  if (dgrad) eqlinear_kernel<T, true><<<grid, NT, 0, s>>>(tab, (const T*)a, (const T*)w, (T*)c, p->batch, a_rows, c_rows, K, N, p->u, p->v);
  else       eqlinear_kernel<T, false><<<grid, NT, 0, s>>>(tab, (const T*)a, (const T*)w, (T*)c, p->batch, a_rows, c_rows, K, N, p->u, p->v);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

// Bt[q][n][k] = coeff[q] * op(W[q])[k][n]: the K-major, pre-scaled weight blocks the tensor-core GEMM multiplies with,
// written as their two TF32 parts (hi: 10 mantissa bits, lo: the exact remainder).
// Forward: K = u, N = v (a transpose of W[q]); grad_x: K = v, N = u (W[q] as stored).
__global__ void pack_weights_kernel(const float* __restrict__ W, float* __restrict__ Bt_hi, float* __restrict__ Bt_lo,
                                    const __grid_constant__ GroupTable tab, int u, int v, bool dgrad) {
  const int K = dgrad ? v : u, N = dgrad ? u : v;
  const long long total = (long long)tab.n_paths * N * K;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % K), n = (int)((i / K) % N), q = (int)(i / ((long long)K * N));
    const float* wq = W + (size_t)tab.path_w[q] * u * v;
    const float val = tab.path_coeff_f[q] * (dgrad ? wq[(size_t)n * v + k] : wq[(size_t)k * v + n]);
    const float hi = __uint_as_float(__float_as_uint(val) & 0xffffe000u);
    Bt_hi[i] = hi;
    Bt_lo[i] = val - hi;
  }
}

// `packed` (optional): the output of pack_weights_kernel for this problem and direction, prepared earlier by
// fasteq_eqlinear_pack; when NULL the weights are packed into a stream-ordered temporary first.
int launch_tensorcore(const fasteq_eqlinear_problem* p, bool dgrad, const void* w, const void* packed, const void* a, void* c,
                      cudaStream_t s, bool* used) {
  *used = false;
  GroupTable tab; bool covers = true;
  int rc = build_table(p, dgrad, &tab, &covers);
  if (rc != FASTEQ_OK) return rc;
  const int K = dgrad ? p->v : p->u, N = dgrad ? p->u : p->v;
  const int a_rows = dgrad ? p->out_rows : p->in_rows, c_rows = dgrad ? p->in_rows : p->out_rows;
  if (p->batch == 0 || (!w && !packed) || !a || !c) return FASTEQ_OK;   // the FMA path reports the error / no-op
  if (!tc::supported(p->batch, a_rows, K, p->num_paths, N, c_rows, a, packed ? packed : w, c)) return FASTEQ_OK;
  tc::TcTable t{};
  t.n_groups = tab.n_groups; t.n_items = 0;
  for (int g = 0; g < tab.n_groups; ++g) {
    t.group_c_row[g] = tab.group_c_row[g]; t.group_first[g] = tab.group_first[g];
    t.item_first[g] = t.n_items; t.n_items += tab.group_rows[g];
  }
  t.group_first[tab.n_groups] = tab.group_first[tab.n_groups];
  t.item_first[tab.n_groups] = t.n_items;
  for (int q = 0; q < tab.n_paths; ++q) { t.path_a_row[q] = tab.path_a_row[q]; t.path_w[q] = q; }   // packed in table order
  float* bt = nullptr;
  const long long total = (long long)p->num_paths * N * K;
  if (!packed) {
    cudaError_t e = cudaMallocAsync((void**)&bt, (size_t)total * 2 * sizeof(float), s);
    if (e != cudaSuccess) return cuda_fail(e);
    pack_weights_kernel<<<(unsigned)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096), 256, 0, s>>>((const float*)w, bt, bt + total, tab, p->u, p->v, dgrad);
  }
  const float* hi = packed ? (const float*)packed : bt;
  if (!covers) zero_uncovered_rows<float>((float*)c, p->batch, c_rows, N, tab, s);
  rc = tc::launch(t, (const float*)a, p->batch, a_rows, K, hi, hi + total, p->num_paths, N, (float*)c, c_rows, s);
  if (bt) cudaFreeAsync(bt, s);
  if (rc == FASTEQ_OK) *used = true;
  return rc;
}

int pack_only(const fasteq_eqlinear_problem* p, bool dgrad, const void* w, void* packed, cudaStream_t s) {
  GroupTable tab; bool covers = true;
  int rc = build_table(p, dgrad, &tab, &covers);
  if (rc != FASTEQ_OK) return rc;
  if (!w || !packed) return FASTEQ_INVALID;
  if (p->precision != FASTEQ_EQLIN_TF32X3) return FASTEQ_UNSUPPORTED;
  const int K = dgrad ? p->v : p->u, N = dgrad ? p->u : p->v;
  const long long total = (long long)p->num_paths * N * K;
  pack_weights_kernel<<<(unsigned)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096), 256, 0, s>>>((const float*)w, (float*)packed, (float*)packed + total, tab, p->u, p->v, dgrad);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

int run_packed(const fasteq_eqlinear_problem* p, bool dgrad, const void* packed, const void* a, void* c, cudaStream_t s) {
  if (!p || !packed) return FASTEQ_INVALID;
  if (p->precision != FASTEQ_EQLIN_TF32X3) return FASTEQ_UNSUPPORTED;
  if (p->batch == 0) return FASTEQ_OK;
  if (!a || !c) return FASTEQ_INVALID;
  bool used = false;
  int rc = launch_tensorcore(p, dgrad, nullptr, packed, a, c, s, &used);
  if (rc != FASTEQ_OK) return rc;
  return used ? FASTEQ_OK : FASTEQ_UNSUPPORTED;      // shapes the tensor-core kernel does not take need the raw weights
}

// ------------------------------------------------------------------------------------------------
// Weight gradient: per path a [u, v] = X^T G product reduced over R = batch * rows GEMM rows.
// grid = (u tiles * v tiles, paths, splits); a CTA reduces its share of R into a 64 x 64 tile
// (chunks of BK rows summed on their own first, like the forward), writes it to partial[split] and
// a second kernel adds the splits in a fixed order and applies the coefficient.
struct WgradTable {
  int in_row[kMaxPaths], out_row[kMaxPaths], rows[kMaxPaths];
  double coeff[kMaxPaths];
};

template <typename T>
__global__ void __launch_bounds__(NT) eqlinear_wgrad_kernel(const __grid_constant__ WgradTable tab, const T* __restrict__ X,
                                                            const T* __restrict__ G, T* __restrict__ partial, long long batch,
                                                            int in_rows, int out_rows, int u, int v, int num_paths,
                                                            long long rows_per_split) {
  __shared__ T sX[BK][BM + 4];
  __shared__ T sG[BK][BN + 4];
  const int q = blockIdx.y;
  const int v_tiles = (v + BN - 1) / BN;
  const int m0 = (blockIdx.x / v_tiles) * BM, n0 = (blockIdx.x % v_tiles) * BN;
  const int gi = tab.rows[q];
  const long long R = batch * gi;
  const long long r_begin = (long long)blockIdx.z * rows_per_split;
  const long long r_end = r_begin + rows_per_split < R ? r_begin + rows_per_split : R;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = T(0);
  const int lc = threadIdx.x % 64, lr0 = threadIdx.x / 64;    // 64 consecutive threads read 64 consecutive channels
  for (long long r0 = r_begin; r0 < r_end; r0 += BK) {
#pragma unroll
    for (int e = 0; e < BK / 4; ++e) {
      const int k = e * 4 + lr0;
      const long long r = r0 + k;
      T xv = T(0), gv = T(0);
      if (r < r_end) {
        const long long b = r / gi;
        const int t = (int)(r % gi);
        if (m0 + lc < u) xv = X[((size_t)b * in_rows + tab.in_row[q] + t) * (size_t)u + m0 + lc];
        if (n0 + lc < v) gv = G[((size_t)b * out_rows + tab.out_row[q] + t) * (size_t)v + n0 + lc];
      }
      sX[k][lc] = xv; sG[k][lc] = gv;
    }
    __syncthreads();
    T part[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) part[i][j] = T(0);
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sX[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = sG[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) part[i][j] += a[i] * b[j];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
    __syncthreads();
  }
  T* dst = partial + ((size_t)blockIdx.z * num_paths + q) * (size_t)u * v;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= u) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < v) dst[(size_t)m * v + n] = acc[i][j];
    }
  }
}

template <typename T>
__global__ void eqlinear_wgrad_reduce_kernel(const __grid_constant__ WgradTable tab, const T* __restrict__ partial,
                                             T* __restrict__ gw, int splits, int num_paths, long long uv) {
  const long long total = (long long)num_paths * uv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    T s = T(0);
    for (int z = 0; z < splits; ++z) s += partial[(size_t)z * total + i];
    gw[i] = (T)tab.coeff[i / uv] * s;
  }
}

template <typename T>
int launch_wgrad(const fasteq_eqlinear_problem* p, const void* x, const void* go, void* gw, cudaStream_t s) {
  if (!p || p->num_paths < 1 || p->num_paths > kMaxPaths || p->u < 1 || p->v < 1 || p->batch < 0) return FASTEQ_INVALID;
  if (!p->in_row || !p->out_row || !p->rows || !p->coeff || !gw) return FASTEQ_INVALID;
  WgradTable tab;
  int max_rows = 1;
  for (int q = 0; q < p->num_paths; ++q) {
    if (p->rows[q] < 1 || p->in_row[q] < 0 || p->in_row[q] + p->rows[q] > p->in_rows || p->out_row[q] < 0 ||
        p->out_row[q] + p->rows[q] > p->out_rows)
      return FASTEQ_INVALID;
    tab.in_row[q] = p->in_row[q]; tab.out_row[q] = p->out_row[q]; tab.rows[q] = p->rows[q]; tab.coeff[q] = p->coeff[q];
    max_rows = std::max(max_rows, p->rows[q]);
  }
  const long long uv = (long long)p->u * p->v, total = uv * p->num_paths;
  if (p->batch == 0) {
    cudaError_t e = cudaMemsetAsync(gw, 0, (size_t)total * sizeof(T), s);
    return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
  }
  if (!x || !go) return FASTEQ_INVALID;
  const int tiles = ((p->u + BM - 1) / BM) * ((p->v + BN - 1) / BN);
  const long long R = p->batch * max_rows;
  // enough CTAs for a few waves of the SMs, but no split shorter than 256 GEMM rows
  long long splits = std::max<long long>(1, 1184 / ((long long)tiles * p->num_paths));
  splits = std::min<long long>(splits, std::max<long long>(1, R / 256));
  splits = std::min<long long>(splits, 1024);
  const long long rows_per_split = ((R + splits - 1) / splits + BK - 1) / BK * BK;
  T* partial = nullptr;
  cudaError_t e = cudaMallocAsync((void**)&partial, (size_t)splits * total * sizeof(T), s);
  if (e != cudaSuccess) return cuda_fail(e);
  dim3 grid((unsigned)tiles, (unsigned)p->num_paths, (unsigned)splits);
  eqlinear_wgrad_kernel<T><<<grid, NT, 0, s>>>(tab, (const T*)x, (const T*)go, partial, p->batch, p->in_rows, p->out_rows,
                                               p->u, p->v, p->num_paths, rows_per_split);
  const unsigned rb = (unsigned)std::min<long long>((total + 255) / 256, 2048);
  eqlinear_wgrad_reduce_kernel<T><<<rb, 256, 0, s>>>(tab, partial, (T*)gw, (int)splits, p->num_paths, uv);
  e = cudaGetLastError();
  cudaFreeAsync(partial, s);
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

int dispatch(const fasteq_eqlinear_problem* p, bool dgrad, const void* w, const void* a, void* c, fasteq_stream_t stream) {
  if (!p) return FASTEQ_INVALID;
  switch (p->precision) {
    case FASTEQ_EQLIN_FP64: return launch<double>(p, dgrad, w, a, c, (cudaStream_t)stream);
    case FASTEQ_EQLIN_TF32X3: {
      bool used = false;
      int rc = launch_tensorcore(p, dgrad, w, nullptr, a, c, (cudaStream_t)stream, &used);
      if (rc != FASTEQ_OK || used) return rc;
      return launch<float>(p, dgrad, w, a, c, (cudaStream_t)stream);   // shapes the tensor-core kernel does not take
    }
    case FASTEQ_EQLIN_FP32: return launch<float>(p, dgrad, w, a, c, (cudaStream_t)stream);
    default: return FASTEQ_INVALID;
  }
}

}  // namespace

extern "C" int fasteq_eqlinear_forward(const fasteq_eqlinear_problem* p, const void* w, const void* x, void* out,
                                       fasteq_stream_t stream) {
  return dispatch(p, false, w, x, out, stream);
}

extern "C" int fasteq_eqlinear_dgrad(const fasteq_eqlinear_problem* p, const void* w, const void* grad_out, void* grad_x,
                                     fasteq_stream_t stream) {
  return dispatch(p, true, w, grad_out, grad_x, stream);
}

extern "C" int fasteq_eqlinear_wgrad(const fasteq_eqlinear_problem* p, const void* x, const void* grad_out, void* grad_w,
                                     fasteq_stream_t stream) {
  if (!p) return FASTEQ_INVALID;
  if (p->precision == FASTEQ_EQLIN_FP64) return launch_wgrad<double>(p, x, grad_out, grad_w, (cudaStream_t)stream);
  if (p->precision == FASTEQ_EQLIN_TF32X3 || p->precision == FASTEQ_EQLIN_FP32)
    return launch_wgrad<float>(p, x, grad_out, grad_w, (cudaStream_t)stream);
  return FASTEQ_INVALID;
}

extern "C" int fasteq_eqlinear_pack(const fasteq_eqlinear_problem* p, int32_t dgrad, const void* w, void* packed,
                                    fasteq_stream_t stream) {
  return pack_only(p, dgrad != 0, w, packed, (cudaStream_t)stream);
}

extern "C" int fasteq_eqlinear_forward_packed(const fasteq_eqlinear_problem* p, const void* packed, const void* x, void* out,
                                              fasteq_stream_t stream) {
  return run_packed(p, false, packed, x, out, (cudaStream_t)stream);
}

extern "C" int fasteq_eqlinear_dgrad_packed(const fasteq_eqlinear_problem* p, const void* packed, const void* grad_out,
                                            void* grad_x, fasteq_stream_t stream) {
  return run_packed(p, true, packed, grad_out, grad_x, (cudaStream_t)stream);
}
