// Hidden layers of the radial MLP (width 64, SiLU) as ONE kernel per direction, so that the per-edge
// activations between the layers never leave the SM:
//
//   forward : b [E, nb] --W1 (CUDA cores)--> h1 = silu(z1) --W2 (tcgen05)--> h2 = silu(z2) --W3--> h3
//             writes h_L [E, 64] and d_l = silu'(z_l) for the tensor-core layers (kept for the backward)
//   backward: g = dE/dh_L;  g <- W_l^T (g * d_l) for l = L..2 (tcgen05);  gz1 = g * silu'(z1) with z1
//             recomputed from b;  dE/db = W1^T gz1  [E, nb]
//
// The radial network of MACE / NequIP models is a small bias-free MLP on the radial basis
// (.../nequip/nn/embedding/_edge.py:174-189 feeds it; the reference leaves the MLP to torch); here its
// 64 x 64 layers run as 3xTF32 tensor-core products (same split as gemm_tf32x3.cu) chained through
// shared memory and TMEM.
//
// One persistent CTA per SM walks tiles of 128 edges, two at a time ("slots"): while the tensor core works on one
// slot's layer the workers compute the other slot's activation, so neither the MMA round trip nor the
// activation arithmetic sits idle; both slots share the one operand region (it is only busy during an MMA) and
// have their own TMEM accumulator:
//   warp 0    : loads the pre-split hidden weights once (TMA, SWIZZLE_128B), they stay resident
//   warp 1    : issues the tcgen05.mma of a layer when the eight worker warps have written its operand
//   warps 2-9 : workers; a thread owns half a row of the tile (TMEM lane = row, 32 of the 64 columns):
//               it writes its part of the A operand (hi / lo, swizzled K-major) itself, reads the
//               accumulator back with tcgen05.ld and applies SiLU / the stored derivative.  Rows of
//               [E, 64] tensors enter and leave through per-warp 32 x 32 swizzled slabs and tiled TMA
//               loads / stores, so that global traffic is made of full 128-byte lines.
// Every mbarrier wait is bounded; a timeout sets a status word and the kernel drains.
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include "fasteq_b200.h"
#include "core_common.h"
#include "fasteq_device.cuh"
#include "gemm_tf32x3.h"
#include "tcgen05_util.cuh"

namespace fasteq {
namespace chain {

using namespace fasteq::tc;

constexpr int H = 64;                 // hidden width
constexpr int BM = 128, BK = 32;
constexpr int NT = 320;
constexpr int N_WORKERS = 8;          // worker warps
constexpr int MAX_TC = 2;             // tensor-core layers (hidden layers after the first)
constexpr int W_LAYER_BYTES = 2 * 2 * H * BK * 4;    // [kb][hi | lo] of a 64 x 64 matrix: 32 KB
constexpr int A_BYTES = 2 * 2 * BM * BK * 4;         // [kb][hi | lo] of a 128 x 64 tile: 64 KB
constexpr int SLAB_BYTES = 32 * 128;                 // 32 rows x 32 FP32 columns
constexpr int MAX_NB = 16;
constexpr int SMEM_BYTES = MAX_TC * W_LAYER_BYTES + A_BYTES + N_WORKERS * 2 * SLAB_BYTES + H * MAX_NB * 4 + 1024 /* barriers */ +
                           1024 /* alignment */;

struct Args {
  const float* basis;      // [M, nb]
  const float* w1;         // [H, nb]
  float* grad_basis;       // backward: dE/db [M, nb], zero-filled by the caller, accumulated with red.add
  long long M;
  int nb, n_tc;
};

__device__ __forceinline__ void silu_and_derivative(float z, float& h, float& d) {
  const float s = __fdividef(1.0f, 1.0f + __expf(-z));
  h = z * s;
  d = s * (1.0f + z * (1.0f - s));
}

// 16-byte chunk c of row r of a 128-byte-row tile sits at chunk position c ^ (r & 7) (SWIZZLE_128B)
__device__ __forceinline__ float4* swz(unsigned char* tile, int r, int c) {
  return reinterpret_cast<float4*>(tile + r * 128 + ((c ^ (r & 7)) << 4));
}

// this thread's 32 values (columns 32 * half ..) -> row `row` of k-block `half` of the A operand
__device__ __forceinline__ void write_operand(unsigned char* A, int half, int row, const float (&v)[32]) {
  unsigned char* hi_tile = A + half * (2 * BM * BK * 4);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    float4 hi, lo;
    split_tf32(v[4 * c + 0], hi.x, lo.x); split_tf32(v[4 * c + 1], hi.y, lo.y);
    split_tf32(v[4 * c + 2], hi.z, lo.z); split_tf32(v[4 * c + 3], hi.w, lo.w);
    *swz(hi_tile, row, c) = hi;
    *swz(hi_tile + BM * BK * 4, row, c) = lo;
  }
}

__device__ __forceinline__ void tma_store_block(const CUtensorMap* map, int col0, long long row0, int z, const void* slab) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
               ::"l"(map), "r"(col0), "r"((int)row0), "r"(z), "r"(smem_u32(slab)) : "memory");
}

// tmW: prepared weights; tmIO0 / tmIO1: forward = (h_L out, derivatives out), backward = (dE/dh_L in, derivatives in),
// all [z][M][64] FP32 with 32 x 32 boxes
template <int NB, bool BWD>
__global__ void __launch_bounds__(NT, 1)
radial_chain_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmIO0,
                    const __grid_constant__ CUtensorMap tmIO1, const __grid_constant__ Args a, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* w_base = smem;                                   // [MAX_TC][kb][hi 8 KB | lo 8 KB]
  unsigned char* a_base = smem + MAX_TC * W_LAYER_BYTES;          // [kb][hi 16 KB | lo 16 KB]
  unsigned char* slab_base = a_base + A_BYTES;                    // [8 warps][2][4 KB]
  float* w1s = reinterpret_cast<float*>(slab_base + N_WORKERS * 2 * SLAB_BYTES);   // [H][NB], zero padded
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(w1s) + H * MAX_NB * 4);
  uint64_t* w_full = bars;            // 1
  uint64_t* a_ready = bars + 1;       // [2 slots] the eight worker warps have written the slot's operand
  uint64_t* z_full = bars + 3;        // [2 slots] the slot's accumulator is complete
  uint64_t* slab_full = bars + 5;     // [8 warps][2] backward: a TMA load has landed in the slab
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5 + 2 * N_WORKERS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long n_tiles = (a.M + BM - 1) / BM;
  const int n_tc = a.n_tc;

  for (int i = threadIdx.x; i < H * NB; i += NT) {
    const int j = i / NB, k = i % NB;
    w1s[i] = k < a.nb ? a.w1[j * a.nb + k] : 0.f;
  }
  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int t = 0; t < 2; ++t) { mbar_init(&a_ready[t], N_WORKERS); mbar_init(&z_full[t], 1); }
    for (int i = 0; i < 2 * N_WORKERS; ++i) mbar_init(&slab_full[i], 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * H);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0 && n_tc > 0) {
      mbar_arrive_expect_tx(w_full, (uint32_t)(n_tc * W_LAYER_BYTES));
      for (int l = 0; l < n_tc; ++l)
        for (int kb = 0; kb < 2; ++kb)
          for (int hl = 0; hl < 2; ++hl)
            tma_load_3d(w_base + l * W_LAYER_BYTES + kb * (2 * H * BK * 4) + hl * (H * BK * 4), &tmW, kb * BK, 0, l * 2 + hl, w_full);
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tc > 0) {
      const uint32_t idesc = idesc_tf32_m128(H);
      mbar_wait(w_full, 0u, status);
      tc_fence_after();
      uint32_t cnt[2] = {0u, 0u};
      // two tiles ("slots") are in flight per CTA; the workers hand over operands in the fixed order
      // (slot 0, step s), (slot 1, step s), (slot 0, step s + 1), ... and both slots share the one operand region
      for (long long pair = 0;; ++pair) {
        const long long t0 = blockIdx.x + 2 * pair * gridDim.x;
        if (t0 >= n_tiles) break;
        const bool has1 = t0 + gridDim.x < n_tiles;
        for (int s = 0; s < n_tc; ++s) {
#pragma unroll
          for (int slot = 0; slot < 2; ++slot) {
            if (slot == 1 && !has1) continue;
            mbar_wait(&a_ready[slot], cnt[slot] & 1u, status);
            ++cnt[slot];
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + (uint32_t)(slot * H);
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
              const uint32_t a_hi = smem_u32(a_base + kb * (2 * BM * BK * 4)), a_lo = a_hi + BM * BK * 4;
              const uint32_t b_hi = smem_u32(w_base + s * W_LAYER_BYTES + kb * (2 * H * BK * 4)), b_lo = b_hi + H * BK * 4;
#pragma unroll
              for (int kk = 0; kk < BK / 8; ++kk) {
                const uint32_t off = kk * 32;
                mma_tf32(tmem_d, make_desc(a_lo + off), make_desc(b_hi + off), idesc, (kb | kk) ? 1u : 0u);
                mma_tf32(tmem_d, make_desc(a_hi + off), make_desc(b_lo + off), idesc, 1u);
                mma_tf32(tmem_d, make_desc(a_hi + off), make_desc(b_hi + off), idesc, 1u);
              }
            }
            mma_commit(&z_full[slot]);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ workers
    const int wk = warp - 2;                          // 0..7
    const int half = wk >> 2;                         // which 32 of the 64 columns
    const int quarter = warp & 3;                     // the TMEM lanes this warp may read
    const int trow = quarter * 32 + lane;             // row of the tile = TMEM lane
    const uint32_t tmem_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 32);
    unsigned char* slab[2] = {slab_base + wk * 2 * SLAB_BYTES, slab_base + wk * 2 * SLAB_BYTES + SLAB_BYTES};
    uint64_t* full[2] = {&slab_full[2 * wk], &slab_full[2 * wk + 1]};
    uint32_t n_full[2] = {0u, 0u}, n_z[2] = {0u, 0u}, n_store = 0;
    const int col0 = half * 32;

    // ---- backward: tiled TMA loads of [32 rows x 32 columns] blocks into this warp's two slabs.  Every block is
    // requested one phase before it is read: the blocks of a slot's start (dE/dh_L -> slab 0, top derivative ->
    // slab 1) while the other slot starts, the lower derivative of slot t (-> slab t) after both slots have started.
    auto request = [&](int which, const CUtensorMap* map, int z, long long row0) {
      fence_async_smem();                 // earlier generic reads of the slab precede the async write
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_expect_tx(full[which], SLAB_BYTES);
        tma_load_3d(slab[which], map, col0, (int)row0, z, full[which]);
      }
    };
    auto landed = [&](int which) { mbar_wait(full[which], n_full[which] & 1u, status); ++n_full[which]; };
    auto request_start = [&](long long row0) {          // the two blocks a slot's start reads
      request(0, &tmIO0, 0, row0);
      if (n_tc > 0) request(1, &tmIO1, n_tc - 1, row0);
    };
    // ---- forward: one 32 x 32 block leaves through the slabs (alternating) as a tiled TMA store
    auto store_block = [&](const float (&val)[32], const CUtensorMap* map, int z, long long row0) {
      unsigned char* sl = slab[n_store & 1u];
      if (lane == 0) bulk_wait_read<1>();     // the slab used two stores ago has been read
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 8; ++c) *swz(sl, lane, c) = make_float4(val[4 * c], val[4 * c + 1], val[4 * c + 2], val[4 * c + 3]);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (row0 < a.M) tma_store_block(map, col0, row0, z, sl);
        bulk_commit();
      }
      ++n_store;
    };
    auto load_basis = [&](float (&bb)[NB], long long row0, bool exists) {
      const long long r = row0 + lane;
#pragma unroll
      for (int k = 0; k < NB; ++k) bb[k] = (exists && r < a.M && k < a.nb) ? __ldg(a.basis + r * a.nb + k) : 0.f;
    };
    auto first_layer = [&](const float (&bb)[NB], int j, float& h, float& d) {
      float z = 0.f;
#pragma unroll
      for (int k = 0; k < NB; ++k) z = fmaf(w1s[(col0 + j) * NB + k], bb[k], z);
      silu_and_derivative(z, h, d);
    };
    auto hand_over = [&](int slot, const float (&val)[32]) {     // operand of the slot's next layer -> MMA warp
      write_operand(a_base, half, trow, val);
      fence_async_smem();              // generic-proxy writes -> visible to the tensor core's async proxy
      tc_fence_before();               // this thread's earlier accumulator reads precede the next MMA
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_ready[slot]);
    };
    auto accumulator = [&](int slot, uint32_t (&r)[32]) {        // waits for the slot's MMA, then reads its 32 columns
      mbar_wait(&z_full[slot], n_z[slot] & 1u, status);
      ++n_z[slot];
      tc_fence_after();
      tmem_ld_32(tmem_lane + (uint32_t)(slot * H), r);
    };

    const long long stride = (long long)gridDim.x * BM;
    long long row0_of[2];
    float b[2][NB], v[32];
    if (BWD && (long long)blockIdx.x < n_tiles) request_start((long long)blockIdx.x * BM + quarter * 32);
    for (long long pair = 0;; ++pair) {
      const long long t0 = blockIdx.x + 2 * pair * gridDim.x;
      if (t0 >= n_tiles) break;
      const bool has1 = t0 + gridDim.x < n_tiles;
      const bool has_next = t0 + 2 * gridDim.x < n_tiles;
      row0_of[0] = t0 * BM + quarter * 32;
      row0_of[1] = row0_of[0] + stride;
      load_basis(b[0], row0_of[0], true);
      load_basis(b[1], row0_of[1], has1);

      // start of a slot: the operand of the first tensor-core layer (or, without one, the final vector)
      auto start = [&](int slot) {
        if (!BWD) {
#pragma unroll
          for (int j = 0; j < 32; ++j) { float d; first_layer(b[slot], j, v[j], d); }
        } else {
          landed(0);
          if (n_tc > 0) landed(1);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float4 gv = *swz(slab[0], lane, c);
            if (n_tc > 0) {
              const float4 dv = *swz(slab[1], lane, c);
              gv.x *= dv.x; gv.y *= dv.y; gv.z *= dv.z; gv.w *= dv.w;
            }
            v[4 * c] = gv.x; v[4 * c + 1] = gv.y; v[4 * c + 2] = gv.z; v[4 * c + 3] = gv.w;
          }
          // both slabs are free: what is read next?
          if (slot == 0 && has1) request_start(row0_of[1]);
          else {
            // both slots have started (or there is only one): the lower derivatives, else the next pair's start
            if (n_tc > 1) {
              request(0, &tmIO1, n_tc - 2, row0_of[0]);
              if (has1) request(1, &tmIO1, n_tc - 2, row0_of[1]);
            } else if (has_next) {
              request_start(row0_of[0] + 2 * stride);
            }
          }
        }
      };
      // after tensor-core layer s of a slot: the operand of layer s + 1, or the final vector
      auto after_layer = [&](int slot, int s, const uint32_t (&r)[32]) {
        if (!BWD) {
          float d[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) silu_and_derivative(__uint_as_float(r[j]), v[j], d[j]);
          store_block(d, &tmIO1, s, row0_of[slot]);
        } else {
          const bool more = s + 1 < n_tc;      // multiply by the derivative of the layer below (n_tc <= 2: s == 0)
          if (more) landed(slot);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float4 dv = make_float4(1.f, 1.f, 1.f, 1.f);
            if (more) dv = *swz(slab[slot], lane, c);
            v[4 * c] = __uint_as_float(r[4 * c]) * dv.x; v[4 * c + 1] = __uint_as_float(r[4 * c + 1]) * dv.y;
            v[4 * c + 2] = __uint_as_float(r[4 * c + 2]) * dv.z; v[4 * c + 3] = __uint_as_float(r[4 * c + 3]) * dv.w;
          }
          // slab `slot` is free again: the next pair's start blocks go there (dE/dh_L into slab 0, derivative into slab 1)
          if (more && has_next) {
            if (slot == 0) request(0, &tmIO0, 0, row0_of[0] + 2 * stride);
            else request(1, &tmIO1, n_tc - 1, row0_of[0] + 2 * stride);
          }
        }
      };
      auto finish = [&](int slot) {
        if (!BWD) {
          store_block(v, &tmIO0, 0, row0_of[slot]);
        } else {
          float gb[NB];
#pragma unroll
          for (int k = 0; k < NB; ++k) gb[k] = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float h, d;
            first_layer(b[slot], j, h, d);
            const float gz = v[j] * d;
#pragma unroll
            for (int k = 0; k < NB; ++k) gb[k] = fmaf(gz, w1s[(col0 + j) * NB + k], gb[k]);
          }
          const long long row = row0_of[slot] + lane;
          if (row < a.M) {
            // the two half-row owners of an edge add into a zero-filled row: two addends, order-independent
#pragma unroll
            for (int k = 0; k < NB; ++k)
              if (k < a.nb) red_add(a.grad_basis + row * a.nb + k, gb[k]);
          }
        }
      };

      if (n_tc == 0) {
        start(0); finish(0);
        if (has1) { start(1); finish(1); }
        continue;
      }
      // slot 0's first operand goes to the tensor core; slot 1's is computed while that MMA runs
      start(0);
      hand_over(0, v);
      if (has1) start(1);
      for (int s = 0; s < n_tc; ++s) {
        uint32_t r[32];
        // here: MMA (slot 0, layer s) is in flight, v holds slot 1's operand for layer s
        accumulator(0, r);                       // the operand region is free again
        if (has1) hand_over(1, v);               // MMA (slot 1, layer s) starts
        after_layer(0, s, r);                    // ... and runs while slot 0's activation is computed
        if (s + 1 == n_tc) finish(0);
        if (has1) {
          accumulator(1, r);                     // the operand region is free again
          if (s + 1 < n_tc) hand_over(0, v);     // MMA (slot 0, layer s + 1) starts
          after_layer(1, s, r);
          if (s + 1 == n_tc) finish(1);
        } else if (s + 1 < n_tc) {
          hand_over(0, v);
        }
      }
    }
    if (!BWD && lane == 0) bulk_wait_read<0>();   // the slabs must outlive their stores
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * H);
  }
}

// prepared[l][hi | lo][r][c] = split(transpose ? W_l[c][r] : W_l[r][c]) for up to MAX_TC 64 x 64 matrices
__global__ void prepare_weights_kernel(const float* __restrict__ w0, const float* __restrict__ w1, int n, bool transpose,
                                       float* __restrict__ prepared) {
  const int total = n * H * H;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int l = i / (H * H), r = (i / H) % H, c = i % H;
    const float* w = l == 0 ? w0 : w1;
    const float v = transpose ? w[c * H + r] : w[r * H + c];
    float hi, lo;
    tc::split_tf32(v, hi, lo);
    prepared[(size_t)(l * 2) * H * H + r * H + c] = hi;
    prepared[(size_t)(l * 2 + 1) * H * H + r * H + c] = lo;
  }
}

__device__ int g_chain_status;

int device_status(int* code) {
  int v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_chain_status, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaMemcpyToSymbol(g_chain_status, &zero, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  *code = v;
  return FASTEQ_OK;
}

template <int NB, bool BWD>
static int launch_nb(const CUtensorMap& tmw, const CUtensorMap& io0, const CUtensorMap& io1, const Args& a, cudaStream_t s) {
  int* st = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&st, g_chain_status);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaFuncSetAttribute(radial_chain_kernel<NB, BWD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return cuda_fail(e);
  int dev = 0, sms = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return cuda_fail(e);
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return cuda_fail(e);
  const long long n_tiles = (a.M + BM - 1) / BM;
  const unsigned grid = (unsigned)(n_tiles < sms ? n_tiles : sms);
  radial_chain_kernel<NB, BWD><<<grid, NT, SMEM_BYTES, s>>>(tmw, io0, io1, a, st);
  e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

static int prepare(const float* const* w_hidden, int n_tc, bool bwd, float* prepared, cudaStream_t s) {
  if (n_tc < 1) return FASTEQ_OK;
  if (n_tc > MAX_TC) return FASTEQ_UNSUPPORTED;
  if (!w_hidden || !prepared) return FASTEQ_INVALID;
  for (int l = 0; l < n_tc; ++l)
    if (!w_hidden[l]) return FASTEQ_INVALID;
  // forward uses W_2, W_3 in order; backward uses W_L^T first
  const float* first = bwd ? w_hidden[n_tc - 1] : w_hidden[0];
  const float* second = n_tc > 1 ? (bwd ? w_hidden[0] : w_hidden[1]) : first;
  prepare_weights_kernel<<<n_tc * 4, 256, 0, s>>>(first, second, n_tc, bwd, prepared);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

// io0: forward h_L out / backward dE/dh_L in, [M, 64]; io1: derivatives [n_tc, M, 64] (out / in)
template <bool BWD>
static int run(Args a, const float* const* w_hidden, const float* prepared_in, const float* io0, const float* io1, cudaStream_t s) {
  if (a.M < 0 || a.nb < 1) return FASTEQ_INVALID;
  if (a.nb > MAX_NB || a.n_tc < 0 || a.n_tc > MAX_TC || a.M > 0x7fffffffLL - BM) return FASTEQ_UNSUPPORTED;
  if (a.M == 0) return FASTEQ_OK;
  if (!a.basis || !a.w1 || !io0 || (a.n_tc > 0 && ((!w_hidden && !prepared_in) || !io1)) || (BWD && !a.grad_basis)) return FASTEQ_INVALID;
  if ((reinterpret_cast<uintptr_t>(io0) | reinterpret_cast<uintptr_t>(io1) | reinterpret_cast<uintptr_t>(prepared_in)) & 15u)
    return FASTEQ_UNSUPPORTED;
  cudaError_t e;
  if (BWD) {
    e = cudaMemsetAsync(a.grad_basis, 0, (size_t)a.M * a.nb * sizeof(float), s);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  float* tmp = nullptr;
  alignas(64) CUtensorMap tmw, tm0, tm1;
  const int n_alloc = a.n_tc > 0 ? a.n_tc : 1;
  int rc = FASTEQ_OK;
  if (!prepared_in || a.n_tc == 0) {
    e = cudaMallocAsync((void**)&tmp, (size_t)n_alloc * 2 * H * H * sizeof(float), s);
    if (e != cudaSuccess) return cuda_fail(e);
    if (a.n_tc > 0) rc = prepare(w_hidden, a.n_tc, BWD, tmp, s);
  }
  const float* prepared = tmp ? tmp : prepared_in;
  if (rc == FASTEQ_OK)
    rc = tc::make_map(&tmw, prepared, (uint64_t)H, (uint64_t)H, (uint64_t)n_alloc * 2, (uint64_t)H, (uint64_t)H * H, BK, H, 1);
  if (rc == FASTEQ_OK) rc = tc::make_map(&tm0, io0, (uint64_t)H, (uint64_t)a.M, 1, (uint64_t)H, (uint64_t)a.M * H, 32, 32, 1);
  if (rc == FASTEQ_OK)
    rc = tc::make_map(&tm1, a.n_tc > 0 ? io1 : io0, (uint64_t)H, (uint64_t)a.M, (uint64_t)n_alloc, (uint64_t)H, (uint64_t)a.M * H, 32, 32, 1);
  if (rc == FASTEQ_OK) rc = a.nb <= 8 ? launch_nb<8, BWD>(tmw, tm0, tm1, a, s) : launch_nb<16, BWD>(tmw, tm0, tm1, a, s);
  if (tmp) cudaFreeAsync(tmp, s);
  return rc;
}

}  // namespace chain
}  // namespace fasteq

extern "C" int fasteq_radial_chain_forward(const float* basis, int64_t n_edges, int32_t n_basis, const float* w_first,
                                           const float* const* w_hidden, const float* prepared, int32_t n_hidden, float* out,
                                           float* deriv, fasteq_stream_t stream) {
  if (n_hidden < 1) return FASTEQ_INVALID;
  fasteq::chain::Args a{};
  a.basis = basis; a.w1 = w_first; a.M = n_edges; a.nb = n_basis; a.n_tc = n_hidden - 1;
  return fasteq::chain::run<false>(a, w_hidden, prepared, out, deriv, (cudaStream_t)stream);
}

extern "C" int fasteq_radial_chain_backward(const float* grad_out, const float* deriv, const float* basis, int64_t n_edges,
                                            int32_t n_basis, const float* w_first, const float* const* w_hidden,
                                            const float* prepared, int32_t n_hidden, float* grad_basis, fasteq_stream_t stream) {
  if (n_hidden < 1) return FASTEQ_INVALID;
  fasteq::chain::Args a{};
  a.basis = basis; a.w1 = w_first; a.grad_basis = grad_basis; a.M = n_edges; a.nb = n_basis; a.n_tc = n_hidden - 1;
  return fasteq::chain::run<true>(a, w_hidden, prepared, grad_out, deriv, (cudaStream_t)stream);
}

extern "C" int fasteq_radial_chain_prepare(const float* const* w_hidden, int32_t n_hidden, int32_t backward, float* prepared,
                                           fasteq_stream_t stream) {
  if (n_hidden < 1) return FASTEQ_INVALID;
  return fasteq::chain::prepare(w_hidden, n_hidden - 1, backward != 0, prepared, (cudaStream_t)stream);
}
