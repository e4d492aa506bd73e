// 3xTF32 grouped GEMM on the sm_100a tensor cores (tcgen05 + TMEM + TMA), used for the dense
// contractions of the path: SO3Linear forward / grad_x and the radial MLP layers.
//
//   C[b, c_row(item), n] = sum_{segments s of item} sum_k A[b, a_row(s), k] * Bt[w(s), n, k]
//
// A is a [M, rows_a, K] FP32 tensor (K contiguous), Bt a [P, N, K] FP32 tensor (K contiguous), C a
// [M, rows_c, N] FP32 tensor.  A plain GEMM is the case rows_a = rows_c = P = 1.
//
// Precision: each FP32 operand v is split into hi = v with the 13 low mantissa bits cleared (exact in
// TF32) and lo = v - hi (exact in FP32); the kernel accumulates hi*hi + hi*lo + lo*hi in FP32, which
// keeps the relative error near 2^-21 (the reference's tf32x3 scheme,
// fasteq/cuda/src/eqlinear/backends/tf32/shape_plan.cu:109-113: three MMAs, no lo*lo term).
//
// Structure of one CTA (persistent: one CTA per SM walks 128 x BN output tiles round-robin, the stage ring
// and two TMEM accumulators carry over from tile to tile so that loads, splits, MMAs and stores of
// neighbouring tiles overlap):
//   warp 0       : TMA producer -- 3-D tiled loads (SWIZZLE_128B) of the raw A and Bt k-blocks
//   warp 1       : allocates TMEM, issues tcgen05.mma (kind::tf32, M = 128, N = BN, K = 8) from one lane,
//                  releases ring stages and signals the epilogue with tcgen05.commit
//   warps 2..5   : split each raw k-block into hi / lo tiles: in place in shared memory at BN = 128 (the
//                  swizzle is position preserving), into tensor memory at BN = 64 (thread = row = TMEM
//                  lane, tcgen05.st; the MMAs then take their A operand from tensor memory)
//   warps 6..9   : read a finished accumulator with tcgen05.ld and store the tile through swizzled
//                  staging slabs and TMA stores
// Every mbarrier wait is bounded (about two seconds), after which a status word is set and the
// waiter falls through; TMEM is always released before the CTA ends.  Single-CTA copies only, no clusters.
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include "fasteq_b200.h"
#include "core_common.h"
#include "fasteq_device.cuh"
#include "gemm_tf32x3.h"
#include "tcgen05_util.cuh"

namespace fasteq {
namespace tc {

constexpr int BM = 128, BK = 32;
constexpr int NT = 192;     // A-stationary kernel: 6 warps
constexpr int NT_P = 320;   // persistent grouped kernel: 10 warps

template <int BN> struct Cfg {
  static constexpr int A_BYTES = BM * BK * 4;          // 16 KB
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  static constexpr int STAGES = (BN <= 64) ? 4 : 3;     // ring depth that fits the 227 KB of one CTA
  static constexpr int STORE_BYTES = 4 * 2 * 4096;     // per epilogue warp: two 32 x 32 FP32 slabs for the TMA stores
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STORE_BYTES + 1024 /* barriers */ + 1024 /* alignment slack */;
};

// one output tile of the persistent loop
struct Tile {
  int g, t, seg0, n_kb, n0;
  long long m0;
};

__device__ __forceinline__ Tile decode_tile(const TcTable& tab, long long tile, int m_tiles, int n_tiles, int kb_per_seg, int BN) {
  Tile r;
  const int mx = (int)(tile % m_tiles);
  const long long rest = tile / m_tiles;
  const int ny = (int)(rest % n_tiles);
  const int z = (int)(rest / n_tiles);
  int g = 0;
  while (g + 1 < tab.n_groups && z >= tab.item_first[g + 1]) ++g;
  r.g = g; r.t = z - tab.item_first[g];
  r.seg0 = tab.group_first[g];
  r.n_kb = (tab.group_first[g + 1] - r.seg0) * kb_per_seg;
  r.m0 = (long long)mx * BM; r.n0 = ny * BN;
  return r;
}

// A_TMEM (BN = 64, where tensor memory has room: accumulators 256 columns, A ring 4 x 64): the split warps write
// the hi / lo parts of a k-block to tensor memory (thread = row = TMEM lane, tcgen05.st) and the MMAs take A from
// there, which removes 32 KB of shared-memory writes and 32 KB of reads per k-block from the pipe that bounds the
// long-K case.
template <int BN, bool A_TMEM>
__global__ void __launch_bounds__(NT_P, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmBhi,
                   const __grid_constant__ CUtensorMap tmBlo, const __grid_constant__ CUtensorMap tmC,
                   const __grid_constant__ TcTable tab, long long M, int N, int K, long long n_tiles_total, int m_tiles,
                   int n_tiles, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using C_ = Cfg<BN>;
  constexpr int STAGES = C_::STAGES;
  constexpr uint32_t TMEM_COLS = A_TMEM ? 512u : (uint32_t)(4 * BN);
  static_assert(!A_TMEM || 4 * BN + STAGES * 2 * BK <= 512, "tensor memory: accumulators + A ring");
  unsigned char* stage_base = smem;
  unsigned char* store_base = smem + STAGES * C_::STAGE_BYTES;     // [4 warps][2 slabs][32 rows x 128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_base + C_::STORE_BYTES);
  uint64_t* full_raw = bars;                 // [STAGES] TMA landed
  uint64_t* full_split = bars + STAGES;      // [STAGES] hi / lo tiles ready
  uint64_t* empty = bars + 2 * STAGES;       // [STAGES] MMAs have consumed the stage
  uint64_t* acc_full = bars + 3 * STAGES;    // [2] accumulator complete
  uint64_t* acc_empty = acc_full + 2;        // [2] accumulator read back by the four epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_per_seg = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_raw[s], 1); mbar_init(&full_split[s], 4); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_a = tmem_base + (uint32_t)(4 * BN);     // A_TMEM: [STAGES][hi 32 columns | lo 32 columns]

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = 0;
      for (long long tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x) {
        const Tile tl = decode_tile(tab, tile, m_tiles, n_tiles, kb_per_seg, BN);
        // each tile starts its walk over the k-blocks at a different one, so that the CTAs do not all fetch the same
        // weight lines from L2 at the same moment (the terms of a sum are the same, their order depends on the tile)
        const int kb_start = (int)(tile % tl.n_kb);
        for (int kbi = 0; kbi < tl.n_kb; ++kbi, ++it) {
          const int kb = kbi + kb_start < tl.n_kb ? kbi + kb_start : kbi + kb_start - tl.n_kb;
          const int s = it % STAGES;
          mbar_wait(&empty[s], ((it / STAGES) & 1u) ^ 1u, status);
          unsigned char* st = stage_base + (size_t)s * C_::STAGE_BYTES;
          const int seg = tl.seg0 + kb / kb_per_seg;
          const int k0 = (kb % kb_per_seg) * BK;
          mbar_arrive_expect_tx(&full_raw[s], (uint32_t)(C_::A_BYTES + 2 * C_::B_BYTES));
          tma_load_3d(st, &tmA, k0, tab.path_a_row[seg] + tl.t, (int)tl.m0, &full_raw[s]);
          tma_load_3d(st + 2 * C_::A_BYTES, &tmBhi, k0, tl.n0, tab.path_w[seg], &full_raw[s]);
          tma_load_3d(st + 2 * C_::A_BYTES + C_::B_BYTES, &tmBlo, k0, tl.n0, tab.path_w[seg], &full_raw[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptors: D = F32, A = B = TF32, both K-major, M = 128; N = 2 BN for the product of
      // A_hi with the stacked [B_hi; B_lo] tile, N = BN for A_lo x B_hi
      const uint32_t idesc2 = idesc_tf32_m128(2 * BN), idesc1 = idesc_tf32_m128(BN);
      int it = 0;
      uint32_t lt = 0;
      for (long long tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x, ++lt) {
        const Tile tl = decode_tile(tab, tile, m_tiles, n_tiles, kb_per_seg, BN);
        const uint32_t buf = lt & 1u;
        mbar_wait(&acc_empty[buf], ((lt >> 1) & 1u) ^ 1u, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // columns [0, BN): hi x hi;  [BN, 2 BN): hi x lo + lo x hi (small terms, kept apart so that their
        // sum is not absorbed one rounding at a time into the large accumulator)
        const uint32_t tmem_d = tmem_base + buf * (uint32_t)(2 * BN);
        for (int kb = 0; kb < tl.n_kb; ++kb, ++it) {
          const int s = it % STAGES;
          mbar_wait(&full_split[s], (it / STAGES) & 1u, status);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_hi = smem_u32(stage_base + (size_t)s * C_::STAGE_BYTES);
          const uint32_t a_lo = a_hi + C_::A_BYTES;
          const uint32_t b_hi = a_hi + 2 * C_::A_BYTES;    // B_hi tile, B_lo tile right behind it
#pragma unroll
          for (int kk = 0; kk < BK / 8; ++kk) {
            const uint32_t off = kk * 32;   // 8 TF32 values = 32 bytes along K inside the 128-byte swizzle row
            if (A_TMEM) {
              const uint32_t ta = tmem_a + (uint32_t)(s * 2 * BK + kk * 8);
              mma_tf32_a_tmem(tmem_d, ta, make_desc(b_hi + off), idesc2, (kb | kk) ? 1u : 0u);
              mma_tf32_a_tmem(tmem_d + (uint32_t)BN, ta + (uint32_t)BK, make_desc(b_hi + off), idesc1, 1u);
            } else {
              mma_tf32(tmem_d, make_desc(a_hi + off), make_desc(b_hi + off), idesc2, (kb | kk) ? 1u : 0u);
              mma_tf32(tmem_d + (uint32_t)BN, make_desc(a_lo + off), make_desc(b_hi + off), idesc1, 1u);
            }
          }
          mma_commit(&empty[s]);            // the stage may be refilled once these MMAs have read it
        }
        mma_commit(&acc_full[buf]);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ split raw tiles into hi / lo
    const int tid = threadIdx.x - 64;     // 0..127
    int it = 0;
    for (long long tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x) {
      const Tile tl = decode_tile(tab, tile, m_tiles, n_tiles, kb_per_seg, BN);
      for (int kb = 0; kb < tl.n_kb; ++kb, ++it) {
        const int s = it % STAGES;
        mbar_wait(&full_raw[s], (it / STAGES) & 1u, status);
        unsigned char* st = stage_base + (size_t)s * C_::STAGE_BYTES;
        float4* a_hi = reinterpret_cast<float4*>(st);
        float4* a_lo = reinterpret_cast<float4*>(st + C_::A_BYTES);
        auto split = [](float4 v, float4& hi, float4& lo) {
          hi.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); lo.x = v.x - hi.x;
          hi.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); lo.y = v.y - hi.y;
          hi.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); lo.z = v.z - hi.z;
          hi.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); lo.w = v.w - hi.w;
        };
        if (A_TMEM) {
          // thread = row of the tile = its TMEM lane; 16-byte chunk j of row r sits at chunk position j ^ (r & 7)
          const int row = (warp & 3) * 32 + lane;
          uint32_t hi_bits[32], lo_bits[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 hi, lo; split(*reinterpret_cast<const float4*>(st + row * 128 + ((j ^ (row & 7)) << 4)), hi, lo);
            hi_bits[4 * j] = __float_as_uint(hi.x); hi_bits[4 * j + 1] = __float_as_uint(hi.y);
            hi_bits[4 * j + 2] = __float_as_uint(hi.z); hi_bits[4 * j + 3] = __float_as_uint(hi.w);
            lo_bits[4 * j] = __float_as_uint(lo.x); lo_bits[4 * j + 1] = __float_as_uint(lo.y);
            lo_bits[4 * j + 2] = __float_as_uint(lo.z); lo_bits[4 * j + 3] = __float_as_uint(lo.w);
          }
          const uint32_t ta = tmem_a + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(s * 2 * BK);
          tmem_st_32(ta, hi_bits);
          tmem_st_32(ta + (uint32_t)BK, lo_bits);
          tc_fence_before();
        } else {
#pragma unroll
          for (int i = 0; i < C_::A_BYTES / 16 / 128; ++i) {
            float4 hi, lo; split(a_hi[tid + i * 128], hi, lo);
            a_hi[tid + i * 128] = hi; a_lo[tid + i * 128] = lo;
          }
          fence_async_smem();               // generic-proxy writes -> visible to the tensor core's async proxy
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_split[s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 6..9)
    // TMEM lane = tile row; warp w may touch lanes 32 * (w % 4) .. + 31
    const int quarter = warp & 3;
    // registers -> swizzled staging slab of this warp -> one 32 x 32 TMA store per column chunk
    unsigned char* slab = store_base + (size_t)quarter * 2 * 4096;
    uint32_t lt = 0;
    int chunk_no = 0;
    for (long long tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x, ++lt) {
      const Tile tl = decode_tile(tab, tile, m_tiles, n_tiles, kb_per_seg, BN);
      const uint32_t buf = lt & 1u;
      mbar_wait(&acc_full[buf], (lt >> 1) & 1u, status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int c_row = tab.group_c_row[tl.g] + tl.t;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c, ++chunk_no) {
        uint32_t r[32], q[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * (uint32_t)(2 * BN) + (uint32_t)(c * 32);
        tmem_ld_32(taddr, r);                      // hi x hi
        tmem_ld_32(taddr + (uint32_t)BN, q);       // hi x lo + lo x hi
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(q[j]));
        unsigned char* sl = slab + (size_t)(chunk_no & 1) * 4096;
        if (lane == 0) bulk_wait_read<1>();     // the slab used two chunks ago has been read by its store
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          *reinterpret_cast<float4*>(sl + lane * 128 + ((j ^ (lane & 7)) << 4)) =
              make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int col0 = tl.n0 + c * 32;
          const long long row0 = tl.m0 + quarter * 32;
          if (col0 < N && row0 < M) {
            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                         ::"l"(&tmC), "r"(col0), "r"(c_row), "r"((int)row0), "r"(smem_u32(sl)) : "memory");
          }
          bulk_commit();
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (lane == 0) bulk_wait_read<0>();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// "A-stationary" variant for a shallow, wide layer (K <= 128, many N tiles: the last layer of the radial
// MLP, 64 -> weight_numel).  One CTA owns a 128-row block of A, loads and splits it once, then walks
// all N tiles: pre-split weight tiles (hi / lo arrays prepared once per call) stream through a ring,
// two TMEM accumulators alternate so that the MMAs of tile n+1 overlap the stores of tile n.
constexpr int AS_BN = 128, AS_RING = 4, AS_MAX_KB = 4;

template <int KB>
struct AsCfg {
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = AS_BN * BK * 4;
  static constexpr int RING = (KB <= 2) ? AS_RING : 2;
  static constexpr int STORE_BYTES = 4 * 2 * 4096;    // per epilogue warp: two 32 x 32 FP32 slabs for the TMA stores
  static constexpr int SMEM_BYTES = KB * 2 * A_BYTES + RING * 2 * B_BYTES + STORE_BYTES + 1024 + 1024;
};

template <int KB>
__global__ void __launch_bounds__(NT, 1)
gemm_tf32x3_as_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmBhi,
                      const __grid_constant__ CUtensorMap tmBlo, const __grid_constant__ CUtensorMap tmC, long long M, int N, int K,
                      int* status) {
  using C_ = AsCfg<KB>;
  constexpr int RING = C_::RING;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* a_base = smem;                                   // [KB][hi 16 KB | lo 16 KB]
  unsigned char* b_base = smem + KB * 2 * C_::A_BYTES;            // [RING][hi 16 KB | lo 16 KB]
  unsigned char* store_base = b_base + RING * 2 * C_::B_BYTES;    // [4 warps][2 slabs][32 rows x 128 B], 1024-aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_base + C_::STORE_BYTES);
  uint64_t* a_full = bars;            // 1
  uint64_t* a_split = bars + 1;       // 4 warps
  uint64_t* b_full = bars + 2;        // [RING]
  uint64_t* b_empty = b_full + RING;  // [RING]
  uint64_t* acc_full = b_empty + RING;   // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long m0 = (long long)blockIdx.x * BM;
  const int n_tiles = (N + AS_BN - 1) / AS_BN;
  const int n_kb = (K + BK - 1) / BK;            // <= KB

  if (threadIdx.x == 0) {
    mbar_init(a_full, 1); mbar_init(a_split, 4);
    for (int s = 0; s < RING; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(a_full, (uint32_t)(n_kb * C_::A_BYTES));
      for (int kb = 0; kb < n_kb; ++kb) tma_load_3d(a_base + (size_t)kb * 2 * C_::A_BYTES, &tmA, kb * BK, 0, (int)m0, a_full);
      int it = 0;
      for (int nt = 0; nt < n_tiles; ++nt) {
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % RING;
          mbar_wait(&b_empty[s], ((it / RING) & 1u) ^ 1u, status);
          unsigned char* st = b_base + (size_t)s * 2 * C_::B_BYTES;
          mbar_arrive_expect_tx(&b_full[s], (uint32_t)(2 * C_::B_BYTES));
          tma_load_3d(st, &tmBhi, kb * BK, nt * AS_BN, 0, &b_full[s]);
          tma_load_3d(st + C_::B_BYTES, &tmBlo, kb * BK, nt * AS_BN, 0, &b_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(AS_BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      mbar_wait(a_split, 0u, status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      int it = 0;
      for (int nt = 0; nt < n_tiles; ++nt) {
        const int buf = nt & 1;
        mbar_wait(&acc_empty[buf], (((uint32_t)nt >> 1) & 1u) ^ 1u, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * AS_BN);
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % RING;
          mbar_wait(&b_full[s], (it / RING) & 1u, status);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_hi = smem_u32(a_base + (size_t)kb * 2 * C_::A_BYTES), a_lo = a_hi + C_::A_BYTES;
          const uint32_t b_hi = smem_u32(b_base + (size_t)s * 2 * C_::B_BYTES), b_lo = b_hi + C_::B_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 8; ++kk) {
            const uint32_t off = kk * 32;
            mma_tf32(tmem_d, make_desc(a_lo + off), make_desc(b_hi + off), idesc, (kb | kk) ? 1u : 0u);
            mma_tf32(tmem_d, make_desc(a_hi + off), make_desc(b_lo + off), idesc, 1u);
            mma_tf32(tmem_d, make_desc(a_hi + off), make_desc(b_hi + off), idesc, 1u);
          }
          mma_commit(&b_empty[s]);
        }
        mma_commit(&acc_full[buf]);
      }
    }
  } else {
    const int tid = threadIdx.x - 64;
    mbar_wait(a_full, 0u, status);
    for (int kb = 0; kb < n_kb; ++kb) {
      float4* hi = reinterpret_cast<float4*>(a_base + (size_t)kb * 2 * C_::A_BYTES);
      float4* lo = reinterpret_cast<float4*>(a_base + (size_t)kb * 2 * C_::A_BYTES + C_::A_BYTES);
#pragma unroll
      for (int i = 0; i < C_::A_BYTES / 16 / 128; ++i) {
        const float4 v = hi[tid + i * 128];
        float4 h, l;
        h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); l.x = v.x - h.x;
        h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); l.y = v.y - h.y;
        h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); l.z = v.z - h.z;
        h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); l.w = v.w - h.w;
        hi[tid + i * 128] = h; lo[tid + i * 128] = l;
      }
    }
    fence_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(a_split);
    const int quarter = warp & 3;
    // this warp's 32 rows leave through its own pair of staging slabs: registers -> swizzled shared
    // memory -> one 32 x 32 TMA store per column chunk (full 128-byte lines, clipped at the edges of C)
    unsigned char* slab = store_base + (size_t)quarter * 2 * 4096;
    int chunk_no = 0;
    for (int nt = 0; nt < n_tiles; ++nt) {
      const int buf = nt & 1;
      mbar_wait(&acc_full[buf], ((uint32_t)nt >> 1) & 1u, status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c = 0; c < AS_BN / 32; ++c, ++chunk_no) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * AS_BN + c * 32);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
              "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
              "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        unsigned char* sl = slab + (size_t)(chunk_no & 1) * 4096;
        // the slab used two chunks ago must have been read by its store
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // SWIZZLE_128B: 16-byte chunk j of row `lane` sits at chunk position j ^ (lane & 7)
          *reinterpret_cast<float4*>(sl + lane * 128 + ((j ^ (lane & 7)) << 4)) =
              make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int col0 = nt * AS_BN + c * 32;
          const long long row0 = m0 + quarter * 32;
          if (col0 < N && row0 < M) {
            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                         ::"l"(&tmC), "r"(col0), "r"((int)row0), "r"(0), "r"(smem_u32(sl)) : "memory");
          }
          bulk_commit();
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (lane == 0) bulk_wait_read<0>();   // the staging slabs must outlive their stores
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// Persistent form of the A-stationary kernel for K <= 64: one CTA per SM walks row blocks round-robin, and the
// A block lives in TENSOR MEMORY.  Shared-memory bandwidth is the busiest resource of this shape (every
// 128 x 128 x 8 TF32 MMA with both operands in shared memory reads 8 KB), so four warps split each raw A block
// (thread = row = TMEM lane) into hi / lo and write both with tcgen05.st; the MMAs then take A from tensor memory
// and only the weight tile from shared memory.  A is double buffered (raw tile in shared memory and hi / lo in
// tensor memory) and the two accumulators alternate across block boundaries, so the load / split prologue and
// the store tail of a block hide behind its neighbours' MMAs.
//   warp 0: TMA producer (A blocks, weight tiles)   warp 1: tcgen05.mma issue   warps 2-5: hi / lo split of A
//   warps 6-9: accumulator read-back and TMA stores
// Tensor memory (512 columns): accumulators [0, 256); A buffer b at 256 + 128 b: hi [0, 64), lo [64, 128).
// Writing the accumulator rows straight from registers (32-byte st.global per thread) instead of staging them
// for TMA stores was measured slower: row-scattered sectors cost more than the staging.
constexpr int NT_ASP = 320;

struct AspCfg {
  static constexpr int KB = 2;
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int A_BUF = KB * A_BYTES;             // raw FP32 block, [KB][16 KB]
  static constexpr int B_BYTES = AS_BN * BK * 4;
  static constexpr int RING = 4;
  static constexpr int STORE_BYTES = 4 * 2 * 4096;
  static constexpr int SMEM_BYTES = 2 * A_BUF + RING * 2 * B_BYTES + STORE_BYTES + 1024 + 1024;
  static constexpr uint32_t TMEM_COLS = 512, TMEM_A0 = 256, TMEM_A_STRIDE = 128, TMEM_A_LO = 64;
};

__global__ void __launch_bounds__(NT_ASP, 1)
gemm_tf32x3_asp_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmBhi,
                       const __grid_constant__ CUtensorMap tmBlo, const __grid_constant__ CUtensorMap tmC, long long M, int N, int K,
                       int m_blocks, int* status) {
  using C_ = AspCfg;
  constexpr int RING = C_::RING;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* a_base = smem;                                   // [2 buffers][KB][raw 16 KB]
  unsigned char* b_base = smem + 2 * C_::A_BUF;                   // [RING][hi 16 KB | lo 16 KB]
  unsigned char* store_base = b_base + RING * 2 * C_::B_BYTES;    // [4 warps][2 slabs][32 rows x 128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_base + C_::STORE_BYTES);
  uint64_t* a_full = bars;              // [2] raw A block landed
  uint64_t* a_split = bars + 2;         // [2] hi / lo are in tensor memory (four split warps)
  uint64_t* a_raw_empty = bars + 4;     // [2] the split warps have read the raw block
  uint64_t* a_tmem_empty = bars + 6;    // [2] the MMAs of the block have completed
  uint64_t* b_full = bars + 8;          // [RING]
  uint64_t* b_empty = b_full + RING;    // [RING]
  uint64_t* acc_full = b_empty + RING;  // [2]
  uint64_t* acc_empty = acc_full + 2;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (N + AS_BN - 1) / AS_BN;
  const int n_kb = (K + BK - 1) / BK;            // <= KB
  const int first = (int)blockIdx.x, stride = (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&a_full[b], 1); mbar_init(&a_split[b], 4); mbar_init(&a_raw_empty[b], 4); mbar_init(&a_tmem_empty[b], 1);
      mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4);
    }
    for (int s = 0; s < RING; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, C_::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      auto load_a = [&](int j, int blk) {
        const int buf = j & 1;
        mbar_wait(&a_raw_empty[buf], (((uint32_t)j >> 1) & 1u) ^ 1u, status);
        unsigned char* dst = a_base + (size_t)buf * C_::A_BUF;
        mbar_arrive_expect_tx(&a_full[buf], (uint32_t)(n_kb * C_::A_BYTES));
        for (int kb = 0; kb < n_kb; ++kb) tma_load_3d(dst + (size_t)kb * C_::A_BYTES, &tmA, kb * BK, 0, blk * BM, &a_full[buf]);
      };
      if (first < m_blocks) load_a(0, first);
      int it = 0;
      for (int j = 0, blk = first; blk < m_blocks; ++j, blk += stride) {
        bool next_pending = blk + stride < m_blocks;
        int local = 0;
        for (int nti = 0; nti < n_tiles; ++nti) {
          const int nt = (nti + blk) % n_tiles;     // staggered walk over the weight tiles (see the epilogue)
          for (int kb = 0; kb < n_kb; ++kb, ++it, ++local) {
            // the next A block is requested once this block's first weight tiles are on their way
            if (next_pending && local == 2) { load_a(j + 1, blk + stride); next_pending = false; }
            const int s = it % RING;
            mbar_wait(&b_empty[s], ((it / RING) & 1u) ^ 1u, status);
            unsigned char* st = b_base + (size_t)s * 2 * C_::B_BYTES;
            mbar_arrive_expect_tx(&b_full[s], (uint32_t)(2 * C_::B_BYTES));
            tma_load_3d(st, &tmBhi, kb * BK, nt * AS_BN, 0, &b_full[s]);
            tma_load_3d(st + C_::B_BYTES, &tmBlo, kb * BK, nt * AS_BN, 0, &b_full[s]);
          }
        }
        if (next_pending) load_a(j + 1, blk + stride);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = idesc_tf32_m128(AS_BN);
      int it = 0;
      uint32_t t = 0;
      for (int j = 0, blk = first; blk < m_blocks; ++j, blk += stride) {
        const int abuf = j & 1;
        mbar_wait(&a_split[abuf], ((uint32_t)j >> 1) & 1u, status);
        tc_fence_after();
        const uint32_t a_hi0 = tmem_base + C_::TMEM_A0 + (uint32_t)abuf * C_::TMEM_A_STRIDE, a_lo0 = a_hi0 + C_::TMEM_A_LO;
        for (int nt = 0; nt < n_tiles; ++nt, ++t) {
          const uint32_t buf = t & 1u;
          mbar_wait(&acc_empty[buf], ((t >> 1) & 1u) ^ 1u, status);
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + buf * AS_BN;
          for (int kb = 0; kb < n_kb; ++kb, ++it) {
            const int s = it % RING;
            mbar_wait(&b_full[s], (it / RING) & 1u, status);
            tc_fence_after();
            const uint32_t b_hi = smem_u32(b_base + (size_t)s * 2 * C_::B_BYTES), b_lo = b_hi + C_::B_BYTES;
#pragma unroll
            for (int kk = 0; kk < BK / 8; ++kk) {
              const uint32_t off = kk * 32, col = (uint32_t)(kb * BK + kk * 8);
              mma_tf32_a_tmem(tmem_d, a_lo0 + col, make_desc(b_hi + off), idesc, (kb | kk) ? 1u : 0u);
              mma_tf32_a_tmem(tmem_d, a_hi0 + col, make_desc(b_lo + off), idesc, 1u);
              mma_tf32_a_tmem(tmem_d, a_hi0 + col, make_desc(b_hi + off), idesc, 1u);
            }
            mma_commit(&b_empty[s]);
          }
          mma_commit(&acc_full[buf]);
        }
        mma_commit(&a_tmem_empty[abuf]);
      }
    }
  } else if (warp < 6) {
    // thread = row of the block = its TMEM lane; 16-byte chunk q of row r sits at chunk position q ^ (r & 7)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    for (int j = 0, blk = first; blk < m_blocks; ++j, blk += stride) {
      const int abuf = j & 1;
      mbar_wait(&a_full[abuf], ((uint32_t)j >> 1) & 1u, status);
      mbar_wait(&a_tmem_empty[abuf], (((uint32_t)j >> 1) & 1u) ^ 1u, status);
      tc_fence_after();
      const uint32_t t_hi = tmem_base + ((uint32_t)(quarter * 32) << 16) + C_::TMEM_A0 + (uint32_t)abuf * C_::TMEM_A_STRIDE;
      for (int kb = 0; kb < n_kb; ++kb) {
        const unsigned char* tile = a_base + (size_t)abuf * C_::A_BUF + (size_t)kb * C_::A_BYTES;
        uint32_t hi_bits[32], lo_bits[32];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 v = *reinterpret_cast<const float4*>(tile + row * 128 + ((q ^ (row & 7)) << 4));
          float4 h, l;
          split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
          hi_bits[4 * q] = __float_as_uint(h.x); hi_bits[4 * q + 1] = __float_as_uint(h.y);
          hi_bits[4 * q + 2] = __float_as_uint(h.z); hi_bits[4 * q + 3] = __float_as_uint(h.w);
          lo_bits[4 * q] = __float_as_uint(l.x); lo_bits[4 * q + 1] = __float_as_uint(l.y);
          lo_bits[4 * q + 2] = __float_as_uint(l.z); lo_bits[4 * q + 3] = __float_as_uint(l.w);
        }
        tmem_st_32(t_hi + (uint32_t)(kb * BK), hi_bits);
        tmem_st_32(t_hi + C_::TMEM_A_LO + (uint32_t)(kb * BK), lo_bits);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&a_split[abuf]); mbar_arrive(&a_raw_empty[abuf]); }
    }
  } else {
    const int quarter = warp & 3;
    unsigned char* slab = store_base + (size_t)quarter * 2 * 4096;
    int chunk_no = 0;
    uint32_t t = 0;
    for (int j = 0, blk = first; blk < m_blocks; ++j, blk += stride) {
      const long long row0 = (long long)blk * BM + quarter * 32;
      for (int nti = 0; nti < n_tiles; ++nti, ++t) {
        // row block b starts at weight tile b mod n_tiles: the CTAs do not all fetch the same weight lines from L2
        // at the same moment
        const int nt = (nti + blk) % n_tiles;
        const uint32_t buf = t & 1u;
        mbar_wait(&acc_full[buf], (t >> 1) & 1u, status);
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < AS_BN / 32; ++c, ++chunk_no) {
          uint32_t r[32];
          tmem_ld_32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * AS_BN + (uint32_t)(c * 32), r);
          unsigned char* sl = slab + (size_t)(chunk_no & 1) * 4096;
          if (lane == 0) bulk_wait_read<1>();     // the slab used two chunks ago has been read by its store
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            // SWIZZLE_128B: 16-byte chunk q of row `lane` sits at chunk position q ^ (lane & 7)
            *reinterpret_cast<float4*>(sl + lane * 128 + ((q ^ (lane & 7)) << 4)) =
                make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int col0 = nt * AS_BN + c * 32;
            if (col0 < N && row0 < M) {
              asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                           ::"l"(&tmC), "r"(col0), "r"((int)row0), "r"(0), "r"(smem_u32(sl)) : "memory");
            }
            bulk_commit();
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      }
    }
    if (lane == 0) bulk_wait_read<0>();   // the staging slabs must outlive their stores
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C_::TMEM_COLS);
  }
}

__global__ void split_weights_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = w[i];
    const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
    hi[i] = h; lo[i] = v - h;
  }
}

// --------------------------------------------------------------------------------- host side
__device__ int g_tc_status;

static PFN_cuTensorMapEncodeTiled get_encode() {
  static PFN_cuTensorMapEncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
  }
  return fn;
}

// 3-D FP32 tensor [d2][d1][d0] (d0 contiguous), box [b2][b1][b0], 128-byte swizzle, zero fill outside
int make_map(CUtensorMap* m, const float* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
                    uint64_t stride2_elems, uint32_t b0, uint32_t b1, uint32_t b2) {
  PFN_cuTensorMapEncodeTiled enc = get_encode();
  if (!enc) return FASTEQ_INTERNAL;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_elems * 4, stride2_elems * 4};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return FASTEQ_CUDA_ERROR;
  }
  return FASTEQ_OK;
}

bool supported(long long M, int a_rows, int K, int P, int N, int c_rows, const void* A, const void* Bt, const void* C) {
  if (M < 1 || K < 4 || N < 4 || (K % 4) || (N % 4)) return false;                 // 16-byte global strides
  if (M > 0x7fffffffLL) return false;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Bt) | reinterpret_cast<uintptr_t>(C)) & 15u) return false;
  if ((long long)a_rows * K > (1LL << 36) || (long long)N * K > (1LL << 36)) return false;
  return true;
}

static int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}

template <int BN>
static int launch_bn(const TcTable& tab, const CUtensorMap& ma, const CUtensorMap& mbh, const CUtensorMap& mbl, const CUtensorMap& mc,
                     long long M, int N, int K, cudaStream_t s) {
  int* st = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&st, g_tc_status);
  if (e != cudaSuccess) return cuda_fail(e);
  constexpr bool A_TMEM = (BN == 64);
  e = cudaFuncSetAttribute(gemm_tf32x3_kernel<BN, A_TMEM>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::SMEM_BYTES);
  if (e != cudaSuccess) return cuda_fail(e);
  const long long m_tiles = (M + BM - 1) / BM;
  const int n_tiles = (N + BN - 1) / BN;
  const long long total = m_tiles * n_tiles * tab.n_items;
  const int sms = sm_count();
  if (sms < 1) return FASTEQ_CUDA_ERROR;
  const unsigned grid = (unsigned)(total < sms ? total : sms);     // one persistent CTA per SM
  gemm_tf32x3_kernel<BN, A_TMEM><<<grid, NT_P, Cfg<BN>::SMEM_BYTES, s>>>(ma, mbh, mbl, mc, tab, M, N, K, total, (int)m_tiles, n_tiles, st);
  e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

// Bt_hi / Bt_lo: the [P, N, K] weight blocks already split into their TF32 parts (split_weights / the
// SO3Linear packing kernel do it once per call; the blocks are tiny next to A)
int launch(const TcTable& tab, const float* A, long long M, int a_rows, int K, const float* Bt_hi, const float* Bt_lo, int P, int N,
           float* C, int c_rows, cudaStream_t s) {
  if (tab.n_items < 1 || tab.n_items > 65535) return FASTEQ_UNSUPPORTED;
  const int BN = N <= 64 ? 64 : 128;
  alignas(64) CUtensorMap ma, mbh, mbl, mc;
  int rc = make_map(&ma, A, (uint64_t)K, (uint64_t)a_rows, (uint64_t)M, (uint64_t)K, (uint64_t)a_rows * K, BK, 1, BM);
  if (rc != FASTEQ_OK) return rc;
  rc = make_map(&mbh, Bt_hi, (uint64_t)K, (uint64_t)N, (uint64_t)P, (uint64_t)K, (uint64_t)N * K, BK, (uint32_t)BN, 1);
  if (rc != FASTEQ_OK) return rc;
  rc = make_map(&mbl, Bt_lo, (uint64_t)K, (uint64_t)N, (uint64_t)P, (uint64_t)K, (uint64_t)N * K, BK, (uint32_t)BN, 1);
  if (rc != FASTEQ_OK) return rc;
  rc = make_map(&mc, C, (uint64_t)N, (uint64_t)c_rows, (uint64_t)M, (uint64_t)N, (uint64_t)c_rows * N, 32, 1, 32);
  if (rc != FASTEQ_OK) return rc;
  return BN == 64 ? launch_bn<64>(tab, ma, mbh, mbl, mc, M, N, K, s) : launch_bn<128>(tab, ma, mbh, mbl, mc, M, N, K, s);
}

// hi / lo parts of n contiguous FP32 values into split[0 .. n) and split[n .. 2n)
int split_weights(const float* w, long long n, float* split, cudaStream_t s) {
  split_weights_kernel<<<(unsigned)((n + 255) / 256 < 1024 ? (n + 255) / 256 : 1024), 256, 0, s>>>(w, split, split + n, n);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

template <int KB>
static int launch_as_kb(const CUtensorMap& ma, const CUtensorMap& mbh, const CUtensorMap& mbl, const CUtensorMap& mc, long long M, int N,
                        int K, cudaStream_t s) {
  int* st = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&st, g_tc_status);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaFuncSetAttribute(gemm_tf32x3_as_kernel<KB>, cudaFuncAttributeMaxDynamicSharedMemorySize, AsCfg<KB>::SMEM_BYTES);
  if (e != cudaSuccess) return cuda_fail(e);
  gemm_tf32x3_as_kernel<KB><<<(unsigned)((M + BM - 1) / BM), NT, AsCfg<KB>::SMEM_BYTES, s>>>(ma, mbh, mbl, mc, M, N, K, st);
  e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

static int launch_as_persistent(const CUtensorMap& ma, const CUtensorMap& mbh, const CUtensorMap& mbl, const CUtensorMap& mc, long long M,
                                int N, int K, cudaStream_t s) {
  int* st = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&st, g_tc_status);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaFuncSetAttribute(gemm_tf32x3_asp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AspCfg::SMEM_BYTES);
  if (e != cudaSuccess) return cuda_fail(e);
  const long long m_blocks = (M + BM - 1) / BM;
  const int sms = sm_count();
  if (sms < 1) return FASTEQ_CUDA_ERROR;
  const unsigned grid = (unsigned)(m_blocks < sms ? m_blocks : sms);     // one persistent CTA per SM
  gemm_tf32x3_asp_kernel<<<grid, NT_ASP, AspCfg::SMEM_BYTES, s>>>(ma, mbh, mbl, mc, M, N, K, (int)m_blocks, st);
  e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

// plain C[M, N] = A[M, K] @ Bt[N, K]^T with K <= 128 and several N tiles
// `split`: hi / lo parts of Bt (2 * N * K floats)
int launch_a_stationary(const float* A, long long M, int K, const float* split, int N, float* C, cudaStream_t s) {
  const long long nw = (long long)N * K;
  alignas(64) CUtensorMap ma, mbh, mbl, mc;
  int rc = make_map(&ma, A, (uint64_t)K, 1, (uint64_t)M, (uint64_t)K, (uint64_t)K, BK, 1, BM);
  if (rc == FASTEQ_OK) rc = make_map(&mc, C, (uint64_t)N, (uint64_t)M, 1, (uint64_t)N, (uint64_t)N * M, 32, 32, 1);
  if (rc == FASTEQ_OK) rc = make_map(&mbh, split, (uint64_t)K, (uint64_t)N, 1, (uint64_t)K, (uint64_t)N * K, BK, AS_BN, 1);
  if (rc == FASTEQ_OK) rc = make_map(&mbl, split + nw, (uint64_t)K, (uint64_t)N, 1, (uint64_t)K, (uint64_t)N * K, BK, AS_BN, 1);
  if (rc == FASTEQ_OK) {
    const int kb = (K + BK - 1) / BK;
    rc = kb <= 2 ? launch_as_persistent(ma, mbh, mbl, mc, M, N, K, s) : launch_as_kb<4>(ma, mbh, mbl, mc, M, N, K, s);
  }
  return rc;
}

// C = A @ Bt^T with Bt given raw (split into a temporary) or already split
int dense(const float* A, const float* Bt, const float* split_in, float* C, long long M, int N, int K, cudaStream_t s) {
  if (M < 0 || N < 1 || K < 1) return FASTEQ_INVALID;
  if (M == 0) return FASTEQ_OK;
  if (!A || (!Bt && !split_in) || !C) return FASTEQ_INVALID;
  if (!supported(M, 1, K, 1, N, 1, A, split_in ? split_in : Bt, C)) return FASTEQ_UNSUPPORTED;
  const long long nw = (long long)N * K;
  float* tmp = nullptr;
  int rc = FASTEQ_OK;
  if (!split_in) {
    cudaError_t e = cudaMallocAsync((void**)&tmp, (size_t)nw * 2 * sizeof(float), s);
    if (e != cudaSuccess) return cuda_fail(e);
    rc = split_weights(Bt, nw, tmp, s);
  }
  const float* split = split_in ? split_in : tmp;
  if (rc == FASTEQ_OK) {
    if (K <= 128 && N >= 256) {
      rc = launch_a_stationary(A, M, K, split, N, C, s);
    } else {
      TcTable tab{};
      tab.n_groups = 1; tab.n_items = 1; tab.group_c_row[0] = 0; tab.group_first[0] = 0; tab.group_first[1] = 1;
      tab.item_first[0] = 0; tab.item_first[1] = 1; tab.path_a_row[0] = 0; tab.path_w[0] = 0;
      rc = launch(tab, A, M, 1, K, split, split + nw, 1, N, C, 1, s);
    }
  }
  if (tmp) cudaFreeAsync(tmp, s);
  return rc;
}

int device_status(int* code) {
  int v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  *code = v;
  return FASTEQ_OK;
}

}  // namespace tc
}  // namespace fasteq

// C[M, N] = A[M, K] @ Bt[N, K]^T, FP32 data, 3xTF32 tensor-core arithmetic (a layer of the radial MLP:
// Bt is torch's [out_features, in_features] weight).  K and N multiples of 4, 16-byte aligned pointers.
extern "C" int fasteq_gemm_tf32x3(const void* A, const void* Bt, void* C, int64_t M, int32_t N, int32_t K,
                                  fasteq_stream_t stream) {
  return fasteq::tc::dense((const float*)A, (const float*)Bt, nullptr, (float*)C, M, N, K, (cudaStream_t)stream);
}

// The two TF32 parts of a weight matrix, prepared once for many fasteq_gemm_tf32x3_presplit calls.
extern "C" int fasteq_gemm_tf32x3_split(const void* Bt, int64_t n_elems, void* split, fasteq_stream_t stream) {
  if (n_elems < 0 || (n_elems > 0 && (!Bt || !split))) return FASTEQ_INVALID;
  if (n_elems == 0) return FASTEQ_OK;
  return fasteq::tc::split_weights((const float*)Bt, n_elems, (float*)split, (cudaStream_t)stream);
}

extern "C" int fasteq_gemm_tf32x3_presplit(const void* A, const void* split, void* C, int64_t M, int32_t N, int32_t K,
                                           fasteq_stream_t stream) {
  if (!split && M > 0) return FASTEQ_INVALID;
  return fasteq::tc::dense((const float*)A, nullptr, (const float*)split, (float*)C, M, N, K, (cudaStream_t)stream);
}

extern "C" int fasteq_tensorcore_device_status(int32_t* code) {
  if (!code) return FASTEQ_INVALID;
  int a = 0, b = 0;
  int rc = fasteq::tc::device_status(&a);
  if (rc != FASTEQ_OK) return rc;
  rc = fasteq::chain::device_status(&b);
  if (rc != FASTEQ_OK) return rc;
  *code = a ? a : b;
  return FASTEQ_OK;
}
