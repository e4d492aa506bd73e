// Producer side of the Uniform1D kernels: one warp walks this CTA's share of the
// receiver-sorted edge list and feeds a ring of shared-memory stages, one edge
// per stage: the edge's weight row, the gathered x row, its y row and a small
// record (output row, flags, edge id).  Rows travel as 1-D bulk asynchronous
// copies (TMA engine) when base pointers and row sizes are 16-byte aligned,
// otherwise as 4/8-byte cp.async; both complete on the stage's mbarrier, so the
// producer never blocks on memory.  Consumer warps (generated code) see only
// shared memory.
//
// The including file must define namespace cfg { T, U, CT, WSEG, XSEG, YSEG,
// OSEG, STAGES, Y_VEC, W_SHARED, X_INDEXED, Y_INDEXED, SCATTERED, NCONS_WARPS,
// STAGE_EXTRA_BYTES, EMIT_EMPTY_ROWS }.
#pragma once
#include "fasteq_device.cuh"

namespace fasteq {
namespace u1d {

using T = cfg::T;
constexpr int U = cfg::U, CT = cfg::CT, WSEG = cfg::WSEG, XSEG = cfg::XSEG, YSEG = cfg::YSEG, OSEG = cfg::OSEG;
constexpr int STAGES = cfg::STAGES;
constexpr int NCT = (U + CT - 1) / CT;           // channel tiles
constexpr bool FULL_ROW = (CT == U);             // a tile is the whole contiguous row

constexpr int round_up(int a, int b) { return (a + b - 1) / b * b; }

struct Meta { int row; int flags; int ct; int e; int xr; int yr; int pad0; int pad1; };
enum : int { F_DATA = 1, F_LAST = 2, F_DONE = 4, F_FIRST = 8 };

constexpr int W_TILE_BYTES = cfg::W_SHARED ? 0 : WSEG * CT * (int)sizeof(T);
constexpr int X_TILE_BYTES = XSEG * CT * (int)sizeof(T);
constexpr int Y_TILE_BYTES = cfg::Y_VEC ? YSEG * CT * (int)sizeof(T) : round_up(YSEG * (int)sizeof(T), 16);
constexpr int OFF_W = 0;
constexpr int OFF_X = OFF_W + W_TILE_BYTES;
constexpr int OFF_Y = OFF_X + X_TILE_BYTES;
constexpr int OFF_META = OFF_Y + Y_TILE_BYTES;
constexpr int OFF_EXTRA = OFF_META + 32;          // per-stage scratch the backward uses (gy partials)
constexpr int STAGE_BYTES = round_up(OFF_EXTRA + cfg::STAGE_EXTRA_BYTES, 128);
constexpr int BAR_BYTES = 256;                    // full[STAGES], empty[STAGES], aux barriers
static_assert(STAGES * 16 + 32 <= BAR_BYTES, "too many stages for the barrier block");

struct Graph {
  long long n_edges, n_out_rows, x_rows, y_rows;
  const int* x_index; const int* y_index; const int* seg_ptr; const int* perm; const int* part_ptr;
  int bulk_ok;      // rows may travel as bulk copies
  int* status;
};

__device__ __forceinline__ void cp_async_elem(void* smem_dst, const void* gsrc) {
  if (sizeof(T) == 4)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Copy `nseg` segments of `valid` channels (row-major [seg][U] in global, [seg][CT] in shared).
__device__ __forceinline__ void copy_tile(unsigned char* sdst, const T* grow, int nseg, int ct, int valid, bool bulk,
                                          uint64_t* bar, int lane) {
  if (bulk) {
    if (FULL_ROW) {
      if (lane == 0) bulk_g2s(sdst, grow, (uint32_t)(nseg * U * sizeof(T)), bar);
    } else {
      for (int s = lane; s < nseg; s += 32)
        bulk_g2s(sdst + (size_t)s * CT * sizeof(T), grow + (size_t)s * U + ct * CT, (uint32_t)(valid * sizeof(T)), bar);
    }
  } else {
    for (int s = 0; s < nseg; ++s)
      for (int c = lane; c < valid; c += 32)
        cp_async_elem(sdst + ((size_t)s * CT + c) * sizeof(T), grow + (size_t)s * U + ct * CT + c);
  }
}

struct Producer {
  const Graph& g; const T* w; const T* x; const T* y;
  unsigned char* stages; uint64_t* full; uint64_t* empty; int lane; uint32_t it;

  // Called when a stage is about to be reused (and once per stage at the end): `prev` is the
  // record of the edge that occupied it.  The backward kernels finish per-edge reductions here.
  template <typename Flush, typename Begin>
  __device__ __forceinline__ void emit(int flags, int row, int ct, int e, int xr, int yr, Flush&& flush, Begin&& begin) {
    const int stage = it % STAGES;
    const uint32_t ph = (it / STAGES) & 1u;
    if (flags & F_FIRST) begin(row, ct, lane);
    mbar_wait(&empty[stage], ph ^ 1u, g.status);
    unsigned char* st = stages + (size_t)stage * STAGE_BYTES;
    if (it >= (uint32_t)STAGES) flush(st, lane);
    const int valid = (U - ct * CT) < CT ? (U - ct * CT) : CT;
    const bool data = (flags & F_DATA) != 0;
    const bool bulk = g.bulk_ok != 0;
    if (lane == 0) {
      Meta m; m.row = row; m.flags = flags; m.ct = ct; m.e = e; m.xr = xr; m.yr = yr; m.pad0 = 0; m.pad1 = 0;
      *reinterpret_cast<Meta*>(st + OFF_META) = m;
      uint32_t tx = 0;
      if (data && bulk) {
        tx = (uint32_t)((cfg::W_SHARED ? 0 : WSEG) + XSEG + (cfg::Y_VEC ? YSEG : 0)) * (uint32_t)(valid * sizeof(T));
      }
      mbar_arrive_expect_tx(&full[stage], tx);
    }
    __syncwarp();
    if (data) {
      if (!cfg::W_SHARED) copy_tile(st + OFF_W, w + (size_t)e * WSEG * U, WSEG, ct, valid, bulk, &full[stage], lane);
      copy_tile(st + OFF_X, x + (size_t)xr * XSEG * U, XSEG, ct, valid, bulk, &full[stage], lane);
      if (cfg::Y_VEC) {
        copy_tile(st + OFF_Y, y + (size_t)yr * YSEG * U, YSEG, ct, valid, bulk, &full[stage], lane);
      } else {
        for (int k = lane; k < YSEG; k += 32) cp_async_elem(st + OFF_Y + k * sizeof(T), y + (size_t)yr * YSEG + k);
      }
    }
    cp_async_arrive_noinc(&full[stage]);
    ++it;
  }

  __device__ __forceinline__ int checked(int r, long long n) {
    if (r < 0 || (long long)r >= n) { atomicExch(g.status, (int)kDevBadIndex); return 0; }
    return r;
  }

  template <typename Flush, typename Begin>
  __device__ __forceinline__ void run(Flush&& flush, Begin&& begin) {
    it = 0;
    const long long n_units = cfg::SCATTERED ? g.n_out_rows : g.n_edges;
    long long s0, s1;
    if (g.part_ptr) { s0 = g.part_ptr[blockIdx.x]; s1 = g.part_ptr[blockIdx.x + 1]; }
    else { s0 = n_units * blockIdx.x / gridDim.x; s1 = n_units * (blockIdx.x + 1) / gridDim.x; }
    for (int ct = 0; ct < NCT; ++ct) {
      if (cfg::SCATTERED) {
        for (long long sb = s0; sb < s1; sb += 32) {
          const int n = (int)((s1 - sb) < 32 ? (s1 - sb) : 32);
          int rp0 = 0, rp1 = 0;
          if (lane < n) { rp0 = g.seg_ptr[sb + lane]; rp1 = g.seg_ptr[sb + lane + 1]; }
          for (int i = 0; i < n; ++i) {
            const int e0 = __shfl_sync(0xffffffffu, rp0, i), e1 = __shfl_sync(0xffffffffu, rp1, i);
            const int row = (int)(sb + i);
            if (e0 >= e1) { if (cfg::EMIT_EMPTY_ROWS) emit(F_LAST, row, ct, 0, 0, 0, flush, begin); continue; }
            for (int pb = e0; pb < e1; pb += 32) {
              const int m = (e1 - pb) < 32 ? (e1 - pb) : 32;
              int me = 0, mx = 0, my = 0;
              if (lane < m) {
                me = g.perm ? g.perm[pb + lane] : pb + lane;
                me = checked(me, g.n_edges);
                mx = cfg::X_INDEXED ? checked(g.x_index[me], g.x_rows) : me;
                my = cfg::Y_INDEXED ? checked(g.y_index[me], g.y_rows) : me;
              }
              for (int j = 0; j < m; ++j) {
                const int e = __shfl_sync(0xffffffffu, me, j);
                const int xr = __shfl_sync(0xffffffffu, mx, j), yr = __shfl_sync(0xffffffffu, my, j);
                emit(F_DATA | ((pb + j == e1 - 1) ? F_LAST : 0) | ((pb + j == e0) ? F_FIRST : 0), row, ct, e, xr, yr, flush, begin);
              }
            }
          }
        }
      } else {
        for (long long pb = s0; pb < s1; pb += 32) {
          const int m = (int)((s1 - pb) < 32 ? (s1 - pb) : 32);
          int me = 0, mx = 0, my = 0;
          if (lane < m) {
            me = (int)(pb + lane);
            mx = cfg::X_INDEXED ? checked(g.x_index[me], g.x_rows) : me;
            my = cfg::Y_INDEXED ? checked(g.y_index[me], g.y_rows) : me;
          }
          for (int j = 0; j < m; ++j) {
            const int e = __shfl_sync(0xffffffffu, me, j);
            const int xr = __shfl_sync(0xffffffffu, mx, j), yr = __shfl_sync(0xffffffffu, my, j);
            emit(F_DATA | F_LAST | F_FIRST, e, ct, e, xr, yr, flush, begin);
          }
        }
      }
    }
    emit(F_DONE, 0, 0, 0, 0, 0, flush, begin);
    // drain: every stage still holding a finished edge gets its flush, in order
    const uint32_t total = it;
    const uint32_t first = total > (uint32_t)STAGES ? total - STAGES : 0;
    for (uint32_t k = first; k < total; ++k) {
      const int stage = k % STAGES;
      const uint32_t ph = (k / STAGES) & 1u;
      mbar_wait(&empty[stage], ph, g.status);
      flush(stages + (size_t)stage * STAGE_BYTES, lane);
    }
  }
};

__device__ __forceinline__ void init_barriers(uint64_t* full, uint64_t* empty) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 33);                 // lane 0's expect_tx arrive + 32 cp.async completion arrives
      mbar_init(&empty[s], cfg::NCONS_WARPS);  // one arrive per consumer warp
    }
    mbar_fence_init();
  }
  __syncthreads();
}

}  // namespace u1d
}  // namespace fasteq
