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
// OSEG, STAGES, PIPES, PREFETCH, Y_VEC, W_SHARED, X_INDEXED, Y_INDEXED, SCATTERED, Y_SH, NCONS_WARPS,
// STAGE_EXTRA_BYTES, EMIT_EMPTY_ROWS, BEGIN_PER_SEGMENT } and namespace fasteq_sh { eval, vjp }
// (spherical harmonics of an edge vector and their vector-Jacobian product; stubs unless Y_SH).
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
  int n_vblocks;    // pipelines that have work (grid * pipelines per CTA may exceed it)
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
  unsigned char* stages; uint64_t* full; uint64_t* empty; int lane; uint32_t it; int vblock;
  bool failed = false;   // a wait of this lane gave up: the warp stops issuing copies and reductions (see dead())

  static __device__ __forceinline__ int valid_of(int ct) { return (U - ct * CT) < CT ? (U - ct * CT) : CT; }
  static __device__ __forceinline__ uint32_t tx_bytes(int valid) {
    return (uint32_t)((cfg::W_SHARED ? 0 : WSEG) + XSEG + (cfg::Y_VEC ? YSEG : 0)) * (uint32_t)(valid * sizeof(T));
  }
  __device__ __forceinline__ int checked(int r, long long n) {
    if (r < 0 || (long long)r >= n) { atomicExch(g.status, (int)kDevBadIndex); return 0; }
    return r;
  }

  // Bulk path: ONE lane fills one stage (record, expected bytes, bulk copies of its edge's rows,
  // 4/8-byte cp.async for a scalar y row).  Up to STAGES lanes do this side by side, so the
  // producer spends about (instructions of one fill) / STAGES per edge.
  // `flush(st)` runs on the same lane before a stage is reused; the backward finishes the
  // per-edge y-gradient there.
  template <typename Flush>
  __device__ __forceinline__ void fill_one(uint32_t myit, int flags, int row, int ct, int e, int xr, int yr, Flush&& flush) {
    const int stage = myit % STAGES;
    const uint32_t ph = (myit / STAGES) & 1u;
    if (!mbar_wait(&empty[stage], ph ^ 1u, g.status)) { failed = true; return; }
    unsigned char* st = stages + (size_t)stage * STAGE_BYTES;
    if (myit >= (uint32_t)STAGES) flush(st);
    const int valid = valid_of(ct);
    Meta m; m.row = row; m.flags = flags; m.ct = ct; m.e = e; m.xr = xr; m.yr = yr; m.pad0 = 0; m.pad1 = 0;
    *reinterpret_cast<Meta*>(st + OFF_META) = m;
    const bool data = (flags & F_DATA) != 0;
    if (cfg::Y_SH && data) sh_row(st, yr);     // plain stores, published by the arrive below
    mbar_arrive_expect_tx(&full[stage], data ? tx_bytes(valid) : 0u);
    if (data) {
      const uint32_t piece = (uint32_t)(valid * sizeof(T));
      if (!cfg::W_SHARED) {
        const T* src = w + (size_t)e * WSEG * U;
        if (FULL_ROW) bulk_g2s(st + OFF_W, src, (uint32_t)(WSEG * U * sizeof(T)), &full[stage]);
        else for (int s = 0; s < WSEG; ++s) bulk_g2s(st + OFF_W + (size_t)s * CT * sizeof(T), src + (size_t)s * U + ct * CT, piece, &full[stage]);
      }
      {
        const T* src = x + (size_t)xr * XSEG * U;
        if (FULL_ROW) bulk_g2s(st + OFF_X, src, (uint32_t)(XSEG * U * sizeof(T)), &full[stage]);
        else for (int s = 0; s < XSEG; ++s) bulk_g2s(st + OFF_X + (size_t)s * CT * sizeof(T), src + (size_t)s * U + ct * CT, piece, &full[stage]);
      }
      if (cfg::Y_VEC) {
        const T* src = y + (size_t)yr * YSEG * U;
        if (FULL_ROW) bulk_g2s(st + OFF_Y, src, (uint32_t)(YSEG * U * sizeof(T)), &full[stage]);
        else for (int s = 0; s < YSEG; ++s) bulk_g2s(st + OFF_Y + (size_t)s * CT * sizeof(T), src + (size_t)s * U + ct * CT, piece, &full[stage]);
      } else if (!cfg::Y_SH) {
        const T* src = y + (size_t)yr * YSEG;
#pragma unroll
        for (int k = 0; k < YSEG; ++k) cp_async_elem(st + OFF_Y + k * sizeof(T), src + k);
      }
    }
    cp_async_arrive_noinc(&full[stage]);
  }

  // True for the whole warp once any lane's wait has given up (or a caller-side wait set `failed`).
  // A stalled pipeline must not go on: the stage records the consumers would read next were never
  // written, and flush() would add partial sums into gradients.
  __device__ __forceinline__ bool dead() { return __any_sync(0xffffffffu, failed) != 0; }

  // After a failed wait: give the copies this warp has already issued a bounded time to land before the
  // CTA may exit (a full barrier completes on the producer's own arrives plus the copied bytes, whatever
  // the consumers do).
  __device__ __forceinline__ void settle() {
    if (lane < STAGES && it > (uint32_t)lane) {
      const uint32_t k = ((it - 1u - (uint32_t)lane) / STAGES) * STAGES + (uint32_t)lane;   // last fill of stage `lane`
      const uint32_t ph = (k / STAGES) & 1u;
#pragma unroll 1
      for (int i = 0; i < 100000; ++i) if (mbar_try_wait(&full[lane], ph)) break;
    }
    __syncwarp();
  }

  // this lane's edge: its weight row and its gathered x row (the tile's share of them) towards L2
  __device__ __forceinline__ void prefetch_rows(int e, int xr, int yr, int ct) {
    (void)yr;
    if (FULL_ROW) {
      if (!cfg::W_SHARED) bulk_prefetch_l2(w + (size_t)e * WSEG * U, (uint32_t)(WSEG * U * sizeof(T)));
      bulk_prefetch_l2(x + (size_t)xr * XSEG * U, (uint32_t)(XSEG * U * sizeof(T)));
    } else {
      const uint32_t piece = (uint32_t)(valid_of(ct) * sizeof(T));
      if (!cfg::W_SHARED) for (int s = 0; s < WSEG; ++s) bulk_prefetch_l2(w + (size_t)e * WSEG * U + (size_t)s * U + ct * CT, piece);
      for (int s = 0; s < XSEG; ++s) bulk_prefetch_l2(x + (size_t)xr * XSEG * U + (size_t)s * U + ct * CT, piece);
    }
  }

  // Y_SH: the y operand is the edge vector; its harmonics are evaluated here, into the stage's y row
  __device__ __forceinline__ void sh_row(unsigned char* st, int yr) {
    const T* v = y + (size_t)yr * 3;
    T sh[YSEG];
    fasteq_sh::eval(v[0], v[1], v[2], sh);
    T* dst = reinterpret_cast<T*>(st + OFF_Y);
#pragma unroll
    for (int k = 0; k < YSEG; ++k) dst[k] = sh[k];
  }

  // Fallback path (operands not 16-byte aligned): the whole warp copies one edge with 4/8-byte cp.async.
  template <typename Flush>
  __device__ __forceinline__ void fill_coop(int flags, int row, int ct, int e, int xr, int yr, Flush&& flush) {
    const int stage = it % STAGES;
    const uint32_t ph = (it / STAGES) & 1u;
    if (!mbar_wait(&empty[stage], ph ^ 1u, g.status)) failed = true;
    if (dead()) return;
    unsigned char* st = stages + (size_t)stage * STAGE_BYTES;
    if (lane == 0) {
      if (it >= (uint32_t)STAGES) flush(st);
      Meta m; m.row = row; m.flags = flags; m.ct = ct; m.e = e; m.xr = xr; m.yr = yr; m.pad0 = 0; m.pad1 = 0;
      *reinterpret_cast<Meta*>(st + OFF_META) = m;
      if (cfg::Y_SH && (flags & F_DATA)) sh_row(st, yr);
      mbar_arrive_expect_tx(&full[stage], 0u);
    }
    __syncwarp();
    if (flags & F_DATA) {
      const int valid = valid_of(ct);
      if (!cfg::W_SHARED) copy_tile(st + OFF_W, w + (size_t)e * WSEG * U, WSEG, ct, valid, false, &full[stage], lane);
      copy_tile(st + OFF_X, x + (size_t)xr * XSEG * U, XSEG, ct, valid, false, &full[stage], lane);
      if (cfg::Y_VEC) copy_tile(st + OFF_Y, y + (size_t)yr * YSEG * U, YSEG, ct, valid, false, &full[stage], lane);
      else if (!cfg::Y_SH) for (int k = lane; k < YSEG; k += 32) cp_async_elem(st + OFF_Y + k * sizeof(T), y + (size_t)yr * YSEG + k);
    }
    cp_async_arrive_noinc(&full[stage]);
    ++it;
  }

  // A stage without rows (an empty receiver, or the end marker).
  template <typename Flush>
  __device__ __forceinline__ void fill_special(int flags, int row, int ct, Flush&& flush) {
    if (g.bulk_ok) {
      if (lane == 0) fill_one(it, flags, row, ct, 0, 0, 0, flush);
      __syncwarp();
      ++it;
    } else {
      fill_coop(flags, row, ct, 0, 0, 0, flush);
    }
  }

  // m <= 32 consecutive edges of one segment (lane l holds edge l: id, x row, y row);
  // first / last tell whether the batch starts / ends the segment.
  template <typename Flush, typename Begin>
  __device__ __forceinline__ void fill_batch(int m, int me, int mx, int my, int row, int ct, bool first, bool last,
                                             bool each_is_segment, Flush&& flush, Begin&& begin) {
    if (g.bulk_ok && !(each_is_segment && cfg::BEGIN_PER_SEGMENT)) {
      // L2 prefetch, PREFETCH ring-fuls ahead of the stage fills: the ring bounds the bytes this pipeline has in
      // flight towards shared memory; rows asked into L2 early shorten the latency of the copies that follow
      if (cfg::PREFETCH > 0 && lane < m && lane < cfg::PREFETCH * STAGES) prefetch_rows(me, mx, my, ct);
      for (int base = 0; base < m; base += STAGES) {
        const int n = (m - base) < STAGES ? (m - base) : STAGES;
        const int l = lane - base;
        if (cfg::PREFETCH > 0) {
          const int pl = l - cfg::PREFETCH * STAGES;
          if (pl >= 0 && pl < STAGES && lane < m) prefetch_rows(me, mx, my, ct);
        }
        if (l >= 0 && l < n) {
          int flags = F_DATA;
          if (each_is_segment || (first && lane == 0)) flags |= F_FIRST;
          if (each_is_segment || (last && lane == m - 1)) flags |= F_LAST;
          fill_one(it + (uint32_t)l, flags, each_is_segment ? me : row, ct, me, mx, my, flush);
        }
        __syncwarp();
        it += (uint32_t)n;
      }
    } else {
      for (int j = 0; j < m; ++j) {
        const int e = __shfl_sync(0xffffffffu, me, j);
        const int xr = __shfl_sync(0xffffffffu, mx, j), yr = __shfl_sync(0xffffffffu, my, j);
        int flags = F_DATA;
        if (each_is_segment || (first && j == 0)) flags |= F_FIRST;
        if (each_is_segment || (last && j == m - 1)) flags |= F_LAST;
        const int r = each_is_segment ? e : row;
        if (each_is_segment) begin(r, ct, lane);
        if (dead()) return;
        if (g.bulk_ok) {
          if (lane == 0) fill_one(it, flags, r, ct, e, xr, yr, flush);
          __syncwarp();
          ++it;
        } else {
          fill_coop(flags, r, ct, e, xr, yr, flush);
        }
      }
    }
  }

  template <typename Flush, typename Begin>
  __device__ __forceinline__ void run(Flush&& flush, Begin&& begin) {
    it = 0;
    const long long n_units = cfg::SCATTERED ? g.n_out_rows : g.n_edges;
    long long s0, s1;
    // vblock: this pipeline's index among all pipelines of the launch (a CTA may hold several)
    if (vblock >= g.n_vblocks) { s0 = 0; s1 = 0; }
    else if (g.part_ptr) { s0 = g.part_ptr[vblock]; s1 = g.part_ptr[vblock + 1]; }
    else { s0 = n_units * vblock / g.n_vblocks; s1 = n_units * (vblock + 1) / g.n_vblocks; }
    for (int ct = 0; ct < NCT; ++ct) {
      if (cfg::SCATTERED) {
        for (long long sb = s0; sb < s1; sb += 32) {
          const int n = (int)((s1 - sb) < 32 ? (s1 - sb) : 32);
          int rp0 = 0, rp1 = 0;
          if (lane < n) { rp0 = g.seg_ptr[sb + lane]; rp1 = g.seg_ptr[sb + lane + 1]; }
          for (int i = 0; i < n; ++i) {
            const int e0 = __shfl_sync(0xffffffffu, rp0, i), e1 = __shfl_sync(0xffffffffu, rp1, i);
            const int row = (int)(sb + i);
            if (e0 >= e1) {
              if (cfg::EMIT_EMPTY_ROWS) { fill_special(F_LAST, row, ct, flush); if (dead()) { settle(); return; } }
              continue;
            }
            begin(row, ct, lane);
            if (dead()) { settle(); return; }
            for (int pb = e0; pb < e1; pb += 32) {
              const int m = (e1 - pb) < 32 ? (e1 - pb) : 32;
              int me = 0, mx = 0, my = 0;
              if (lane < m) {
                me = g.perm ? g.perm[pb + lane] : pb + lane;
                me = checked(me, g.n_edges);
                mx = cfg::X_INDEXED ? checked(g.x_index[me], g.x_rows) : me;
                my = cfg::Y_INDEXED ? checked(g.y_index[me], g.y_rows) : me;
              }
              fill_batch(m, me, mx, my, row, ct, pb == e0, pb + m == e1, false, flush, begin);
              if (dead()) { settle(); return; }
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
          fill_batch(m, me, mx, my, 0, ct, true, true, true, flush, begin);
          if (dead()) { settle(); return; }
        }
      }
    }
    fill_special(F_DONE, 0, 0, flush);
    if (dead()) { settle(); return; }
    // drain: every stage still holding a finished edge gets its flush
    const uint32_t total = it;
    const uint32_t first = total > (uint32_t)STAGES ? total - STAGES : 0;
    const uint32_t k = first + (uint32_t)lane;
    if (k < total) {
      const int stage = k % STAGES;
      const uint32_t ph = (k / STAGES) & 1u;
      if (mbar_wait(&empty[stage], ph, g.status)) flush(stages + (size_t)stage * STAGE_BYTES);
    }
    __syncwarp();
  }
};

// full[s] expects: bulk path = the filling lane's expect_tx arrive + its cp.async completion arrive;
// fallback path = lane 0's arrive + one cp.async completion arrive per lane.
__device__ __forceinline__ void init_barriers(uint64_t* full, uint64_t* empty, int bulk_ok) {
  for (int s = 0; s < STAGES; ++s) {
    mbar_init(&full[s], bulk_ok ? 2 : 33);
    mbar_init(&empty[s], cfg::NCONS_WARPS);  // one arrive per consumer warp of the pipeline
  }
}

}  // namespace u1d
}  // namespace fasteq
