// Periodic radius graph on the GPU: receiver-sorted edge list + CSR offsets for batches of
// orthorhombic boxes, in the canonical order (receiver, sender, image) of the host builder.
//
//   cell list : atoms binned into cells at least `cutoff` wide where the box allows (one cell and
//               several periodic images per side where it does not)
//   count     : one warp per receiver walks the (2R+1)^3 neighbouring cells, lanes stride over the
//               atoms of a cell; degrees -> exclusive scan = seg_ptr (the CSR the tensor-product
//               kernels consume, so no sortedness check or binary search is needed afterwards)
//   fill      : the same walk collects (sender, image) keys in shared memory, the warp sorts them
//               (bitonic) and writes sender, receiver and the cartesian image shift
//
// Distances are evaluated in FP64 with explicitly rounded operations in the order
// ((r_j + shift) - r_i), (dx^2 + dy^2) + dz^2, so that membership (r^2 < cutoff^2) is bit-identical to a
// numpy evaluation of the same expression.  The reference has no neighbour-list builder (its callers
// bring edge lists from ASE / matscipy); this is a neighbour of the hot path.
#include <cstdio>
#include <cstdint>
#include <cmath>
#include <vector>
#include <cuda_runtime.h>
#include "fasteq_b200.h"
#include "core_common.h"

using namespace fasteq;

namespace {

constexpr int kMaxDegree = 1024;        // neighbours of one receiver the sorting buffer holds
constexpr int kWarpsPerBlock = 4;

struct StructGrid {          // per structure, device copy
  int n[3];                  // cells per dimension
  int reach[3];              // neighbouring cells (or images) to visit on each side
  int cell_off;              // first global cell of the structure
  int pad;
  double box[3];
  double inv_w[3];           // 1 / cell width
};

struct Work {                // views into the caller's workspace
  StructGrid* grids;         // [S]
  int* cell_start;           // [C + 1] exclusive scan of the cell occupancy
  int* cell_cursor;          // [C]
  int* atom_cell;            // [N]
  int* cell_atoms;           // [N]
  int* header;               // [4]: max degree, error flag
  long long n_cells;
};

size_t align_up(size_t v) { return (v + 255) & ~size_t(255); }

size_t layout(const fasteq_nl_problem* p, long long n_cells, unsigned char* base, Work* w) {
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off += align_up(bytes); return base ? base + o : nullptr; };
  StructGrid* g = (StructGrid*)take(sizeof(StructGrid) * (size_t)p->n_structs);
  int* cs = (int*)take(sizeof(int) * (size_t)(n_cells + 1));
  int* cc = (int*)take(sizeof(int) * (size_t)n_cells);
  int* ac = (int*)take(sizeof(int) * (size_t)p->n_atoms);
  int* ca = (int*)take(sizeof(int) * (size_t)p->n_atoms);
  int* hd = (int*)take(sizeof(int) * 4);
  if (w) { w->grids = g; w->cell_start = cs; w->cell_cursor = cc; w->atom_cell = ac; w->cell_atoms = ca; w->header = hd; w->n_cells = n_cells; }
  return off;
}

int make_grids(const fasteq_nl_problem* p, std::vector<StructGrid>* out, long long* n_cells, int* max_reach) {
  if (!p || p->n_atoms < 0 || p->n_structs < 1 || !(p->cutoff > 0.0) || !p->box) return FASTEQ_INVALID;
  if (p->n_atoms > 0x7fffffffLL - 1) return FASTEQ_UNSUPPORTED;
  out->resize(p->n_structs);
  long long cells = 0;
  int mr = 0;
  for (int s = 0; s < p->n_structs; ++s) {
    StructGrid& g = (*out)[s];
    long long c = 1;
    for (int d = 0; d < 3; ++d) {
      const double L = p->box[3 * s + d];
      if (!(L > 0.0)) return FASTEQ_INVALID;
      int n = (int)std::floor(L / p->cutoff);
      n = n < 1 ? 1 : (n > 64 ? 64 : n);           // wider cells are still correct, only more candidates
      const double w = L / n;
      int r = w >= p->cutoff ? 1 : (int)std::ceil(p->cutoff / w);
      if (r > 8) return FASTEQ_UNSUPPORTED;         // box far smaller than the cutoff
      g.n[d] = n; g.reach[d] = r; g.box[d] = L; g.inv_w[d] = 1.0 / w;
      c *= n;
      mr = r > mr ? r : mr;
    }
    if (cells + c > 0x3fffffffLL) return FASTEQ_UNSUPPORTED;
    g.cell_off = (int)cells; g.pad = 0;
    cells += c;
  }
  *n_cells = cells; *max_reach = mr;
  return FASTEQ_OK;
}

__device__ __forceinline__ int cell_of(const StructGrid& g, const double* r, int* c) {
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    int v = (int)floor(r[d] * g.inv_w[d]);
    c[d] = v < 0 ? 0 : (v >= g.n[d] ? g.n[d] - 1 : v);
  }
  return g.cell_off + (c[0] * g.n[1] + c[1]) * g.n[2] + c[2];
}

__global__ void nl_bin_kernel(const double* __restrict__ pos, const int* __restrict__ atom_struct, long long n_atoms, Work w) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_atoms) return;
  const StructGrid g = w.grids[atom_struct[i]];
  const double r[3] = {pos[3 * i], pos[3 * i + 1], pos[3 * i + 2]};
  int c[3];
  const int cid = cell_of(g, r, c);
  w.atom_cell[i] = cid;
  atomicAdd(&w.cell_cursor[cid], 1);
}

// exclusive scan of `in[0..n)` into `out[0..n]` by one block (n up to a few million)
__global__ void nl_scan_kernel(const int* __restrict__ in, long long n, int* __restrict__ out) {
  __shared__ int warp_sums[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (long long base = 0; base < n; base += blockDim.x) {
    const long long i = base + threadIdx.x;
    const int v = i < n ? in[i] : 0;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[wid] = x;
    __syncthreads();
    if (wid == 0) {
      int s = lane < (int)(blockDim.x >> 5) ? warp_sums[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, s, o);
        if (lane >= o) s += y;
      }
      warp_sums[lane] = s;
    }
    __syncthreads();
    const int before = carry + (wid > 0 ? warp_sums[wid - 1] : 0) + x - v;
    if (i < n) out[i] = before;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry = before + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) out[n] = carry;
}

__global__ void nl_place_kernel(long long n_atoms, Work w) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_atoms) return;
  const int cid = w.atom_cell[i];
  const int slot = atomicAdd(&w.cell_cursor[cid], 1);
  w.cell_atoms[w.cell_start[cid] + slot] = (int)i;
}

// Walks the neighbourhood of receiver i with the whole warp; emit(sender, code, shift) is called by the
// lane that found a neighbour.  `code` orders images like their cartesian shifts.
template <typename Emit>
__device__ __forceinline__ void walk(const double* __restrict__ pos, const Work& w, const StructGrid& g, long long i, double c2,
                                     int code_base, int lane, Emit emit) {
  const double ri[3] = {pos[3 * i], pos[3 * i + 1], pos[3 * i + 2]};
  int c[3];
  cell_of(g, ri, c);
  for (int ox = -g.reach[0]; ox <= g.reach[0]; ++ox) {
    const int nbx = c[0] + ox;
    const int wx = nbx >= 0 ? nbx / g.n[0] : -((-nbx + g.n[0] - 1) / g.n[0]);
    const int cx = nbx - wx * g.n[0];
    const double sx = (double)wx * g.box[0];
    for (int oy = -g.reach[1]; oy <= g.reach[1]; ++oy) {
      const int nby = c[1] + oy;
      const int wy = nby >= 0 ? nby / g.n[1] : -((-nby + g.n[1] - 1) / g.n[1]);
      const int cy = nby - wy * g.n[1];
      const double sy = (double)wy * g.box[1];
      for (int oz = -g.reach[2]; oz <= g.reach[2]; ++oz) {
        const int nbz = c[2] + oz;
        const int wz = nbz >= 0 ? nbz / g.n[2] : -((-nbz + g.n[2] - 1) / g.n[2]);
        const int cz = nbz - wz * g.n[2];
        const double sz = (double)wz * g.box[2];
        const int cid = g.cell_off + (cx * g.n[1] + cy) * g.n[2] + cz;
        const int begin = w.cell_start[cid], end = w.cell_start[cid + 1];
        const bool home = (wx | wy | wz) == 0;
        const int code = ((wx + code_base) * (2 * code_base + 1) + (wy + code_base)) * (2 * code_base + 1) + (wz + code_base);
        for (int a = begin + lane; a < end; a += 32) {
          const int j = w.cell_atoms[a];
          if (home && j == (int)i) continue;
          const double dx = __dsub_rn(__dadd_rn(pos[3 * (long long)j], sx), ri[0]);
          const double dy = __dsub_rn(__dadd_rn(pos[3 * (long long)j + 1], sy), ri[1]);
          const double dz = __dsub_rn(__dadd_rn(pos[3 * (long long)j + 2], sz), ri[2]);
          const double r2 = __dadd_rn(__dadd_rn(__dmul_rn(dx, dx), __dmul_rn(dy, dy)), __dmul_rn(dz, dz));
          if (r2 < c2) emit(j, code, sx, sy, sz);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(32 * kWarpsPerBlock)
nl_count_kernel(const double* __restrict__ pos, const int* __restrict__ atom_struct, long long n_atoms, double c2, int code_base,
                Work w, int* __restrict__ degree) {
  const int lane = threadIdx.x & 31;
  const long long i = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (i >= n_atoms) return;
  const StructGrid g = w.grids[atom_struct[i]];
  int cnt = 0;
  walk(pos, w, g, i, c2, code_base, lane, [&](int, int, double, double, double) { ++cnt; });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (lane == 0) {
    degree[i] = cnt;
    atomicMax(&w.header[0], cnt);
  }
}

__global__ void __launch_bounds__(32 * kWarpsPerBlock)
nl_fill_kernel(const double* __restrict__ pos, const int* __restrict__ atom_struct, long long n_atoms, double c2, int code_base,
               Work w, const int* __restrict__ seg_ptr, int* __restrict__ edge_src, int* __restrict__ edge_dst,
               double* __restrict__ edge_shift) {
  __shared__ unsigned long long keys[kWarpsPerBlock][kMaxDegree];
  __shared__ int counters[kWarpsPerBlock];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const long long i = (long long)blockIdx.x * kWarpsPerBlock + wid;
  if (i >= n_atoms) return;
  const StructGrid g = w.grids[atom_struct[i]];
  const int begin = seg_ptr[i], deg = seg_ptr[i + 1] - begin;
  if (deg <= 0) return;
  if (deg > kMaxDegree) { if (lane == 0) atomicExch(&w.header[1], 1); return; }
  if (lane == 0) counters[wid] = 0;
  __syncwarp();
  unsigned long long* k = keys[wid];
  walk(pos, w, g, i, c2, code_base, lane, [&](int j, int code, double, double, double) {
    const int slot = atomicAdd(&counters[wid], 1);
    if (slot < kMaxDegree) k[slot] = ((unsigned long long)(unsigned)j << 20) | (unsigned)code;
  });
  __syncwarp();
  int n_pad = 1;
  while (n_pad < deg) n_pad <<= 1;
  for (int t = deg + lane; t < n_pad; t += 32) k[t] = ~0ull;
  __syncwarp();
  for (int size = 2; size <= n_pad; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = lane; t < (n_pad >> 1); t += 32) {
        const int lo = 2 * t - (t & (stride - 1));       // element whose partner is lo + stride
        const int hi = lo + stride;
        const bool up = (lo & size) == 0;
        const unsigned long long a = k[lo], b = k[hi];
        if ((a > b) == up) { k[lo] = b; k[hi] = a; }
      }
      __syncwarp();
    }
  }
  const int span = 2 * code_base + 1;
  for (int t = lane; t < deg; t += 32) {
    const unsigned long long key = k[t];
    const int j = (int)(key >> 20), code = (int)(key & 0xfffffu);
    const int wz = code % span - code_base, wy = (code / span) % span - code_base, wx = code / (span * span) - code_base;
    const long long e = begin + t;
    edge_src[e] = j;
    edge_dst[e] = (int)i;
    edge_shift[3 * e] = (double)wx * g.box[0];
    edge_shift[3 * e + 1] = (double)wy * g.box[1];
    edge_shift[3 * e + 2] = (double)wz * g.box[2];
  }
}

}  // namespace

extern "C" int fasteq_neighbors_work_bytes(const fasteq_nl_problem* p, int64_t* bytes) {
  std::vector<StructGrid> grids;
  long long n_cells = 0;
  int mr = 0;
  int rc = make_grids(p, &grids, &n_cells, &mr);
  if (rc != FASTEQ_OK) return rc;
  if (!bytes) return FASTEQ_INVALID;
  *bytes = (int64_t)layout(p, n_cells, nullptr, nullptr);
  return FASTEQ_OK;
}

static int prepare(const fasteq_nl_problem* p, void* work, int64_t work_bytes, Work* w, int* code_base, bool upload, cudaStream_t s) {
  std::vector<StructGrid> grids;
  long long n_cells = 0;
  int mr = 0;
  int rc = make_grids(p, &grids, &n_cells, &mr);
  if (rc != FASTEQ_OK) return rc;
  if (!work || (p->n_atoms > 0 && (!p->pos || !p->atom_struct))) return FASTEQ_INVALID;
  if ((int64_t)layout(p, n_cells, (unsigned char*)work, w) > work_bytes) return FASTEQ_INVALID;
  *code_base = mr;
  if (upload) {
    cudaError_t e = cudaMemcpyAsync(w->grids, grids.data(), sizeof(StructGrid) * grids.size(), cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  return FASTEQ_OK;
}

extern "C" int fasteq_neighbors_count(const fasteq_nl_problem* p, void* work, int64_t work_bytes, int32_t* seg_ptr,
                                      int32_t* max_degree, fasteq_stream_t stream) {
  cudaStream_t s = (cudaStream_t)stream;
  Work w{};
  int code_base = 0;
  int rc = prepare(p, work, work_bytes, &w, &code_base, true, s);
  if (rc != FASTEQ_OK) return rc;
  if (!seg_ptr) return FASTEQ_INVALID;
  const long long N = p->n_atoms;
  cudaError_t e = cudaMemsetAsync(w.cell_cursor, 0, sizeof(int) * (size_t)w.n_cells, s);
  if (e == cudaSuccess) e = cudaMemsetAsync(w.header, 0, sizeof(int) * 4, s);
  if (e != cudaSuccess) return cuda_fail(e);
  if (N > 0) nl_bin_kernel<<<(unsigned)((N + 255) / 256), 256, 0, s>>>(p->pos, p->atom_struct, N, w);
  nl_scan_kernel<<<1, 1024, 0, s>>>(w.cell_cursor, w.n_cells, w.cell_start);
  e = cudaMemsetAsync(w.cell_cursor, 0, sizeof(int) * (size_t)w.n_cells, s);
  if (e != cudaSuccess) return cuda_fail(e);
  if (N > 0) {
    nl_place_kernel<<<(unsigned)((N + 255) / 256), 256, 0, s>>>(N, w);
    // degrees into atom_cell (not needed any more), then their scan into seg_ptr
    nl_count_kernel<<<(unsigned)((N + kWarpsPerBlock - 1) / kWarpsPerBlock), 32 * kWarpsPerBlock, 0, s>>>(
        p->pos, p->atom_struct, N, p->cutoff * p->cutoff, code_base, w, w.atom_cell);
  }
  nl_scan_kernel<<<1, 1024, 0, s>>>(w.atom_cell, N, seg_ptr);
  if (max_degree) {
    e = cudaMemcpyAsync(max_degree, w.header, sizeof(int), cudaMemcpyDeviceToDevice, s);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

extern "C" int fasteq_neighbors_fill(const fasteq_nl_problem* p, void* work, int64_t work_bytes, const int32_t* seg_ptr,
                                     int32_t* edge_src, int32_t* edge_dst, double* edge_shift, fasteq_stream_t stream) {
  cudaStream_t s = (cudaStream_t)stream;
  Work w{};
  int code_base = 0;
  int rc = prepare(p, work, work_bytes, &w, &code_base, false, s);
  if (rc != FASTEQ_OK) return rc;
  if (!seg_ptr) return FASTEQ_INVALID;
  const long long N = p->n_atoms;
  if (N == 0) return FASTEQ_OK;
  if (!edge_src || !edge_dst || !edge_shift) return FASTEQ_INVALID;
  nl_fill_kernel<<<(unsigned)((N + kWarpsPerBlock - 1) / kWarpsPerBlock), 32 * kWarpsPerBlock, 0, s>>>(
      p->pos, p->atom_struct, N, p->cutoff * p->cutoff, code_base, w, seg_ptr, edge_src, edge_dst, edge_shift);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}
