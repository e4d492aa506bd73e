"""CUDA source emitters for the Uniform1D (ChannelwiseTensorProduct) kernels, sm_100a.

One generated translation unit = one operator signature (path table, segment
counts, channel count, dtype, indexing mode) with the non-zero Clebsch-Gordan
coefficients as literals, exporting the C ABI of include/fasteq_b200.h.
Counterpart of the reference's emitters
(fasteq/ops/auto_schedule/uniform1d_forward.py:253-632 forward,
uniform1d_backward.py:256-888 backward), with a different execution model:

* persistent CTAs, each owning a contiguous range of receiver segments (CSR over
  receiver-sorted edges) instead of one CTA per edge;
* a producer warp stages each edge's rows into a shared-memory ring with bulk
  asynchronous copies; consumer threads (one per channel) only read shared memory;
* the forward keeps the receiver's output row in registers across the segment and
  writes it once with plain stores -- no atomics and no zero-fill of ``out``;
* products ``x[j] * y[k]`` are shared between paths, and the weight multiplies the
  finished sum of a (weight segment, output segment) term once.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

from .u1d_common import U1DSpec, Block, build_blocks, lit, split_out_segments


@dataclass(frozen=True)
class Tuning:
    ct: int            # channels per tile (= consumer threads per group), multiple of 32
    groups: int        # thread groups that split the output segments (forward only)
    stages: int
    min_blocks: int    # CTAs per SM targeted by __launch_bounds__


def default_tuning(spec: U1DSpec, direction: str) -> Tuning:
    ct = min((spec.u + 31) // 32 * 32, 128 if spec.dtype == "f32" else 64)
    if spec.u % ct != 0 and spec.u > ct:
        # keep tiles uniform when possible
        for cand in (128, 96, 64, 32):
            if cand <= ct and spec.u % cand == 0:
                ct = cand
                break
    if direction == "fwd":
        groups = 2 if spec.out_segs >= 32 else 1
        return Tuning(ct=ct, groups=groups, stages=4, min_blocks=2)
    return Tuning(ct=ct, groups=1, stages=3, min_blocks=2)


def _cfg(spec: U1DSpec, tun: Tuning, extra_bytes: int, ncons_warps: int, emit_empty: bool = True) -> str:
    b = lambda v: "true" if v else "false"
    return f"""namespace cfg {{
using T = {spec.ctype};
constexpr int U = {spec.u}, CT = {tun.ct}, WSEG = {spec.w_segs}, XSEG = {spec.x_segs}, YSEG = {spec.y_segs}, OSEG = {spec.out_segs};
constexpr int STAGES = {tun.stages}, GROUPS = {tun.groups}, NCONS_WARPS = {ncons_warps}, STAGE_EXTRA_BYTES = {extra_bytes};
constexpr bool EMIT_EMPTY_ROWS = {b(emit_empty)};
constexpr bool Y_VEC = {b(spec.y_vec)}, W_SHARED = {b(spec.w_shared)}, X_INDEXED = {b(spec.x_indexed)}, Y_INDEXED = {b(spec.y_indexed)}, SCATTERED = {b(spec.scattered)};
}}  // namespace cfg
"""


_HOST_COMMON = r"""
__device__ int g_status_word;

static int* status_ptr() {
  int* p = nullptr;
  cudaGetSymbolAddress((void**)&p, g_status_word);
  return p;
}

static thread_local char g_err[256];
static int cuda_fail(cudaError_t e) {
  snprintf(g_err, sizeof(g_err), "%s", cudaGetErrorString(e));
  return FASTEQ_CUDA_ERROR;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int fill_graph(const fasteq_u1d_graph* g, fasteq::u1d::Graph* o, int* grid, int ctas_per_sm) {
  if (!g || g->n_edges < 0 || g->n_out_rows < 0) return FASTEQ_INVALID;
  if (cfg::X_INDEXED && g->n_edges > 0 && !g->x_index) return FASTEQ_INVALID;
  if (cfg::Y_INDEXED && g->n_edges > 0 && !g->y_index) return FASTEQ_INVALID;
  if (cfg::SCATTERED && !g->seg_ptr) return FASTEQ_INVALID;
  if (g->n_edges > 0x7fffffffLL || g->n_out_rows > 0x7fffffffLL) return FASTEQ_UNSUPPORTED;
  o->n_edges = g->n_edges; o->n_out_rows = g->n_out_rows; o->x_rows = g->x_rows; o->y_rows = g->y_rows;
  o->x_index = g->x_index; o->y_index = g->y_index; o->seg_ptr = g->seg_ptr; o->perm = g->perm; o->part_ptr = g->part_ptr;
  o->status = status_ptr();
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return cuda_fail(e);
  const long long units = cfg::SCATTERED ? g->n_out_rows : g->n_edges;
  long long want = (long long)sms * ctas_per_sm;
  if (g->part_ptr) want = g->n_parts;
  else if (want > units) want = units;
  if (want < 1) want = 1;
  *grid = (int)want;
  return FASTEQ_OK;
}

extern "C" int fasteq_u1d_device_status(int32_t* code) {
  if (!code) return FASTEQ_INVALID;
  int v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  *code = v;
  return FASTEQ_OK;
}

extern "C" const char* fasteq_last_cuda_error(void) { return g_err; }
"""


def _prelude(spec: U1DSpec, tun: Tuning, extra_bytes: int, ncons_warps: int, emit_empty: bool = True) -> str:
    return ("// Generated by fasteq_b200.codegen.u1d -- do not edit.\n"
            "#include <cstdio>\n#include <cstdint>\n#include <cuda_runtime.h>\n"
            '#include "fasteq_b200.h"\n' + _cfg(spec, tun, extra_bytes, ncons_warps, emit_empty) +
            '#include "u1d_pipeline.cuh"\nusing namespace fasteq;\nusing namespace fasteq::u1d;\n')


def _describe(spec: U1DSpec, tun: Tuning, direction: int, needs=(0, 0, 0), threads=0) -> str:
    return f"""
extern "C" int fasteq_u1d_describe(fasteq_u1d_desc* d) {{
  if (!d) return FASTEQ_INVALID;
  d->abi_version = FASTEQ_ABI_VERSION; d->dtype = {0 if spec.dtype == 'f32' else 1};
  d->u = {spec.u}; d->w_segs = {spec.w_segs}; d->x_segs = {spec.x_segs}; d->y_segs = {spec.y_segs}; d->out_segs = {spec.out_segs};
  d->num_paths = {len(spec.paths)}; d->y_vec = {int(spec.y_vec)}; d->w_shared = {int(spec.w_shared)};
  d->x_indexed = {int(spec.x_indexed)}; d->y_indexed = {int(spec.y_indexed)}; d->scattered = {int(spec.scattered)};
  d->direction = {direction}; d->need_gw = {needs[0]}; d->need_gx = {needs[1]}; d->need_gy = {needs[2]};
  d->ctas_per_sm = {tun.min_blocks}; d->threads = {threads}; d->smem_bytes = SMEM_BYTES;
  return FASTEQ_OK;
}}
"""


# --------------------------------------------------------------------------- forward

def _emit_block_fwd(spec: U1DSpec, b: Block, owned: set, slot_of: Dict[int, int], ind: str) -> List[str]:
    terms = [t for t in b.terms if t.v in owned]
    if not terms:
        return []
    used = sorted({(j, k) for t in terms for j, k, _ in t.items})
    L = [ind + "{"]
    for (j, k) in used:
        L.append(f"{ind}  const T p_{j}_{k} = x{j} * y{k};")
    for t in terms:
        expr = " + ".join(f"{lit(c, spec.dtype)} * p_{j}_{k}" for j, k, c in t.items)
        L.append(f"{ind}  acc[{slot_of[t.v]}] += W({t.i}) * ({expr});")
    L.append(ind + "}")
    return L


def emit_forward(spec: U1DSpec, tun: Tuning) -> str:
    blocks = build_blocks(spec)
    G = tun.groups
    owners = split_out_segments(blocks, spec.out_segs, G)
    max_slots = max(1, max(len(o) for o in owners))
    ncons_warps = G * tun.ct // 32
    threads = G * tun.ct + 32
    src = [_prelude(spec, tun, 0, ncons_warps)]
    src.append(f"""
constexpr int NTHREADS = {threads};
constexpr int W_SHARED_BYTES = cfg::W_SHARED ? WSEG * CT * (int)sizeof(T) : 0;
constexpr int SMEM_BYTES = BAR_BYTES + STAGES * STAGE_BYTES + W_SHARED_BYTES;

__global__ void __launch_bounds__(NTHREADS, {tun.min_blocks})
fasteq_u1d_fwd_kernel(const Graph g, const T* __restrict__ w, const T* __restrict__ x, const T* __restrict__ y,
                      T* __restrict__ out) {{
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + STAGES;
  unsigned char* stages = smem + BAR_BYTES;
  init_barriers(full, empty);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == cfg::NCONS_WARPS) {{
    Producer p{{g, w, x, y, stages, full, empty, lane, 0u}};
    p.run([](unsigned char*, int) {{}}, [](int, int, int) {{}});
    return;
  }}
  const int grp = threadIdx.x / CT, ch = threadIdx.x % CT;
  T acc[{max_slots}];
#pragma unroll
  for (int s = 0; s < {max_slots}; ++s) acc[s] = T(0);
  uint32_t it = 0;
  for (;;) {{
    const int stage = it % STAGES;
    const uint32_t ph = (it / STAGES) & 1u;
    mbar_wait(&full[stage], ph, g.status);
    const unsigned char* st = stages + (size_t)stage * STAGE_BYTES;
    const Meta m = *reinterpret_cast<const Meta*>(st + OFF_META);
    const int valid = (U - m.ct * CT) < CT ? (U - m.ct * CT) : CT;
    const bool live = ch < valid;
    if ((m.flags & F_DATA) && live) {{
      const T* sw = reinterpret_cast<const T*>(st + OFF_W) + ch;
      const T* sx = reinterpret_cast<const T*>(st + OFF_X) + ch;
      const T* sy = reinterpret_cast<const T*>(st + OFF_Y){' + ch' if spec.y_vec else ''};
#define W(i) sw[(i) * CT]
""")
    # shared weights are read straight from global memory (one row for the whole launch, L1/L2 resident)
    if spec.w_shared:
        src[-1] = src[-1].replace("#define W(i) sw[(i) * CT]", "#define W(i) __ldg(w + (size_t)(i) * U + m.ct * CT + ch)")
        src[-1] = src[-1].replace("      const T* sw = reinterpret_cast<const T*>(st + OFF_W) + ch;\n", "")
    body = []
    for j in range(spec.x_segs):
        body.append(f"      const T x{j} = sx[{j} * CT];")
    if spec.y_vec:
        for k in range(spec.y_segs):
            body.append(f"      const T y{k} = sy[{k} * CT];")
    else:
        for k in range(spec.y_segs):
            body.append(f"      const T y{k} = sy[{k}];")
    for gi in range(G):
        owned = set(owners[gi])
        slot_of = {v: s for s, v in enumerate(owners[gi])}
        cond = f"      if (grp == {gi}) {{" if G > 1 else "      {"
        body.append(cond)
        for b in blocks:
            body += _emit_block_fwd(spec, b, owned, slot_of, "        ")
        body.append("      }")
    body.append("#undef W")
    body.append("    }")
    # store on the last edge of a segment
    body.append("    if (m.flags & F_LAST) {")
    body.append("      if (live) {")
    body.append("        T* o = out + (size_t)m.row * OSEG * U + (size_t)m.ct * CT + ch;")
    for gi in range(G):
        cond = f"        if (grp == {gi}) {{" if G > 1 else "        {"
        body.append(cond)
        for s, v in enumerate(owners[gi]):
            body.append(f"          o[{v} * U] = acc[{s}];")
        body.append("        }")
    body.append("      }")
    body.append("#pragma unroll")
    body.append(f"      for (int s = 0; s < {max_slots}; ++s) acc[s] = T(0);")
    body.append("    }")
    body.append("    __syncwarp();")
    body.append("    if (lane == 0) mbar_arrive(&empty[stage]);")
    body.append("    ++it;")
    body.append("    if (m.flags & F_DONE) break;")
    body.append("  }")
    body.append("}")
    src.append("\n".join(body))
    src.append(_HOST_COMMON)
    src.append(_describe(spec, tun, 0, threads=threads))
    src.append(f"""
extern "C" int fasteq_u1d_forward(const fasteq_u1d_graph* gh, const void* w, const void* x, const void* y, void* out,
                                  fasteq_stream_t stream) {{
  Graph g; int grid = 1;
  int rc = fill_graph(gh, &g, &grid, {tun.min_blocks});
  if (rc != FASTEQ_OK) return rc;
  if (gh->n_out_rows == 0 && gh->n_edges == 0) return FASTEQ_OK;
  if (!out || (gh->n_edges > 0 && (!w || !x || !y))) return FASTEQ_INVALID;
  g.bulk_ok = aligned16(w) && aligned16(x) && aligned16(y) && ((U * sizeof(T)) % 16 == 0) && ((CT * sizeof(T)) % 16 == 0);
  cudaError_t e = cudaFuncSetAttribute(fasteq_u1d_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return cuda_fail(e);
  fasteq_u1d_fwd_kernel<<<grid, NTHREADS, SMEM_BYTES, (cudaStream_t)stream>>>(
      g, (const T*)w, (const T*)x, (const T*)y, (T*)out);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return FASTEQ_OK;
}}

extern "C" int fasteq_u1d_backward(const fasteq_u1d_graph*, const void*, const void*, const void*, const void*, void*,
                                   void*, void*, fasteq_stream_t) {{
  return FASTEQ_UNSUPPORTED;  // this module holds the forward kernel only
}}
""")
    return "\n".join(src)


# --------------------------------------------------------------------------- backward

def emit_backward(spec: U1DSpec, tun: Tuning, need_gw: bool, need_gx: bool, need_gy: bool) -> str:
    """Backward module: grad_w, grad_x, grad_y of ``sum(out * grad_out)`` (any subset).

    Per edge and channel, with ``g = grad_out[v]``:  ``gw[i] += g * sum c p_jk``,
    ``q_jk += c * w[i] * g``, then ``gx[j] += q_jk * y[k]`` and ``gy[k] += q_jk * x[j]``
    (fasteq/ops/auto_schedule/models.py:145-152 states the three gradient terms).
    The receiver's grad_out row is staged once per receiver segment; gx goes out through
    ``red.global.add`` when x is gathered; a scalar-y gradient is summed over channels
    with warp shuffles, then across warps by the producer warp when the stage is recycled.
    """
    assert tun.groups == 1
    blocks = build_blocks(spec)
    ncons_warps = tun.ct // 32
    threads = tun.ct + 32
    scalar_gy = need_gy and not spec.y_vec
    extra = ncons_warps * spec.y_segs * spec.elem_bytes if scalar_gy else 0
    extra = (extra + 15) // 16 * 16
    T = spec.ctype
    src = [_prelude(spec, tun, extra, ncons_warps, emit_empty=False)]
    src.append(f"""
constexpr int NTHREADS = {threads};
constexpr int NGO = {tun.min_blocks and 1};            // grad_out row buffers
constexpr int GO_BYTES = round_up(OSEG * CT * (int)sizeof(T), 128);
constexpr int SMEM_BYTES = BAR_BYTES + STAGES * STAGE_BYTES + NGO * GO_BYTES;
constexpr bool NEED_GW = {str(need_gw).lower()}, NEED_GX = {str(need_gx).lower()}, NEED_GY = {str(need_gy).lower()};
constexpr bool GY_ATOMIC = cfg::Y_INDEXED || (!cfg::Y_VEC && NCT > 1);

__global__ void __launch_bounds__(NTHREADS, {tun.min_blocks})
fasteq_u1d_bwd_kernel(const Graph g, const T* __restrict__ go, const T* __restrict__ w, const T* __restrict__ x,
                      const T* __restrict__ y, T* __restrict__ gw, T* __restrict__ gx, T* __restrict__ gy) {{
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + STAGES;
  uint64_t* go_full = empty + STAGES;
  uint64_t* go_empty = go_full + NGO;
  unsigned char* stages = smem + BAR_BYTES;
  unsigned char* gobuf = stages + STAGES * STAGE_BYTES;
  if (threadIdx.x == 0) {{
    for (int b = 0; b < NGO; ++b) {{ mbar_init(&go_full[b], 33); mbar_init(&go_empty[b], cfg::NCONS_WARPS); }}
  }}
  init_barriers(full, empty);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == cfg::NCONS_WARPS) {{
    Producer p{{g, w, x, y, stages, full, empty, lane, 0u}};
    uint32_t nseg = 0;
    auto begin = [&](int row, int ct, int ln) {{
      // stage the receiver's grad_out tile once per segment
      const int b = nseg % NGO;
      const uint32_t ph = (nseg / NGO) & 1u;
      mbar_wait(&go_empty[b], ph ^ 1u, g.status);
      const int valid = (U - ct * CT) < CT ? (U - ct * CT) : CT;
      if (ln == 0) mbar_arrive_expect_tx(&go_full[b], g.bulk_ok ? (uint32_t)(OSEG * valid * sizeof(T)) : 0u);
      __syncwarp();
      copy_tile(gobuf + (size_t)b * GO_BYTES, go + (size_t)row * OSEG * U, OSEG, ct, valid, g.bulk_ok != 0, &go_full[b], ln);
      cp_async_arrive_noinc(&go_full[b]);
      ++nseg;
    }};
    auto flush = [&](unsigned char* st, int ln) {{
      if ({'true' if scalar_gy else 'false'}) {{
        const Meta pm = *reinterpret_cast<const Meta*>(st + OFF_META);
        if (pm.flags & F_DATA) {{
          const T* part = reinterpret_cast<const T*>(st + OFF_EXTRA);
          for (int k = ln; k < YSEG; k += 32) {{
            T s = T(0);
#pragma unroll
            for (int wp = 0; wp < cfg::NCONS_WARPS; ++wp) s += part[wp * YSEG + k];
            T* dst = gy + (size_t)pm.yr * YSEG + k;
            if (GY_ATOMIC) red_add(dst, s); else *dst = s;
          }}
        }}
      }}
    }};
    p.run(flush, begin);
    return;
  }}
  const int ch = threadIdx.x;
  uint32_t it = 0, nseg = 0;
""")
    L: List[str] = []
    if spec.w_shared and need_gw:
        L.append(f"  T gws[{spec.w_segs}];")
        L.append("#pragma unroll")
        L.append(f"  for (int i = 0; i < {spec.w_segs}; ++i) gws[i] = T(0);")
        L.append("  int gws_ct = 0;")
    L.append("""  for (;;) {
    const int stage = it % STAGES;
    const uint32_t ph = (it / STAGES) & 1u;
    mbar_wait(&full[stage], ph, g.status);
    unsigned char* st = stages + (size_t)stage * STAGE_BYTES;
    const Meta m = *reinterpret_cast<const Meta*>(st + OFF_META);
    const int valid = (U - m.ct * CT) < CT ? (U - m.ct * CT) : CT;
    const bool live = ch < valid;
    const int gb = nseg % NGO;
    if (m.flags & F_FIRST) mbar_wait(&go_full[gb], (nseg / NGO) & 1u, g.status);""")
    if spec.w_shared and need_gw:
        L.append("    if ((m.flags & (F_DATA | F_DONE)) && (m.ct != gws_ct || (m.flags & F_DONE))) {")
        L.append("      if (ch < ((U - gws_ct * CT) < CT ? (U - gws_ct * CT) : CT)) {")
        for i in range(spec.w_segs):
            L.append(f"        red_add(gw + (size_t){i} * U + gws_ct * CT + ch, gws[{i}]); gws[{i}] = T(0);")
        L.append("      }")
        L.append("      gws_ct = m.ct;")
        L.append("    }")
    if scalar_gy:
        for k in range(spec.y_segs):
            L.append(f"    T gy{k} = T(0);")
    L.append("    if ((m.flags & F_DATA) && live) {")
    L.append("      const T* sx = reinterpret_cast<const T*>(st + OFF_X) + ch;")
    L.append(f"      const T* sy = reinterpret_cast<const T*>(st + OFF_Y){' + ch' if spec.y_vec else ''};")
    L.append("      const T* sgo = reinterpret_cast<const T*>(gobuf + (size_t)gb * GO_BYTES) + ch;")
    if spec.w_shared:
        L.append("#define W(i) __ldg(w + (size_t)(i) * U + m.ct * CT + ch)")
    else:
        L.append("      const T* sw = reinterpret_cast<const T*>(st + OFF_W) + ch;")
        L.append("#define W(i) sw[(i) * CT]")
    L.append("#define GO(v) sgo[(v) * CT]")
    for j in range(spec.x_segs):
        L.append(f"      const T x{j} = sx[{j} * CT];")
    for k in range(spec.y_segs):
        L.append(f"      const T y{k} = sy[{k}{' * CT' if spec.y_vec else ''}];")
    if need_gx:
        for j in range(spec.x_segs):
            L.append(f"      T gx{j} = T(0);")
    if need_gy and spec.y_vec:
        for k in range(spec.y_segs):
            L.append(f"      T gy{k} = T(0);")
    # which block is the last to touch weight segment i
    last_block_of_i: Dict[int, int] = {}
    for bi, b in enumerate(blocks):
        for t in b.terms:
            last_block_of_i[t.i] = bi
    if need_gw:
        for i in sorted(last_block_of_i):
            L.append(f"      T gw{i} = T(0);")
        if not spec.w_shared:
            L.append("      T* gwp = gw + (size_t)m.e * WSEG * U + (size_t)m.ct * CT + ch;")
    need_q = need_gx or need_gy
    for bi, b in enumerate(blocks):
        L.append("      {")
        if need_gw:
            for (j, k) in b.products:
                L.append(f"        const T p_{j}_{k} = x{j} * y{k};")
        if need_q:
            for (j, k) in b.products:
                L.append(f"        T q_{j}_{k} = T(0);")
        for t in b.terms:
            L.append(f"        {{ const T gv = GO({t.v});")
            if need_gw:
                expr = " + ".join(f"{lit(c, spec.dtype)} * p_{j}_{k}" for j, k, c in t.items)
                L.append(f"          gw{t.i} += gv * ({expr});")
            if need_q:
                L.append(f"          const T gp = W({t.i}) * gv;")
                for j, k, c in t.items:
                    L.append(f"          q_{j}_{k} += {lit(c, spec.dtype)} * gp;")
            L.append("        }")
        if need_gx:
            for (j, k) in b.products:
                L.append(f"        gx{j} += q_{j}_{k} * y{k};")
        if need_gy:
            for (j, k) in b.products:
                L.append(f"        gy{k} += q_{j}_{k} * x{j};")
        if need_gw:
            for i in sorted(i for i, last in last_block_of_i.items() if last == bi):
                if spec.w_shared:
                    L.append(f"        gws[{i}] += gw{i};")
                else:
                    L.append(f"        gwp[{i} * U] = gw{i};")
        L.append("      }")
    if need_gw and not spec.w_shared:
        # weight segments no path touches still need a defined gradient
        for i in range(spec.w_segs):
            if i not in last_block_of_i:
                L.append(f"      gwp[{i} * U] = T(0);")
    if need_gx:
        L.append("      T* gxp = gx + (size_t)m.xr * XSEG * U + (size_t)m.ct * CT + ch;")
        for j in range(spec.x_segs):
            if spec.x_indexed:
                L.append(f"      red_add(gxp + {j} * U, gx{j});")
            else:
                L.append(f"      gxp[{j} * U] = gx{j};")
    if need_gy and spec.y_vec:
        L.append("      T* gyp = gy + (size_t)m.yr * YSEG * U + (size_t)m.ct * CT + ch;")
        for k in range(spec.y_segs):
            if spec.y_indexed:
                L.append(f"      red_add(gyp + {k} * U, gy{k});")
            else:
                L.append(f"      gyp[{k} * U] = gy{k};")
    L.append("#undef W")
    L.append("#undef GO")
    L.append("    }")
    if scalar_gy:
        L.append("    if (m.flags & F_DATA) {")
        L.append("      T* part = reinterpret_cast<T*>(st + OFF_EXTRA) + warp * YSEG;")
        for k in range(spec.y_segs):
            L.append(f"      gy{k} = warp_sum(gy{k});")
        L.append("      if (lane == 0) {")
        for k in range(spec.y_segs):
            L.append(f"        part[{k}] = gy{k};")
        L.append("      }")
        L.append("    }")
    L.append("""    __syncwarp();
    if (lane == 0) {
      if (m.flags & F_LAST) mbar_arrive(&go_empty[gb]);
      mbar_arrive(&empty[stage]);
    }
    if (m.flags & F_LAST) ++nseg;
    ++it;
    if (m.flags & F_DONE) break;
  }
}""")
    src.append("\n".join(L))
    src.append(_HOST_COMMON)
    src.append(_describe(spec, tun, 1, (int(need_gw), int(need_gx), int(need_gy)), threads=threads))
    zero = []
    if need_gw and spec.w_shared:
        zero.append("if (gw) { e = cudaMemsetAsync(gw, 0, (size_t)WSEG * U * sizeof(T), s); if (e != cudaSuccess) return cuda_fail(e); }")
    if need_gx and spec.x_indexed:
        zero.append("if (gx) { e = cudaMemsetAsync(gx, 0, (size_t)gh->x_rows * XSEG * U * sizeof(T), s); if (e != cudaSuccess) return cuda_fail(e); }")
    if need_gy:
        ycols = "YSEG * U" if spec.y_vec else "YSEG"
        if spec.y_indexed:
            zero.append(f"if (gy) {{ e = cudaMemsetAsync(gy, 0, (size_t)gh->y_rows * {ycols} * sizeof(T), s); if (e != cudaSuccess) return cuda_fail(e); }}")
        elif not spec.y_vec:
            zero.append(f"if (gy && GY_ATOMIC) {{ e = cudaMemsetAsync(gy, 0, (size_t)gh->n_edges * {ycols} * sizeof(T), s); if (e != cudaSuccess) return cuda_fail(e); }}")
    src.append(f"""
extern "C" int fasteq_u1d_forward(const fasteq_u1d_graph*, const void*, const void*, const void*, void*, fasteq_stream_t) {{
  return FASTEQ_UNSUPPORTED;  // this module holds the backward kernel only
}}

extern "C" int fasteq_u1d_backward(const fasteq_u1d_graph* gh, const void* go, const void* w, const void* x,
                                   const void* y, void* gw, void* gx, void* gy, fasteq_stream_t stream) {{
  Graph g; int grid = 1;
  int rc = fill_graph(gh, &g, &grid, {tun.min_blocks});
  if (rc != FASTEQ_OK) return rc;
  if ((NEED_GW && !gw) || (NEED_GX && !gx) || (NEED_GY && !gy)) return FASTEQ_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  {' '.join(zero)}
  if (gh->n_edges == 0) return FASTEQ_OK;
  if (!go || !w || !x || !y) return FASTEQ_INVALID;
  g.bulk_ok = aligned16(w) && aligned16(x) && aligned16(y) && aligned16(go) && ((U * sizeof(T)) % 16 == 0) &&
              ((CT * sizeof(T)) % 16 == 0);
  e = cudaFuncSetAttribute(fasteq_u1d_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return cuda_fail(e);
  fasteq_u1d_bwd_kernel<<<grid, NTHREADS, SMEM_BYTES, s>>>(g, (const T*)go, (const T*)w, (const T*)x, (const T*)y,
                                                          (T*)gw, (T*)gx, (T*)gy);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return FASTEQ_OK;
}}
""")
    return "\n".join(src)
