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

from .u1d_common import U1DSpec, Block, build_blocks, lit, restrict_blocks, split_out_segments, split_w_segments
from .sh import SH_DEVICE_STUB, emit_sh_device


@dataclass(frozen=True)
class Tuning:
    ct: int            # channels per tile, multiple of 32 * vec
    groups: int        # thread groups that split the output segments (forward only)
    stages: int
    min_blocks: int    # CTAs per SM targeted by __launch_bounds__
    vec: int = 1       # channels per thread: 2 = packed f32x2 arithmetic (FP32, even u)
    two_pass: bool = False  # backward: evaluate a block once for grad_w and once for grad_x / grad_y
    pipes: int = 1     # independent producer/consumer pipelines per CTA (keeps all four SM sub-partitions busy)
    go_smem: bool = True   # backward: stage the receiver's grad_out row in shared memory (else read it through L1)
    prefetch: int = 0      # ring-fuls by which the producer asks rows into L2 ahead of the stage fills (0 = no prefetch)
    go_tmem: bool = False  # backward: park the receiver's grad_out row in tensor memory (one lane per thread) instead


def default_tuning(spec: U1DSpec, direction: str) -> Tuning:
    """Defaults from sweeps on B200 (128-channel FP32 signatures with 55 and 106 output segments).

    With 128-channel FP32 tiles both directions use packed two-channel arithmetic; the forward keeps
    the receiver row in registers (two thread groups split the output segments when there are too
    many for one thread).  When the receiver row fits one thread group, one CTA of four pipelines
    (eight consumer warps) per SM measured 5-10 % faster than two CTAs of two pipelines; signatures
    whose ring stage is only a few KB (scalar sender rows) run two such CTAs with deeper rings.  Other shapes: one channel per
    thread, as many pipelines per CTA as give four consumer warps, residency from the shared-memory
    footprint."""
    f32 = spec.dtype == "f32"
    packed = f32 and spec.u % 64 == 0
    e = spec.elem_bytes
    if packed:
        ct = 128 if spec.u % 128 == 0 else 64
        vec, wpg = 2, ct // 64                        # consumer warps per thread group
    else:
        cap = 128 if f32 else 64
        ct = min((spec.u + 31) // 32 * 32, cap)
        if spec.u > ct and spec.u % ct != 0:
            for cand in (128, 96, 64, 32):
                if cand <= ct and spec.u % cand == 0:
                    ct = cand
                    break
        vec, wpg = 1, ct // 32
    big = spec.out_segs > 64
    wide = packed and ct == 128 and not big                    # 128-channel tiles, receiver row fits one thread group
    small = _stage_bytes(spec, ct, 0) <= 4096                  # e.g. a scalar-only sender row (first interaction layer)
    if direction == "fwd":
        groups = 2 if big else 1
        pipes = max(1, 4 // (groups * wpg))                    # four consumer warps per CTA
        stages = 6 if f32 else 4
        if wide:                                               # one CTA of four pipelines (eight consumer warps) per SM
            pipes = 4
            if small:                                          # few bytes per stage: deeper rings, two such CTAs
                stages = 10
        elif packed and big and ct == 128:                     # two thread groups per pipeline: two pipelines, shorter rings
            pipes, stages = 2, 5
        per_pipe = 256 + stages * _stage_bytes(spec, ct, 0)
        fit = max(1, _SMEM_BUDGET // per_pipe)                 # pipelines one SM can hold
        if fit < pipes:
            pipes = fit
        if packed:
            residency = 1 if (big or (wide and not small)) else 2
        else:
            residency = 2 if (big or not f32) else 3
        return Tuning(ct=ct, groups=groups, stages=stages, pipes=pipes, vec=vec, min_blocks=max(1, min(residency, fit // pipes)))
    pipes = 4 if wide else max(1, 4 // wpg)
    extra = wpg * spec.y_segs * e
    go_bytes = (spec.out_segs * ct * e + 127) // 128 * 128
    stages = 4 if (wide and small) else 3
    per_pipe = 256 + stages * _stage_bytes(spec, ct, extra) + go_bytes
    if pipes * per_pipe > _SMEM_BUDGET:
        stages = 2
        per_pipe = 256 + stages * _stage_bytes(spec, ct, extra) + go_bytes
    fit = max(1, _SMEM_BUDGET // per_pipe)
    if fit < pipes:
        pipes = fit
    if packed:
        residency = 1 if (big or (wide and not small)) else 2
    else:
        residency = 1 if big else (3 if f32 else 2)
    return Tuning(ct=ct, groups=1, stages=stages, pipes=pipes, vec=vec, min_blocks=max(1, min(residency, fit // pipes)))


_SMEM_BUDGET = 220 * 1024


def _stage_bytes(spec: U1DSpec, ct: int, extra: int) -> int:
    """Shared memory of one ring stage (mirrors the layout constants of u1d_pipeline.cuh)."""
    e = spec.elem_bytes
    w = 0 if spec.w_shared else spec.w_segs * ct * e
    x = spec.x_segs * ct * e
    y = spec.y_segs * ct * e if spec.y_vec else (spec.y_segs * e + 15) // 16 * 16
    return (w + x + y + 32 + extra + 127) // 128 * 128

def _cfg(spec: U1DSpec, tun: Tuning, extra_bytes: int, ncons_warps: int, emit_empty: bool = True) -> str:
    b = lambda v: "true" if v else "false"
    vtype = "float2" if tun.vec == 2 else spec.ctype
    return f"""namespace cfg {{
using T = {spec.ctype};
using V = {vtype};   // what one thread carries per segment: one channel, or two packed FP32 channels
constexpr int U = {spec.u}, CT = {tun.ct}, WSEG = {spec.w_segs}, XSEG = {spec.x_segs}, YSEG = {spec.y_segs}, OSEG = {spec.out_segs};
constexpr int STAGES = {tun.stages}, GROUPS = {tun.groups}, PIPES = {tun.pipes}, NCONS_WARPS = {ncons_warps}, STAGE_EXTRA_BYTES = {extra_bytes};
constexpr int PREFETCH = {tun.prefetch};
constexpr bool EMIT_EMPTY_ROWS = {b(emit_empty)}, BEGIN_PER_SEGMENT = {b(not emit_empty)};
constexpr bool Y_VEC = {b(spec.y_vec)}, W_SHARED = {b(spec.w_shared)}, X_INDEXED = {b(spec.x_indexed)}, Y_INDEXED = {b(spec.y_indexed)}, SCATTERED = {b(spec.scattered)};
constexpr bool Y_SH = {b(bool(spec.y_sh))};   // the y operand holds edge vectors [rows, 3]; the producer evaluates their harmonics
}}  // namespace cfg
""" + (emit_sh_device(spec.y_sh[0], spec.dtype, spec.y_sh[1], spec.y_sh[2]) if spec.y_sh else SH_DEVICE_STUB)


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
  long long want = (long long)sms * ctas_per_sm * cfg::PIPES;   // pipelines
  if (g->part_ptr) want = g->n_parts;
  else if (want > units) want = units;
  if (want < 1) want = 1;
  o->n_vblocks = (int)want;
  *grid = (int)((want + cfg::PIPES - 1) / cfg::PIPES);
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


_NOALLOC_FORWARD = r"""
// ---------------------------------------------------------------------------------------------
// Forward without any allocation.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need the operator:
// a molecular-dynamics engine plug-in that was handed a fixed device arena at start-up, or a
// real-time control loop where an allocation (an implicit device synchronisation) is forbidden.  The regular entry point leaves
// the CSR offsets and the per-CTA partition to the caller, who must own buffers for them.  This
// variant builds both into a fixed array that lives inside this library image and then runs the
// same forward kernel on them.
//
// Limits and rules:
//   * at most FASTEQ_NOALLOC_MAX_ROWS output rows (receivers); larger calls are refused with
//     FASTEQ_UNSUPPORTED and nothing is launched;
//   * edges must already be sorted by receiver (there is no room for a permutation);
//   * the array (about 1 MB) belongs to THIS module (one generated library per operator signature; a
//     process that loads several forward modules holds one array per module) and is reserved on every
//     GPU that loads it until the process exits; all calls into the module share it.  Every entry a call reads is written earlier in the same
//     call, so nothing has to be cleared between calls, but two calls that overlap on the GPU
//     (different streams, or different host threads) overwrite each other's offsets: serialise them;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress,
//     with that device current).  Make that first call outside of any stream capture.  The look-up
//     may run on several host threads at once (they store the same address);
//   * a call that is refused (bad argument, size limit, misaligned operand) launches nothing, so it
//     cannot disturb the offsets of a call in flight;
//   * receiver indices outside [0, n_out_rows) are not reported: such edges belong to no row and
//     are left out.
// ---------------------------------------------------------------------------------------------
#define FASTEQ_NOALLOC_MAX_ROWS 262144
#define FASTEQ_NOALLOC_MAX_PARTS 4096
static __device__ __align__(256) int g_noalloc_scratch[FASTEQ_NOALLOC_MAX_ROWS + 1 + FASTEQ_NOALLOC_MAX_PARTS + 1];

namespace {
__global__ void na_build_csr(const int* __restrict__ dst, long long n_edges, long long n_rows, int* __restrict__ seg_ptr) {
  const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (r > n_rows) return;
  long long lo = 0, hi = n_edges;
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if ((long long)dst[mid] < r) lo = mid + 1; else hi = mid;
  }
  seg_ptr[r] = (int)lo;
}
__global__ void na_partition(const int* __restrict__ seg_ptr, long long n_rows, long long n_edges, int n_parts,
                             int* __restrict__ part_ptr) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p > n_parts) return;
  if (p == n_parts) { part_ptr[p] = (int)n_rows; return; }
  const long long target = (n_edges + n_rows) * p / n_parts;
  long long lo = 0, hi = n_rows;
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if ((long long)seg_ptr[mid] + mid < target) lo = mid + 1; else hi = mid;
  }
  part_ptr[p] = (int)lo;
}
constexpr int kMaxDevices = 64;
std::atomic<int*> g_noalloc_addr[kMaxDevices];   // device address of g_noalloc_scratch per device, filled on first use
}  // namespace

extern "C" int fasteq_u1d_forward_noalloc(const int32_t* dst_sorted, const int32_t* x_index, int64_t n_edges,
                                          int64_t n_out_rows, int64_t x_rows, const void* w, const void* x,
                                          const void* y, void* out, fasteq_stream_t stream) {
  if (!cfg::SCATTERED || cfg::Y_INDEXED) return FASTEQ_UNSUPPORTED;
  if (n_edges < 0 || n_out_rows < 0 || n_edges > 0x7fffffffLL) return FASTEQ_INVALID;
  if (n_out_rows > FASTEQ_NOALLOC_MAX_ROWS) {
    snprintf(g_err, sizeof(g_err), "fasteq_u1d_forward_noalloc: %lld output rows exceed the built-in scratch (%d rows)",
             (long long)n_out_rows, FASTEQ_NOALLOC_MAX_ROWS);
    return FASTEQ_UNSUPPORTED;
  }
  if (n_out_rows == 0) return FASTEQ_OK;
  if (!out || (n_edges > 0 && (!dst_sorted || !w || !x || !y || (cfg::X_INDEXED && !x_index)))) return FASTEQ_INVALID;
  // everything fasteq_u1d_forward would refuse is refused here, before anything touches the shared array
  if (VEC == 2 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(w)) & 7u)) return FASTEQ_INVALID;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= kMaxDevices) return FASTEQ_UNSUPPORTED;
  int* seg_ptr = g_noalloc_addr[dev].load(std::memory_order_acquire);
  if (!seg_ptr) {
    // once per device, with that device current: the symbol's name is only a host-side handle
    e = cudaGetSymbolAddress((void**)&seg_ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return cuda_fail(e);
    g_noalloc_addr[dev].store(seg_ptr, std::memory_order_release);
  }
  int* part_ptr = seg_ptr + FASTEQ_NOALLOC_MAX_ROWS + 1;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return cuda_fail(e);
  long long n_parts = (long long)sms * @MINB@ * cfg::PIPES;
  if (n_parts > n_out_rows) n_parts = n_out_rows;
  if (n_parts > FASTEQ_NOALLOC_MAX_PARTS) n_parts = FASTEQ_NOALLOC_MAX_PARTS;
  cudaStream_t s = (cudaStream_t)stream;
  na_build_csr<<<(int)((n_out_rows + 1 + 255) / 256), 256, 0, s>>>(dst_sorted, n_edges, n_out_rows, seg_ptr);
  na_partition<<<(int)((n_parts + 1 + 255) / 256), 256, 0, s>>>(seg_ptr, n_out_rows, n_edges, (int)n_parts, part_ptr);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  fasteq_u1d_graph gh;
  gh.n_edges = n_edges; gh.n_out_rows = n_out_rows; gh.x_rows = x_rows; gh.y_rows = n_edges;
  gh.x_index = x_index; gh.y_index = nullptr; gh.seg_ptr = seg_ptr; gh.perm = nullptr; gh.part_ptr = part_ptr;
  gh.n_parts = (int32_t)n_parts;
  return fasteq_u1d_forward(&gh, w, x, y, out, stream);
}
"""


def _prelude(spec: U1DSpec, tun: Tuning, extra_bytes: int, ncons_warps: int, emit_empty: bool = True) -> str:
    return ("// Generated by fasteq_b200.codegen.u1d -- do not edit.\n"
            "#include <atomic>\n#include <cstdio>\n#include <cstdint>\n#include <cuda_runtime.h>\n"
            '#include "fasteq_b200.h"\n' + _cfg(spec, tun, extra_bytes, ncons_warps, emit_empty) +
            '#include "u1d_pipeline.cuh"\nusing namespace fasteq;\nusing namespace fasteq::u1d;\n'
            "using V = cfg::V;\nusing VS = VT<V>;\nconstexpr int VEC = VS::N;\nconstexpr int TPG = CT / VEC;  // threads per group\n")


def _describe(spec: U1DSpec, tun: Tuning, direction: int, needs=(0, 0, 0), threads=0) -> str:
    return f"""
extern "C" int fasteq_u1d_describe(fasteq_u1d_desc* d) {{
  if (!d) return FASTEQ_INVALID;
  d->abi_version = FASTEQ_ABI_VERSION; d->dtype = {0 if spec.dtype == 'f32' else 1};
  d->u = {spec.u}; d->w_segs = {spec.w_segs}; d->x_segs = {spec.x_segs}; d->y_segs = {spec.y_segs}; d->out_segs = {spec.out_segs};
  d->num_paths = {len(spec.paths)}; d->y_vec = {int(spec.y_vec)}; d->w_shared = {int(spec.w_shared)};
  d->x_indexed = {int(spec.x_indexed)}; d->y_indexed = {int(spec.y_indexed)}; d->scattered = {int(spec.scattered)};
  d->direction = {direction}; d->need_gw = {needs[0]}; d->need_gx = {needs[1]}; d->need_gy = {needs[2]};
  d->ctas_per_sm = {tun.min_blocks * tun.pipes}; d->threads = {threads}; d->smem_bytes = SMEM_BYTES;
  return FASTEQ_OK;
}}
"""


def _check_tuning(spec: U1DSpec, tun: Tuning) -> None:
    if tun.vec not in (1, 2):
        raise ValueError("vec must be 1 or 2")
    if tun.vec == 2 and (spec.dtype != "f32" or spec.u % 2):
        raise ValueError("packed arithmetic needs FP32 and an even channel count")
    if tun.ct % (32 * tun.vec):
        raise ValueError("ct must be a multiple of 32 * vec")
    if tun.go_tmem:
        if tun.go_smem or tun.groups != 1 or spec.u % tun.ct:
            raise ValueError("the tensor-memory gradient row needs whole channel tiles, one thread group and no shared-memory tile")
        if tmem_columns(spec, tun) * max(1, tun.min_blocks) > 512:
            raise ValueError("the gradient rows of this layout (times the resident CTAs asked for) do not fit 512 columns of tensor memory")
        if tun.stages > 13:
            raise ValueError("at most 13 stages beside the tensor-memory slot")


def tmem_columns(spec: U1DSpec, tun: Tuning) -> int:
    """Tensor-memory columns the ``go_tmem`` layout allocates: consumer warps with the same warp index modulo four share
    a lane quarter and stack their rows (vec * out_segs values of one or two 32-bit columns each); allocations are powers
    of two >= 32."""
    ncons = tun.pipes * tun.groups * (tun.ct // tun.vec) // 32
    need = (ncons + 3) // 4 * tun.vec * spec.out_segs * (spec.elem_bytes // 4)
    cols = 32
    while cols < need:
        cols *= 2
    return cols


def _vlit(c: float, dtype: str) -> str:
    return f"VS::bc({lit(c, dtype)})"


def _sum_expr(items, dtype: str) -> List[str]:
    """Statements computing ``t = sum c * p_j_k`` with fused multiply-adds."""
    out = []
    for n, (j, k, c) in enumerate(items):
        if n == 0:
            out.append(f"V t = p_{j}_{k};" if c == 1.0 else f"V t = vmul({_vlit(c, dtype)}, p_{j}_{k});")
        else:
            out.append(f"t = vfma({_vlit(c, dtype)}, p_{j}_{k}, t);")
    return out


def _load_xy(spec: U1DSpec, ind: str) -> List[str]:
    L = [f"{ind}const V x{j} = VS::ld(sx + {j} * CT);" for j in range(spec.x_segs)]
    if spec.y_vec:
        L += [f"{ind}const V y{k} = VS::ld(sy + {k} * CT);" for k in range(spec.y_segs)]
    else:
        L += [f"{ind}const V y{k} = VS::bc(sy[{k}]);" for k in range(spec.y_segs)]
    return L


# --------------------------------------------------------------------------- forward

def _diagonal_runs(terms) -> List[Tuple[str, int, int, float, List[Tuple[int, int]]]]:
    """For a block whose terms all have one product: runs ``(kind, i, shared, c, [(other, v), ...])``.  ``kind`` "x":
    the outputs ``v`` share ``c * w[i] * x[shared]`` and differ in ``y[other]`` (an l1 = 0 coupling); "y": they share
    ``c * w[i] * y[shared]`` and differ in ``x[other]`` (l2 = 0).  One multiply per run and one FMA per output forward;
    backward, the sum over the run's outputs is formed once before it meets the shared operand."""
    by_ic: Dict[Tuple[int, float], List[Tuple[int, int, int]]] = {}
    for t in terms:
        (j, k, c), = t.items
        by_ic.setdefault((t.i, c), []).append((j, k, t.v))
    runs = []
    for (i, c), jkv in by_ic.items():
        if len({j for j, _, _ in jkv}) <= len({k for _, k, _ in jkv}):
            groups: Dict[int, List[Tuple[int, int]]] = {}
            for j, k, v in jkv:
                groups.setdefault(j, []).append((k, v))
            runs += [("x", i, j, c, kv) for j, kv in groups.items()]
        else:
            groups = {}
            for j, k, v in jkv:
                groups.setdefault(k, []).append((j, v))
            runs += [("y", i, k, c, jv) for k, jv in groups.items()]
    return runs


def _is_diagonal(terms) -> bool:
    return bool(terms) and all(len(t.items) == 1 for t in terms)


def _emit_block_fwd(spec: U1DSpec, b: Block, owned: set, slot_of: Dict[int, int], ind: str) -> List[str]:
    terms = [t for t in b.terms if t.v in owned]
    if not terms:
        return []
    if _is_diagonal(terms):
        L = [ind + "{"]
        for kind, i, sh, c, ov in _diagonal_runs(terms):
            shared, other = ("x", "y") if kind == "x" else ("y", "x")
            sexpr = f"vmul(W({i}), {shared}{sh})" if c == 1.0 else f"vmul(vmul({_vlit(c, spec.dtype)}, W({i})), {shared}{sh})"
            L.append(f"{ind}  {{ const V s = {sexpr};")
            for o, v in ov:
                L.append(f"{ind}    acc{slot_of[v]} = vfma(s, {other}{o}, acc{slot_of[v]});")
            L.append(f"{ind}  }}")
        L.append(ind + "}")
        return L
    used = sorted({(j, k) for t in terms for j, k, _ in t.items})
    L = [ind + "{"]
    for (j, k) in used:
        L.append(f"{ind}  const V p_{j}_{k} = vmul(x{j}, y{k});")
    for t in terms:
        L.append(f"{ind}  {{ " + " ".join(_sum_expr(t.items, spec.dtype)) + f" acc{slot_of[t.v]} = vfma(W({t.i}), t, acc{slot_of[t.v]}); }}")
    L.append(ind + "}")
    return L


def emit_forward(spec: U1DSpec, tun: Tuning) -> str:
    _check_tuning(spec, tun)
    blocks = build_blocks(spec)
    G = tun.groups
    owners = split_out_segments(blocks, spec.out_segs, G)
    max_slots = max(1, max(len(o) for o in owners))
    tpg = tun.ct // tun.vec
    ncons_warps = G * tpg // 32
    threads = tun.pipes * (G * tpg + 32)
    src = [_prelude(spec, tun, 0, ncons_warps)]
    acc_decl = " ".join(f"V acc{s_} = VS::zero();" for s_ in range(max_slots))
    wdef = ("#define W(i) VS::ld(w + (size_t)(i) * U + m.ct * CT + ch)" if spec.w_shared
            else "#define W(i) VS::ld(sw + (i) * CT)")
    src.append(f"""
constexpr int NTHREADS = {threads};
constexpr int PIPE_BYTES = BAR_BYTES + STAGES * STAGE_BYTES;
constexpr int SMEM_BYTES = cfg::PIPES * PIPE_BYTES;

__global__ void __launch_bounds__(NTHREADS, {tun.min_blocks})
fasteq_u1d_fwd_kernel(const Graph g, const T* __restrict__ w, const T* __restrict__ x, const T* __restrict__ y,
                      T* __restrict__ out) {{
  extern __shared__ __align__(128) unsigned char smem_all[];
  if (threadIdx.x == 0) {{
    for (int p = 0; p < cfg::PIPES; ++p) {{
      uint64_t* f = reinterpret_cast<uint64_t*>(smem_all + (size_t)p * PIPE_BYTES);
      init_barriers(f, f + STAGES, g.bulk_ok);
    }}
    mbar_fence_init();
  }}
  __syncthreads();
  // warps [0, PIPES * NCONS_WARPS) consume, the last PIPES warps produce; pipeline p owns consumer
  // warps [p * NCONS_WARPS, (p + 1) * NCONS_WARPS) and producer warp PIPES * NCONS_WARPS + p
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool is_producer = warp >= cfg::PIPES * cfg::NCONS_WARPS;
  const int pipe = is_producer ? warp - cfg::PIPES * cfg::NCONS_WARPS : warp / cfg::NCONS_WARPS;
  unsigned char* smem = smem_all + (size_t)pipe * PIPE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + STAGES;
  unsigned char* stages = smem + BAR_BYTES;
  if (is_producer) {{
    Producer p{{g, w, x, y, stages, full, empty, lane, 0u, (int)blockIdx.x * cfg::PIPES + pipe}};
    p.run([](unsigned char*) {{}}, [](int, int, int) {{}});
    return;
  }}
  const int ptid = threadIdx.x - pipe * cfg::NCONS_WARPS * 32;   // thread index inside the pipeline
  const int grp = ptid / TPG, ch = (ptid % TPG) * VEC;
  {acc_decl}
  uint32_t it = 0;
  for (;;) {{
    const int stage = it % STAGES;
    const uint32_t ph = (it / STAGES) & 1u;
    // a wait that gave up means the stage record below was never written: stop, do not address memory from it
    if (!mbar_wait(&full[stage], ph, g.status)) break;
    const unsigned char* st = stages + (size_t)stage * STAGE_BYTES;
    const Meta m = *reinterpret_cast<const Meta*>(st + OFF_META);
    const int valid = (U % CT == 0) ? CT : ((U - m.ct * CT) < CT ? (U - m.ct * CT) : CT);
    const bool live = ch < valid;
    if ((m.flags & F_DATA) && live) {{
      const T* sw = reinterpret_cast<const T*>(st + OFF_W) + ch; (void)sw;
      const T* sx = reinterpret_cast<const T*>(st + OFF_X) + ch;
      const T* sy = reinterpret_cast<const T*>(st + OFF_Y){' + ch' if spec.y_vec else ''};
{wdef}
""")
    body = _load_xy(spec, "      ")
    for gi in range(G):
        owned = set(owners[gi])
        slot_of = {v: s for s, v in enumerate(owners[gi])}
        body.append(f"      if (grp == {gi}) {{" if G > 1 else "      {")
        for b in blocks:
            body += _emit_block_fwd(spec, b, owned, slot_of, "        ")
        body.append("      }")
    body.append("#undef W")
    body.append("    }")
    body.append("    if (m.flags & F_LAST) {")
    body.append("      if (live) {")
    body.append("        T* o = out + (size_t)m.row * OSEG * U + (size_t)m.ct * CT + ch;")
    for gi in range(G):
        body.append(f"        if (grp == {gi}) {{" if G > 1 else "        {")
        for s, v in enumerate(owners[gi]):
            body.append(f"          VS::st(o + {v} * U, acc{s});")
        body.append("        }")
    body.append("      }")
    body.append("      " + " ".join(f"acc{s_} = VS::zero();" for s_ in range(max_slots)))
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
  if (VEC == 2 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(w)) & 7u)) return FASTEQ_INVALID;
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
    src.append(_NOALLOC_FORWARD.replace("@MINB@", str(tun.min_blocks)))
    return "\n".join(src)


# --------------------------------------------------------------------------- backward

def _emit_warp_reduce_scatter(exprs: List[str], ind: str) -> List[str]:
    """Sum each of n per-lane values over the 32 lanes with a halving butterfly: at every step a
    lane keeps half of its values and hands the other half to its partner, so n values cost about
    n + log2(32) shuffles instead of 5 n.  Ends with ``part[k] = total_k`` from one lane per k."""
    n = len(exprs)
    P = 1
    while P < n:
        P *= 2
    P = min(P, 32)
    if n > 32:
        raise ValueError("more than 32 scalar y segments are not supported by the warp reduction")
    L = [f"{ind}T r{i} = {exprs[i]};" if i < n else f"{ind}T r{i} = T(0);" for i in range(P)]
    half, off = P // 2, 16
    kterms = []
    while half >= 1:
        L.append(f"{ind}{{ const bool up = (lane & {off}) != 0;")
        for i in range(half):
            L.append(f"{ind}  {{ const T send = up ? r{i} : r{i + half}; const T keep = up ? r{i + half} : r{i}; "
                     f"r{i} = keep + __shfl_xor_sync(0xffffffffu, send, {off}); }}")
        L.append(f"{ind}}}")
        kterms.append(f"((lane & {off}) ? {half} : 0)")
        half //= 2
        off //= 2
    rest_mask = 0
    while off >= 1:
        L.append(f"{ind}r0 += __shfl_xor_sync(0xffffffffu, r0, {off});")
        rest_mask |= off
        off //= 2
    k = " + ".join(kterms) if kterms else "0"
    L.append(f"{ind}{{ const int k = {k}; if ((lane & {rest_mask}) == 0 && k < {n}) part[k] = r0; }}")
    return L


def emit_backward(spec: U1DSpec, tun: Tuning, need_gw: bool, need_gx: bool, need_gy: bool) -> str:
    """Backward module: grad_w, grad_x, grad_y of ``sum(out * grad_out)`` (any subset).

    Per edge and channel, with ``g = grad_out[v]``:  ``gw[i] += g * sum c p_jk``,
    ``q_jk += c * w[i] * g``, then ``gx[j] += q_jk * y[k]`` and ``gy[k] += q_jk * x[j]``
    (fasteq/ops/auto_schedule/models.py:145-152 states the three gradient terms).
    The receiver's grad_out row is staged once per receiver segment; gx goes out through
    ``red.global.add`` when x is gathered; a scalar-y gradient is summed over channels
    with warp shuffles, then across warps by the producer warp when the stage is recycled.
    """
    _check_tuning(spec, tun)
    G = tun.groups
    if G not in (1, 2):
        raise ValueError("the backward kernel takes one or two thread groups")
    if G == 2 and (spec.w_shared or spec.y_vec or spec.y_indexed or not spec.x_indexed):
        # two groups split the (weight segment, output segment) terms of one edge: each owns its grad_w rows, both add
        # into grad_x (red.global.add) and into the per-warp partial sums of the scalar grad_y
        raise ValueError("two backward thread groups need per-edge weights, a gathered x and a per-edge scalar y")
    blocks = build_blocks(spec)
    owners = split_w_segments(blocks, spec.w_segs, G)          # weight segments each thread group differentiates
    tpg = tun.ct // tun.vec
    ncons_warps = G * tpg // 32
    threads = tun.pipes * (G * tpg + 32)
    scalar_gy = need_gy and not spec.y_vec
    extra = ncons_warps * spec.y_segs * spec.elem_bytes if scalar_gy else 0
    extra = (extra + 15) // 16 * 16
    dt = spec.dtype
    src = [_prelude(spec, tun, extra, ncons_warps, emit_empty=False)]
    src.append(f"""
constexpr int NTHREADS = {threads};
constexpr int NGO = {1 if tun.go_smem else 0};                                 // grad_out row buffers in shared memory (0: read through L1)
constexpr bool GO_TMEM = {'true' if tun.go_tmem else 'false'};                 // ... or parked in tensor memory, one lane per consumer thread
constexpr uint32_t TMEM_COLS = {tmem_columns(spec, tun) if tun.go_tmem else 0};
constexpr uint32_t GO_COLS = VEC * (uint32_t)(sizeof(T) / 4);                  // 32-bit columns one segment of a thread's row takes
constexpr int GO_BYTES = round_up(OSEG * CT * (int)sizeof(T), 128);
constexpr int PIPE_BYTES = BAR_BYTES + STAGES * STAGE_BYTES + NGO * GO_BYTES;
constexpr int SMEM_BYTES = cfg::PIPES * PIPE_BYTES;
constexpr bool NEED_GW = {str(need_gw).lower()}, NEED_GX = {str(need_gx).lower()}, NEED_GY = {str(need_gy).lower()};
constexpr bool GY_ATOMIC = cfg::Y_INDEXED || (!cfg::Y_VEC && NCT > 1);

__global__ void __launch_bounds__(NTHREADS, {tun.min_blocks})
fasteq_u1d_bwd_kernel(const Graph g, const T* __restrict__ go, const T* __restrict__ w, const T* __restrict__ x,
                      const T* __restrict__ y, T* __restrict__ gw, T* __restrict__ gx, T* __restrict__ gy) {{
  extern __shared__ __align__(128) unsigned char smem_all[];
  if (threadIdx.x == 0) {{
    for (int p = 0; p < cfg::PIPES; ++p) {{
      uint64_t* f = reinterpret_cast<uint64_t*>(smem_all + (size_t)p * PIPE_BYTES);
      init_barriers(f, f + STAGES, g.bulk_ok);
      uint64_t* gf = f + 2 * STAGES;
      for (int b = 0; b < NGO; ++b) {{ mbar_init(&gf[b], 33); mbar_init(&gf[NGO + b], cfg::NCONS_WARPS); }}
    }}
    mbar_fence_init();
  }}
  __syncthreads();
  const int warp_all = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // tensor-memory gradient rows: warp 0 allocates, everyone reads the base address from the last word of the first
  // barrier block (free when no gradient tile lives in shared memory)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_all + BAR_BYTES - 4);
  if (GO_TMEM) {{
    if (warp_all == 0) scratch_tmem_alloc(tmem_slot, TMEM_COLS);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }}
  const uint32_t tmem_base = GO_TMEM ? *tmem_slot : 0u;
  const bool is_producer = warp_all >= cfg::PIPES * cfg::NCONS_WARPS;
  const int pipe = is_producer ? warp_all - cfg::PIPES * cfg::NCONS_WARPS : warp_all / cfg::NCONS_WARPS;
  const int warp = warp_all - pipe * cfg::NCONS_WARPS;           // consumer warp index inside the pipeline
  unsigned char* smem = smem_all + (size_t)pipe * PIPE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + STAGES;
  uint64_t* go_full = empty + STAGES;
  uint64_t* go_empty = go_full + NGO;
  unsigned char* stages = smem + BAR_BYTES;
  unsigned char* gobuf = stages + STAGES * STAGE_BYTES;
  if (is_producer) {{
    Producer p{{g, w, x, y, stages, full, empty, lane, 0u, (int)blockIdx.x * cfg::PIPES + pipe}};
    uint32_t nseg = 0;
    auto begin = [&](int row, int ct, int ln) {{
      if (NGO == 0) return;
      // stage the receiver's grad_out tile once per segment
      const int b = nseg % (NGO ? NGO : 1);
      const uint32_t ph = (nseg / (NGO ? NGO : 1)) & 1u;
      if (!mbar_wait(&go_empty[b], ph ^ 1u, g.status)) {{ p.failed = true; return; }}
      const int valid = (U - ct * CT) < CT ? (U - ct * CT) : CT;
      if (ln == 0) mbar_arrive_expect_tx(&go_full[b], g.bulk_ok ? (uint32_t)(OSEG * valid * sizeof(T)) : 0u);
      __syncwarp();
      copy_tile(gobuf + (size_t)b * GO_BYTES, go + (size_t)row * OSEG * U, OSEG, ct, valid, g.bulk_ok != 0, &go_full[b], ln);
      cp_async_arrive_noinc(&go_full[b]);
      ++nseg;
    }};
    auto flush = [&](unsigned char* st) {{
      // one lane finishes the y gradient of the edge that occupied this stage: sum the consumer
      // warps' partial sums and write the row
      if ({'true' if scalar_gy else 'false'}) {{
        const Meta pm = *reinterpret_cast<const Meta*>(st + OFF_META);
        if (pm.flags & F_DATA) {{
          const T* part = reinterpret_cast<const T*>(st + OFF_EXTRA);
          if (cfg::Y_SH) {{
            // the y operand is the edge vector: chain the harmonics' Jacobian and write d/d(vector)
            T gk[YSEG];
#pragma unroll
            for (int k = 0; k < YSEG; ++k) {{
              T s = T(0);
#pragma unroll
              for (int wp = 0; wp < cfg::NCONS_WARPS; ++wp) s += part[wp * YSEG + k];
              gk[k] = s;
            }}
            const T* vsrc = y + (size_t)pm.yr * 3;
            T gv[3];
            fasteq_sh::vjp(vsrc[0], vsrc[1], vsrc[2], gk, gv);
            T* dst = gy + (size_t)pm.yr * 3;
#pragma unroll
            for (int k = 0; k < 3; ++k) {{ if (GY_ATOMIC) red_add(dst + k, gv[k]); else dst[k] = gv[k]; }}
          }} else {{
          T* dst = gy + (size_t)pm.yr * YSEG;
#pragma unroll
          for (int k = 0; k < YSEG; ++k) {{
            T s = T(0);
#pragma unroll
            for (int wp = 0; wp < cfg::NCONS_WARPS; ++wp) s += part[wp * YSEG + k];
            if (GY_ATOMIC) red_add(dst + k, s); else dst[k] = s;
          }}
          }}
        }}
      }}
    }};
    p.run(flush, begin);
    return;
  }}
  const int ptid = threadIdx.x - pipe * cfg::NCONS_WARPS * 32;   // thread index inside the pipeline
  const int grp = ptid / TPG, ch = (ptid % TPG) * VEC; (void)grp;
  uint32_t it = 0, nseg = 0;
  // this thread's gradient row in tensor memory: lane = 32 * (warp % 4) + lane id, the consumer warps of one lane quarter
  // stacked GO_COLS * OSEG columns apart
  const uint32_t tmem_go = tmem_base + ((uint32_t)(32 * (warp_all & 3)) << 16) + (uint32_t)(warp_all >> 2) * GO_COLS * OSEG;
  (void)tmem_go;
""")
    L: List[str] = []
    if spec.w_shared and need_gw:
        L.append(f"  V gws[{spec.w_segs}];")
        L.append("#pragma unroll")
        L.append(f"  for (int i = 0; i < {spec.w_segs}; ++i) gws[i] = VS::zero();")
        L.append("  int gws_ct = 0;")
    L.append("""  for (;;) {
    const int stage = it % STAGES;
    const uint32_t ph = (it / STAGES) & 1u;
    // a wait that gave up means the stage record (or the grad_out tile) was never written: stop here
    if (!mbar_wait(&full[stage], ph, g.status)) break;
    unsigned char* st = stages + (size_t)stage * STAGE_BYTES;
    const Meta m = *reinterpret_cast<const Meta*>(st + OFF_META);
    const int valid = (U % CT == 0) ? CT : ((U - m.ct * CT) < CT ? (U - m.ct * CT) : CT);
    const bool live = ch < valid;
    const int gb = nseg % (NGO ? NGO : 1);
    if (NGO && (m.flags & F_FIRST) && !mbar_wait(&go_full[gb], (nseg / (NGO ? NGO : 1)) & 1u, g.status)) break;
    if (GO_TMEM && (m.flags & F_FIRST)) {
      // a new receiver (or channel tile): its grad_out row moves from global memory into this thread's tensor-memory lane
      const T* grow = go + (size_t)m.row * OSEG * U + (size_t)m.ct * CT + ch;
#pragma unroll
      for (int v = 0; v < OSEG; ++v) scratch_tmem_st(tmem_go + GO_COLS * (uint32_t)v, VS::ldg(grow + (size_t)v * U));
      scratch_tmem_wait_st();
    }""")
    if spec.w_shared and need_gw:
        L.append("    if ((m.flags & (F_DATA | F_DONE)) && (m.ct != gws_ct || (m.flags & F_DONE))) {")
        L.append("      if (ch < ((U - gws_ct * CT) < CT ? (U - gws_ct * CT) : CT)) {")
        for i in range(spec.w_segs):
            L.append(f"        VS::red(gw + (size_t){i} * U + gws_ct * CT + ch, gws[{i}]); gws[{i}] = VS::zero();")
        L.append("      }")
        L.append("      gws_ct = m.ct;")
        L.append("    }")
    if scalar_gy:
        for k in range(spec.y_segs):
            L.append(f"    V gy{k} = VS::zero();")
    L.append("    if ((m.flags & F_DATA) && live) {")
    L.append("      const T* sx = reinterpret_cast<const T*>(st + OFF_X) + ch;")
    L.append(f"      const T* sy = reinterpret_cast<const T*>(st + OFF_Y){' + ch' if spec.y_vec else ''};")
    if tun.go_smem:
        L.append("      const T* sgo = reinterpret_cast<const T*>(gobuf + (size_t)gb * GO_BYTES) + ch;")
    else:
        L.append("      const T* sgo = go + (size_t)m.row * OSEG * U + (size_t)m.ct * CT + ch;")
    if spec.w_shared:
        L.append("#define W(i) VS::ld(w + (size_t)(i) * U + m.ct * CT + ch)")
    else:
        L.append("      const T* sw = reinterpret_cast<const T*>(st + OFF_W) + ch;")
        L.append("#define W(i) VS::ld(sw + (i) * CT)")
    if tun.go_tmem:
        L.append("#define GO(v) go_##v")       # loaded from tensor memory at the head of each block
    else:
        L.append("#define GO(v) VS::ld(sgo + (v) * CT)" if tun.go_smem else "#define GO(v) VS::ldg(sgo + (size_t)(v) * U)")
    L += _load_xy(spec, "      ")
    if need_gx:
        L += [f"      V gx{j} = VS::zero();" for j in range(spec.x_segs)]
    if need_gy and spec.y_vec:
        L += [f"      V gy{k} = VS::zero();" for k in range(spec.y_segs)]
    used_i = sorted({t.i for b in blocks for t in b.terms})
    if need_gw:
        L += [f"      V gw{i} = VS::zero();" for i in used_i]
        if not spec.w_shared:
            L.append("      T* gwp = gw + (size_t)m.e * WSEG * U + (size_t)m.ct * CT + ch;")
    need_q = need_gx or need_gy

    def gw_part(b: Block, ind: str) -> List[str]:
        out = [f"{ind}const V p_{j}_{k} = vmul(x{j}, y{k});" for (j, k) in b.products]
        for t in b.terms:
            out.append(f"{ind}{{ " + " ".join(_sum_expr(t.items, dt)) + f" gw{t.i} = vfma(GO({t.v}), t, gw{t.i}); }}")
        return out

    def q_part(b: Block, ind: str) -> List[str]:
        out = []
        first_use = set()
        for t in b.terms:
            out.append(f"{ind}{{ const V gp = vmul(W({t.i}), GO({t.v}));")
            for j, k, c in t.items:
                if (j, k) in first_use:
                    out.append(f"{ind}  q_{j}_{k} = vfma({_vlit(c, dt)}, gp, q_{j}_{k});")
                else:
                    first_use.add((j, k))
                    out.append(f"{ind}  q_{j}_{k} = vmul({_vlit(c, dt)}, gp);")
            out.append(f"{ind}}}")
        decl = [f"{ind}V q_{j}_{k};" for (j, k) in b.products]
        tail = []
        if need_gx:
            tail += [f"{ind}gx{j} = vfma(q_{j}_{k}, y{k}, gx{j});" for (j, k) in b.products]
        if need_gy:
            tail += [f"{ind}gy{k} = vfma(q_{j}_{k}, x{j}, gy{k});" for (j, k) in b.products]
        return decl + out + tail

    def diag_part(b: Block, ind: str) -> List[str]:
        # out[v] += c * w[i] * S * O[v] with S the run's shared operand (x[j] or y[k]) and O[v] the other one:
        #   d = sum_v go[v] * O[v];  gw[i] += c * S * d;  gS += c * w[i] * d;  gO[v] += (c * w[i] * S) * go[v]
        out = []
        for kind, i, sh, c, ov in _diagonal_runs(b.terms):
            S, O = (f"x{sh}", "y") if kind == "x" else (f"y{sh}", "x")
            need_gs, need_go = (need_gx, need_gy) if kind == "x" else (need_gy, need_gx)
            gS = ("gx" if kind == "x" else "gy") + str(sh)
            gO = "gy" if kind == "x" else "gx"
            out.append(f"{ind}{{")
            if need_gw or need_gs:
                o0, v0 = ov[0]
                out.append(f"{ind}  V d = vmul(GO({v0}), {O}{o0});")
                for o, v in ov[1:]:
                    out.append(f"{ind}  d = vfma(GO({v}), {O}{o}, d);")
            cw = f"W({i})" if c == 1.0 else f"vmul({_vlit(c, dt)}, W({i}))"
            out.append(f"{ind}  const V cw = {cw};")
            if need_gw:
                cs = S if c == 1.0 else f"vmul({_vlit(c, dt)}, {S})"
                out.append(f"{ind}  gw{i} = vfma({cs}, d, gw{i});")
            if need_gs:
                out.append(f"{ind}  {gS} = vfma(cw, d, {gS});")
            if need_go:
                out.append(f"{ind}  const V s = vmul(cw, {S});")
                for o, v in ov:
                    out.append(f"{ind}  {gO}{o} = vfma(s, GO({v}), {gO}{o});")
            out.append(f"{ind}}}")
        return out

    for gi in range(G):
        gblocks = blocks if G == 1 else restrict_blocks(blocks, owners[gi])
        last_block_of_i: Dict[int, int] = {}
        for bi, b in enumerate(gblocks):
            for t in b.terms:
                last_block_of_i[t.i] = bi
        if G > 1:
            L.append(f"      if (grp == {gi}) {{")
        for bi, b in enumerate(gblocks):
            if tun.go_tmem:
                # the block's grad_out values: issued together, released by one wait that names them
                vs = sorted({t.v for t in b.terms})
                L.append("      {")
                L.append("      V " + ", ".join(f"go_{v}" for v in vs) + ";")
                L += [f"      scratch_tmem_ld(tmem_go + {v}u * GO_COLS, go_{v});" for v in vs]
                L.append(f"      scratch_tmem_wait_ld(go_{vs[0]});")
                L += [f"      scratch_tmem_pin(go_{v});" for v in vs[1:]]
            if _is_diagonal(b.terms):
                L.append("      {"); L += diag_part(b, "        "); L.append("      }")
            elif tun.two_pass or not (need_gw and need_q):
                if need_gw:
                    L.append("      {"); L += gw_part(b, "        "); L.append("      }")
                if need_q:
                    L.append("      {"); L += q_part(b, "        "); L.append("      }")
            else:
                # single pass: products and their gradients live together, grad_out / weight read once
                L.append("      {")
                L += [f"        const V p_{j}_{k} = vmul(x{j}, y{k});" for (j, k) in b.products]
                L += [f"        V q_{j}_{k};" for (j, k) in b.products]
                first_use = set()
                for t in b.terms:
                    L.append(f"        {{ const V gv = GO({t.v});")
                    L.append("          " + " ".join(_sum_expr(t.items, dt)) + f" gw{t.i} = vfma(gv, t, gw{t.i});")
                    L.append(f"          const V gp = vmul(W({t.i}), gv);")
                    for j, k, c in t.items:
                        if (j, k) in first_use:
                            L.append(f"          q_{j}_{k} = vfma({_vlit(c, dt)}, gp, q_{j}_{k});")
                        else:
                            first_use.add((j, k))
                            L.append(f"          q_{j}_{k} = vmul({_vlit(c, dt)}, gp);")
                    L.append("        }")
                if need_gx:
                    L += [f"        gx{j} = vfma(q_{j}_{k}, y{k}, gx{j});" for (j, k) in b.products]
                if need_gy:
                    L += [f"        gy{k} = vfma(q_{j}_{k}, x{j}, gy{k});" for (j, k) in b.products]
                L.append("      }")
            if tun.go_tmem:
                L.append("      }")
            if need_gw:
                for i in sorted(i for i, last in last_block_of_i.items() if last == bi):
                    if spec.w_shared:
                        L.append(f"      gws[{i}] = vadd(gws[{i}], gw{i});")
                    else:
                        L.append(f"      VS::st(gwp + {i} * U, gw{i});")
        if need_gw and not spec.w_shared:
            # weight segments no path touches get a zero gradient (written by the group that owns them)
            for i in (range(spec.w_segs) if G == 1 else owners[gi]):
                if i not in last_block_of_i:
                    L.append(f"      VS::st(gwp + {i} * U, VS::zero());")
        if G > 1:
            L.append("      }")
    if need_gx:
        L.append("      T* gxp = gx + (size_t)m.xr * XSEG * U + (size_t)m.ct * CT + ch;")
        for j in range(spec.x_segs):
            L.append(f"      VS::{'red' if spec.x_indexed else 'st'}(gxp + {j} * U, gx{j});")
    if need_gy and spec.y_vec:
        L.append("      T* gyp = gy + (size_t)m.yr * YSEG * U + (size_t)m.ct * CT + ch;")
        for k in range(spec.y_segs):
            L.append(f"      VS::{'red' if spec.y_indexed else 'st'}(gyp + {k} * U, gy{k});")
    L.append("#undef W")
    L.append("#undef GO")
    L.append("    }")
    if scalar_gy:
        L.append("    if (m.flags & F_DATA) {")
        L.append("      T* part = reinterpret_cast<T*>(st + OFF_EXTRA) + warp * YSEG;")
        L += _emit_warp_reduce_scatter([f"VS::hsum(gy{k})" for k in range(spec.y_segs)], "      ")
        L.append("    }")
    L.append("""    __syncwarp();
    if (lane == 0) {
      if (NGO && (m.flags & F_LAST)) mbar_arrive(&go_empty[gb]);
      mbar_arrive(&empty[stage]);
    }
    if (m.flags & F_LAST) ++nseg;
    ++it;
    if (m.flags & F_DONE) break;
  }
  if (GO_TMEM) {
    // every consumer warp is done with its lanes (also after a wait that gave up): warp 0 returns the columns
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    asm volatile("bar.sync 1, %0;" ::"r"(cfg::PIPES * cfg::NCONS_WARPS * 32) : "memory");
    if (warp_all == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      scratch_tmem_free(tmem_base, TMEM_COLS);
    }
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
        ycols = "YSEG * U" if spec.y_vec else ("3" if spec.y_sh else "YSEG")
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
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  {' '.join(zero)}
  if (gh->n_edges == 0) return FASTEQ_OK;          // per-edge buffers are empty (and may be null); the rest is zeroed
  if ((NEED_GW && !gw) || (NEED_GX && !gx) || (NEED_GY && !gy)) return FASTEQ_INVALID;
  if (!go || !w || !x || !y) return FASTEQ_INVALID;
  g.bulk_ok = aligned16(w) && aligned16(x) && aligned16(y) && aligned16(go) && ((U * sizeof(T)) % 16 == 0) &&
              ((CT * sizeof(T)) % 16 == 0);
  if (VEC == 2 && ((reinterpret_cast<uintptr_t>(gw) | reinterpret_cast<uintptr_t>(gx) | reinterpret_cast<uintptr_t>(gy)) & 7u))
    return FASTEQ_INVALID;
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


def arith_ops(spec: U1DSpec, tun: Tuning, direction: str, needs=(True, True, True)) -> Dict[str, int]:
    """Floating-point instructions the consumers execute per (edge, channel), counted in the generated source: every
    ``vfma`` / ``vmul`` / ``vadd`` of the straight-line edge body (with two thread groups the groups' shares add up;
    a packed instruction counts once per channel it serves).  ``fma + mul + add`` against ``SMs x 128 x clock`` is the
    kernel's FP32-pipe floor, which for the larger signatures lies above the HBM floor."""
    import re
    src = emit_forward(spec, tun) if direction == "fwd" else emit_backward(spec, tun, *needs)
    body = src[src.index("if ((m.flags & F_DATA) && live)"):]
    body = body[:body.index("#undef W")]
    return {"fma": len(re.findall(r"\bvfma\(", body)), "mul": len(re.findall(r"\bvmul\(", body)), "add": len(re.findall(r"\bvadd\(", body))}
