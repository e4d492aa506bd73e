"""CUDA source emitter for the symmetric tensor contraction (STC Uniform1D) kernels, sm_100a.

    out[b, v, u] = sum_p c_p * prod_t x1[b, a_{p,t}, u] * x0[i0[b], d_p, u]

One thread per (node, channel).  Paths are grouped by (weight segment d, output segment v);
inside a group the polynomial in x1 is evaluated in nested (Horner) form over sorted index
tuples, so a degree-3 path costs one FMA and each shared prefix one more, with the coefficients
as literals.  The species gather ``x0[i0[b]]`` happens in the kernel (the reference materialises
it with a torch gather first, fasteq/ops/stc_uniform1d_jit.py:1016).  Counterpart of the
reference's emitters fasteq/ops/auto_schedule/stc_forward.py:158-340 and stc_backward.py:103-524.
The backward re-evaluates each nest and runs it in reverse; it produces grad_x1 and, on request,
the per-node weight gradient that the caller reduces over nodes of equal species.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np

from .u1d_common import lit


@dataclass(frozen=True)
class STCSpec:
    paths: Tuple[Tuple[Tuple[int, ...], int, int, float], ...]   # (x1 indices, d, v, c)
    x1_segs: int
    x0_segs: int
    out_segs: int
    u: int
    dtype: str = "f32"

    @property
    def ctype(self) -> str:
        return "float" if self.dtype == "f32" else "double"

    def key(self, extra: str = "") -> str:
        h = hashlib.sha256()
        h.update(repr((self.paths, self.x1_segs, self.x0_segs, self.out_segs, self.u, self.dtype, extra)).encode())
        return h.hexdigest()[:16]


def make_stc_spec(paths, coeffs, *, x1_segs, x0_segs, out_segs, u, dtype, pad_value=-1) -> STCSpec:
    cs = np.asarray(coeffs, dtype=np.float64)
    if dtype == "f32":
        cs = cs.astype(np.float32).astype(np.float64)
    rows = []
    for row, c in zip(np.asarray(paths), cs):
        vals = [int(t) for t in row if int(t) != pad_value]
        if not 3 <= len(vals) <= 5:
            raise ValueError(f"bad STC path length {len(vals)}; expected 3..5")
        a, d, v = tuple(sorted(vals[:-2])), vals[-2], vals[-1]
        if not (all(0 <= t < x1_segs for t in a) and 0 <= d < x0_segs and 0 <= v < out_segs):
            raise ValueError("STC path index outside its operand's segment count")
        rows.append((a, d, v, float(c)))
    return STCSpec(tuple(rows), int(x1_segs), int(x0_segs), int(out_segs), int(u), dtype)


def _groups(spec: STCSpec):
    """{(d, v): {sorted index tuple: coefficient}} with duplicates merged."""
    g: Dict[Tuple[int, int], Dict[Tuple[int, ...], float]] = {}
    for a, d, v, c in spec.paths:
        m = g.setdefault((d, v), {})
        m[a] = m.get(a, 0.0) + c
    return {k: {a: c for a, c in m.items() if c != 0.0} for k, m in sorted(g.items())}


def _trie(mono: Dict[Tuple[int, ...], float]):
    """Nested dict: index -> (constant coefficient or None, children)."""
    root: Dict[int, list] = {}
    for a, c in sorted(mono.items()):
        node = root
        for depth, idx in enumerate(a):
            ent = node.setdefault(idx, [None, {}])
            if depth == len(a) - 1:
                ent[0] = c
            node = ent[1]
    return root


def _emit_value(node: Dict[int, list], dt: str, ind: str, name: str, uid: List[int]) -> List[str]:
    """Statements that set ``T name = sum_idx x[idx] * (const + value(children))``."""
    L = []
    first = True
    for idx, (const, children) in node.items():
        if children:
            uid[0] += 1
            sub = f"r{uid[0]}"
            L += _emit_value(children, dt, ind, sub, uid)
            inner = sub if const is None else f"({sub} + {lit(const, dt)})"
            if const is not None:
                L.append(f"{ind}{sub} += {lit(const, dt)};")
                inner = sub
            term = (f"x{idx}", inner)
        else:
            term = (lit(const, dt), f"x{idx}")
        if first:
            L.append(f"{ind}T {name} = {term[0]} * {term[1]};")
            first = False
        else:
            L.append(f"{ind}{name} = fma({term[0]}, {term[1]}, {name});")
    return L


def _emit_reverse(node: Dict[int, list], dt: str, ind: str, gname: str, uid: List[int]) -> List[str]:
    """Given ``gname`` = d(out)/d(value of this node), accumulate into ga*; recomputes child values."""
    L = []
    for idx, (const, children) in node.items():
        if children:
            uid[0] += 1
            sub = f"r{uid[0]}"
            L += _emit_value(children, dt, ind, sub, uid)
            if const is not None:
                L.append(f"{ind}{sub} += {lit(const, dt)};")
            L.append(f"{ind}ga{idx} = fma({gname}, {sub}, ga{idx});")
            uid[0] += 1
            gsub = f"g{uid[0]}"
            L.append(f"{ind}const T {gsub} = {gname} * x{idx};")
            L += _emit_reverse(children, dt, ind, gsub, uid)
        else:
            L.append(f"{ind}ga{idx} = fma({gname}, {lit(const, dt)}, ga{idx});")
    return L


_COMMON = r"""
__device__ int g_status_word;
static thread_local char g_err[256];
static int cuda_fail(cudaError_t e) { snprintf(g_err, sizeof(g_err), "%s", cudaGetErrorString(e)); return FASTEQ_CUDA_ERROR; }
extern "C" const char* fasteq_last_cuda_error(void) { return g_err; }
extern "C" int fasteq_stc_device_status(int32_t* code) {
  if (!code) return FASTEQ_INVALID;
  int v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  *code = v;
  return FASTEQ_OK;
}
"""


def _emit_double_backward(spec: STCSpec, groups, dt: str) -> List[str]:
    """Second-order kernel: with ``t = ggx1`` and ``tw = ggx0`` (per node) the cotangents of the first
    backward's outputs, and ``m = prod x[a_i] * w`` one monomial,

        D     = d/d eps  m(x + eps t, w + eps tw)            d_go[v] += c D
        d_w  += c go[v] * dP                                 (dP = sum_i t[a_i] prod_{j != i} x[a_j])
        d_x[a_k] += c go[v] * (w * d(dP)/dx[a_k] + tw * dP/dx[a_k])

    Factors are handled by position, so repeated indices need no special case.  Straight-line code per
    monomial (no nesting): this kernel serves force-loss training, not the benchmarked inference path.
    Counterpart of fasteq/ops/stc_uniform1d_jit.py:964-968 (double-backward ``run(go, x1, x0, i0, ggx0, ggx1, V)``)."""
    L: List[str] = [f"""
__global__ void __launch_bounds__(NT) fasteq_stc_dbwd_kernel(const T* __restrict__ go, const T* __restrict__ x1,
    const T* __restrict__ x0, const int* __restrict__ i0, const T* __restrict__ ggx1, const T* __restrict__ ggx0n,
    long long batch, long long n_species, T* __restrict__ d_go, T* __restrict__ d_x1, T* __restrict__ d_x0n, int* status) {{
  for (long long b = blockIdx.x; b < batch; b += gridDim.x) {{
    int sp = i0[b];
    if (sp < 0 || sp >= n_species) {{ atomicExch(status, 2); sp = 0; }}
    for (int u = threadIdx.x; u < U; u += NT) {{
      const T* xp = x1 + (size_t)b * A * U + u;
      const T* tp = ggx1 + (size_t)b * A * U + u;
      const T* wp = x0 + (size_t)sp * D * U + u;
      const T* twp = ggx0n + (size_t)b * D * U + u;
      const T* gp = go + (size_t)b * V * U + u;"""]
    L += [f"      const T x{a} = xp[{a} * U], t{a} = tp[{a} * U];" for a in range(spec.x1_segs)]
    L += [f"      const T go{v} = gp[{v} * U];" for v in range(spec.out_segs)]
    L += [f"      T dx{a} = T(0);" for a in range(spec.x1_segs)]
    L += [f"      T dg{v} = T(0);" for v in range(spec.out_segs)]
    by_d: Dict[int, List[int]] = {}
    for (d, v) in groups:
        by_d.setdefault(d, []).append(v)
    for d, vs in by_d.items():
        L.append(f"      {{ const T w = wp[{d} * U], tw = twp[{d} * U]; T dw = T(0);")
        for v in vs:
            for a, c in sorted(groups[(d, v)].items()):
                cl = lit(c, dt)
                n = len(a)
                L.append(f"        {{ const T cg = {cl} * go{v};")
                if n == 1:
                    (p,) = a
                    L.append(f"          dg{v} = fma({cl}, fma(t{p}, w, x{p} * tw), dg{v}); dw = fma(cg, t{p}, dw); dx{p} = fma(cg, tw, dx{p}); }}")
                elif n == 2:
                    p, q = a
                    L.append(f"          const T P = x{p} * x{q}, dP = fma(t{p}, x{q}, x{p} * t{q});")
                    L.append(f"          dg{v} = fma({cl}, fma(dP, w, P * tw), dg{v}); dw = fma(cg, dP, dw);")
                    L.append(f"          dx{p} = fma(cg, fma(w, t{q}, tw * x{q}), dx{p}); dx{q} = fma(cg, fma(w, t{p}, tw * x{p}), dx{q}); }}")
                else:
                    p, q, r = a
                    L.append(f"          const T pq = x{p} * x{q}, pr = x{p} * x{r}, qr = x{q} * x{r};")
                    L.append(f"          const T P = pq * x{r}, dP = fma(t{p}, qr, fma(t{q}, pr, t{r} * pq));")
                    L.append(f"          dg{v} = fma({cl}, fma(dP, w, P * tw), dg{v}); dw = fma(cg, dP, dw);")
                    L.append(f"          dx{p} = fma(cg, fma(w, fma(t{q}, x{r}, x{q} * t{r}), tw * qr), dx{p});")
                    L.append(f"          dx{q} = fma(cg, fma(w, fma(t{p}, x{r}, x{p} * t{r}), tw * pr), dx{q});")
                    L.append(f"          dx{r} = fma(cg, fma(w, fma(t{p}, x{q}, x{p} * t{q}), tw * pq), dx{r}); }}")
        L.append(f"        d_x0n[((size_t)b * D + {d}) * U + u] = dw; }}")
    for d in range(spec.x0_segs):
        if d not in by_d:
            L.append(f"      d_x0n[((size_t)b * D + {d}) * U + u] = T(0);")
    L.append("      T* dxp = d_x1 + (size_t)b * A * U + u;")
    L += [f"      dxp[{a} * U] = dx{a};" for a in range(spec.x1_segs)]
    L.append("      T* dgp = d_go + (size_t)b * V * U + u;")
    L += [f"      dgp[{v} * U] = dg{v};" for v in range(spec.out_segs)]
    L.append("    }\n  }\n}")
    L.append("""
extern "C" int fasteq_stc_forward(const void*, const void*, const int32_t*, int64_t, int64_t, void*, fasteq_stream_t) {
  return FASTEQ_UNSUPPORTED;  // double-backward module
}
extern "C" int fasteq_stc_backward(const void*, const void*, const void*, const int32_t*, int64_t, int64_t, void*, void*, fasteq_stream_t) {
  return FASTEQ_UNSUPPORTED;  // double-backward module
}
extern "C" int fasteq_stc_double_backward(const void* go, const void* x1, const void* x0, const int32_t* i0, const void* ggx1,
                                          const void* ggx0_per_node, int64_t batch, int64_t n_species, void* d_go, void* d_x1,
                                          void* d_x0_per_node, fasteq_stream_t stream) {
  if (batch < 0 || n_species < 0) return FASTEQ_INVALID;
  if (batch == 0) return FASTEQ_OK;
  if (!go || !x1 || !x0 || !i0 || !ggx1 || !ggx0_per_node || !d_go || !d_x1 || !d_x0_per_node) return FASTEQ_INVALID;
  int* st = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&st, g_status_word);
  if (e != cudaSuccess) return cuda_fail(e);
  const long long grid = batch < (1LL << 30) ? batch : (1LL << 30);
  fasteq_stc_dbwd_kernel<<<(unsigned)grid, NT, 0, (cudaStream_t)stream>>>((const T*)go, (const T*)x1, (const T*)x0, i0, (const T*)ggx1,
      (const T*)ggx0_per_node, batch, n_species, (T*)d_go, (T*)d_x1, (T*)d_x0_per_node, st);
  e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}""")
    return L


def emit_stc(spec: STCSpec, direction: str, need_gx0: bool = False) -> str:
    dt = spec.dtype
    groups = _groups(spec)
    threads = min((spec.u + 31) // 32 * 32, 128)
    head = f"""// Generated by fasteq_b200.codegen.stc -- do not edit.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "fasteq_b200.h"
typedef {spec.ctype} T;
constexpr int U = {spec.u}, A = {spec.x1_segs}, D = {spec.x0_segs}, V = {spec.out_segs}, NT = {threads};
{_COMMON}
extern "C" int fasteq_stc_describe(fasteq_stc_desc* d) {{
  if (!d) return FASTEQ_INVALID;
  d->abi_version = FASTEQ_ABI_VERSION; d->dtype = {0 if dt == 'f32' else 1}; d->u = U; d->x1_segs = A; d->x0_segs = D;
  d->out_segs = V; d->num_paths = {len(spec.paths)}; d->direction = {dict(fwd=0, bwd=1, dbwd=2)[direction]}; d->need_gx0 = {int(need_gx0)};
  return FASTEQ_OK;
}}
"""
    uid = [0]
    body: List[str] = []
    if direction == "fwd":
        body.append(f"""
__global__ void __launch_bounds__(NT) fasteq_stc_fwd_kernel(const T* __restrict__ x1, const T* __restrict__ x0,
    const int* __restrict__ i0, long long batch, long long n_species, T* __restrict__ out, int* status) {{
  for (long long b = blockIdx.x; b < batch; b += gridDim.x) {{
    int sp = i0[b];
    if (sp < 0 || sp >= n_species) {{ atomicExch(status, 2); sp = 0; }}
    for (int u = threadIdx.x; u < U; u += NT) {{
      const T* xp = x1 + (size_t)b * A * U + u;
      const T* wp = x0 + (size_t)sp * D * U + u;""")
        body += [f"      const T x{a} = xp[{a} * U];" for a in range(spec.x1_segs)]
        body += [f"      T o{v} = T(0);" for v in range(spec.out_segs)]
        for (d, v), mono in groups.items():
            body.append("      {")
            body += _emit_value(_trie(mono), dt, "        ", "r", uid)
            body.append(f"        o{v} = fma(wp[{d} * U], r, o{v});")
            body.append("      }")
        body.append("      T* op = out + (size_t)b * V * U + u;")
        body += [f"      op[{v} * U] = o{v};" for v in range(spec.out_segs)]
        body.append("    }\n  }\n}")
        body.append("""
extern "C" int fasteq_stc_forward(const void* x1, const void* x0, const int32_t* i0, int64_t batch, int64_t n_species,
                                  void* out, fasteq_stream_t stream) {
  if (batch < 0 || n_species < 0) return FASTEQ_INVALID;
  if (batch == 0) return FASTEQ_OK;
  if (!x1 || !x0 || !i0 || !out) return FASTEQ_INVALID;
  int* st = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&st, g_status_word);
  if (e != cudaSuccess) return cuda_fail(e);
  const long long grid = batch < (1LL << 30) ? batch : (1LL << 30);
  fasteq_stc_fwd_kernel<<<(unsigned)grid, NT, 0, (cudaStream_t)stream>>>((const T*)x1, (const T*)x0, i0, batch, n_species, (T*)out, st);
  e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}
extern "C" int fasteq_stc_backward(const void*, const void*, const void*, const int32_t*, int64_t, int64_t, void*, void*, fasteq_stream_t) {
  return FASTEQ_UNSUPPORTED;  // forward module
}
extern "C" int fasteq_stc_double_backward(const void*, const void*, const void*, const int32_t*, const void*, const void*, int64_t,
                                          int64_t, void*, void*, void*, fasteq_stream_t) {
  return FASTEQ_UNSUPPORTED;  // this module holds another direction
}
""")
    elif direction == "dbwd":
        body += _emit_double_backward(spec, groups, dt)
    else:
        body.append(f"""
constexpr bool NEED_GX0 = {str(need_gx0).lower()};
__global__ void __launch_bounds__(NT) fasteq_stc_bwd_kernel(const T* __restrict__ go, const T* __restrict__ x1,
    const T* __restrict__ x0, const int* __restrict__ i0, long long batch, long long n_species, T* __restrict__ gx1,
    T* __restrict__ gx0n, int* status) {{
  for (long long b = blockIdx.x; b < batch; b += gridDim.x) {{
    int sp = i0[b];
    if (sp < 0 || sp >= n_species) {{ atomicExch(status, 2); sp = 0; }}
    for (int u = threadIdx.x; u < U; u += NT) {{
      const T* xp = x1 + (size_t)b * A * U + u;
      const T* wp = x0 + (size_t)sp * D * U + u;
      const T* gp = go + (size_t)b * V * U + u;""")
        body += [f"      const T x{a} = xp[{a} * U];" for a in range(spec.x1_segs)]
        body += [f"      const T go{v} = gp[{v} * U];" for v in range(spec.out_segs)]
        body += [f"      T ga{a} = T(0);" for a in range(spec.x1_segs)]
        by_d: Dict[int, List[int]] = {}
        for (d, v) in groups:
            by_d.setdefault(d, []).append(v)
        for d, vs in by_d.items():
            body.append(f"      {{ const T w = wp[{d} * U];")
            if need_gx0:
                body.append("        T gw = T(0);")
            for v in vs:
                tr = _trie(groups[(d, v)])
                body.append("        {")
                if need_gx0:
                    body += _emit_value(tr, dt, "          ", "r", uid)
                    body.append(f"          gw = fma(go{v}, r, gw);")
                body.append(f"          const T g = w * go{v};")
                body += _emit_reverse(tr, dt, "          ", "g", uid)
                body.append("        }")
            if need_gx0:
                body.append(f"        gx0n[((size_t)b * D + {d}) * U + u] = gw;")
            body.append("      }")
        if need_gx0:
            used = set(by_d)
            for d in range(spec.x0_segs):
                if d not in used:
                    body.append(f"      gx0n[((size_t)b * D + {d}) * U + u] = T(0);")
        body.append("      T* gxp = gx1 + (size_t)b * A * U + u;")
        body += [f"      gxp[{a} * U] = ga{a};" for a in range(spec.x1_segs)]
        body.append("    }\n  }\n}")
        body.append("""
extern "C" int fasteq_stc_forward(const void*, const void*, const int32_t*, int64_t, int64_t, void*, fasteq_stream_t) {
  return FASTEQ_UNSUPPORTED;  // backward module
}
extern "C" int fasteq_stc_backward(const void* go, const void* x1, const void* x0, const int32_t* i0, int64_t batch,
                                   int64_t n_species, void* gx1, void* gx0_per_node, fasteq_stream_t stream) {
  if (batch < 0 || n_species < 0) return FASTEQ_INVALID;
  if (batch == 0) return FASTEQ_OK;
  if (!go || !x1 || !x0 || !i0 || !gx1 || (NEED_GX0 && !gx0_per_node)) return FASTEQ_INVALID;
  int* st = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&st, g_status_word);
  if (e != cudaSuccess) return cuda_fail(e);
  const long long grid = batch < (1LL << 30) ? batch : (1LL << 30);
  fasteq_stc_bwd_kernel<<<(unsigned)grid, NT, 0, (cudaStream_t)stream>>>((const T*)go, (const T*)x1, (const T*)x0, i0, batch,
                                                                        n_species, (T*)gx1, (T*)gx0_per_node, st);
  e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}
extern "C" int fasteq_stc_double_backward(const void*, const void*, const void*, const int32_t*, const void*, const void*, int64_t,
                                          int64_t, void*, void*, void*, fasteq_stream_t) {
  return FASTEQ_UNSUPPORTED;  // this module holds another direction
}
""")
    return head + "\n".join(body) + "\n"


def arith_ops(spec: STCSpec, direction: str, need_gx0: bool = False) -> Dict[str, int]:
    """Floating-point instructions one (node, channel) thread executes in the generated kernel, counted in its
    source text: ``fma(...)`` calls and explicit multiplications (the kernel body is straight-line code, so the
    count is the executed count).  Used to state the kernels' FP32-issue utilisation."""
    import re
    src = emit_stc(spec, direction, need_gx0)
    body = src[src.index("__global__"):]
    end = body.find('extern "C"')
    body = body[:end if end > 0 else len(body)]
    body = re.sub(r"//[^\n]*", "", body)
    body = re.sub(r"\[[^\]]*\]", "[]", body)                                   # subscripts hold index arithmetic only
    body = "\n".join(ln for ln in body.splitlines() if "size_t" not in ln and "const T*" not in ln)
    fma = len(re.findall(r"\bfma\(", body))
    mul = len(re.findall(r"\s\*\s", body)) - len(re.findall(r"\b1\.0f? \* ", body))   # x * 1.0 is folded away by the compiler
    return {"fma": fma, "mul": mul}
