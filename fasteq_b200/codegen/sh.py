"""CUDA source emitter for the real spherical harmonics of edge vectors (forward and vector gradient).

One thread per edge evaluates the polynomials of ``fasteq_b200.sh.sh_polynomials`` as straight-line
code with literal coefficients (monomials shared between components), the analytic Jacobian for the
backward, and the chain rule through ``r / max(|r|, 1e-12)`` when ``normalize`` is set.  Same job as
the reference's generated Triton kernels (fasteq/triton/spherical_harmonics.py:352-422; analytic
Jacobian recipe :368-383).
"""
from __future__ import annotations

from math import pi, sqrt
from typing import Dict, List, Tuple

from ..sh import Poly, derivative, sh_polynomials
from .u1d_common import lit


def _mono_name(e: Tuple[int, int, int]) -> str:
    return f"m_{e[0]}_{e[1]}_{e[2]}"


def _collect(polys: List[Poly]) -> List[Tuple[int, int, int]]:
    need = set()
    for p in polys:
        need |= set(p)
    # close under "drop one factor" so that every monomial is one multiply from a smaller one
    out = set()
    def add(e):
        if e in out or sum(e) == 0:
            return
        out.add(e)
        for ax in range(3):
            if e[ax] > 0:
                s = list(e); s[ax] -= 1
                add(tuple(s))
                break
    for e in need:
        add(e)
    return sorted(out, key=lambda e: (sum(e), e))


def _emit_monomials(monos, ind) -> List[str]:
    L = []
    names = {(1, 0, 0): "x", (0, 1, 0): "y", (0, 0, 1): "z"}
    for e in monos:
        if sum(e) == 1:
            continue
        for ax in range(3):
            if e[ax] > 0:
                s = list(e); s[ax] -= 1; s = tuple(s)
                base = names.get(s, _mono_name(s))
                L.append(f"{ind}const T {_mono_name(e)} = {base} * {'xyz'[ax]};")
                break
    return L


def _poly_expr(p: Poly, dt: str) -> str:
    names = {(1, 0, 0): "x", (0, 1, 0): "y", (0, 0, 1): "z"}
    terms = []
    for e, c in sorted(p.items()):
        if sum(e) == 0:
            terms.append(lit(c, dt))
        else:
            terms.append(f"{lit(c, dt)} * {names.get(e, _mono_name(e))}")
    return " + ".join(terms) if terms else ("0.0f" if dt == "f32" else "0.0")


def _emit_double_backward(ls, comps, grads, load: str, dt: str) -> str:
    """Second-order kernel.  With ``t = ggvec`` (cotangent of the vector gradient) and ``g = grad_out``:

        d_grad_out[i] = <dY_i/dv, t>            d_vec = sum_i g_i (d^2 Y_i / dv dv) t

    For normalised input ``Y_i(v) = P_i(v) |v|^-l`` (``P_i`` homogeneous of degree ``l``), so with ``u = v/|v|``:

        dY/dv_a        = (dP/da - l u_a P) / |v|
        d2Y/dv_a dv_b  = (d2P/da db - l (u_b dP/da + u_a dP/db + delta_ab P) + l (l + 2) u_a u_b P) / |v|^2

    all evaluated at ``u`` (the reference keeps an analytic Hessian-vector product for the same purpose,
    fasteq/triton/spherical_harmonics.py:368-383)."""
    n = len(comps)
    degs = [l for l in ls for _ in range(2 * l + 1)]
    hess = [[[derivative(grads[a][i], b) for b in range(3)] for a in range(3)] for i in range(n)]
    polys = list(comps) + [grads[a][i] for a in range(3) for i in range(n)] + [hess[i][a][b] for i in range(n) for a in range(3) for b in range(3)]
    L = [f"""
__global__ void __launch_bounds__(256) fasteq_sh_dbwd_kernel(const T* __restrict__ v, const T* __restrict__ gout,
                                                            const T* __restrict__ ggv, long long n, T* __restrict__ d_gout,
                                                            T* __restrict__ d_v) {{
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {{
{load}
    const T tx = ggv[3 * e], ty = ggv[3 * e + 1], tz = ggv[3 * e + 2];
    const bool proj = NORMALIZE && (x * x + y * y + z * z) > T(0.5);    // above the clamp: true unit vector
    const T ut = x * tx + y * ty + z * tz;
    const T* g = gout + e * NOUT;
    T* dg = d_gout + e * NOUT;
    T dvx = T(0), dvy = T(0), dvz = T(0);"""]
    L += _emit_monomials(_collect(polys), "    ")
    zero = "T(0)"
    for i in range(n):
        l = degs[i]
        ex = lambda p: _poly_expr(p, dt) if p else zero
        L.append("    {")
        L.append(f"      const T P = {ex(comps[i])}, gx_ = {ex(grads[0][i])}, gy_ = {ex(grads[1][i])}, gz_ = {ex(grads[2][i])};")
        for b, nm in enumerate(("hx", "hy", "hz")):
            L.append(f"      const T {nm} = tx * ({ex(hess[i][0][b])}) + ty * ({ex(hess[i][1][b])}) + tz * ({ex(hess[i][2][b])});")
        L.append("      const T gt = gx_ * tx + gy_ * ty + gz_ * tz, gi = g[%d];" % i)
        L.append(f"      T dgi = gt, ax = hx, ay = hy, az = hz;")
        if l > 0:
            L.append(f"      if (proj) {{ dgi -= T({l}) * ut * P;")
            L.append(f"        ax += -T({l}) * (x * gt + ut * gx_ + tx * P) + T({l * (l + 2)}) * x * ut * P;")
            L.append(f"        ay += -T({l}) * (y * gt + ut * gy_ + ty * P) + T({l * (l + 2)}) * y * ut * P;")
            L.append(f"        az += -T({l}) * (z * gt + ut * gz_ + tz * P) + T({l * (l + 2)}) * z * ut * P; }}")
        L.append(f"      dg[{i}] = dgi * inv; dvx += gi * ax; dvy += gi * ay; dvz += gi * az;")
        L.append("    }")
    L.append("    const T inv2 = inv * inv;")
    L.append("    d_v[3 * e] = dvx * inv2; d_v[3 * e + 1] = dvy * inv2; d_v[3 * e + 2] = dvz * inv2;")
    L.append("  }\n}")
    return "\n".join(L)


def emit_sh(ls: Tuple[int, ...], dtype: str, normalize: bool, normalization: str) -> str:
    dt = dtype
    ctype = "float" if dt == "f32" else "double"
    lmax = max(ls)
    table = sh_polynomials(lmax)
    comps: List[Poly] = []
    for l in ls:
        scale = {"component": 1.0, "norm": 1.0 / sqrt(2 * l + 1), "integral": 1.0 / sqrt(4 * pi)}[normalization]
        for p in table[l]:
            comps.append({e: c * scale for e, c in p.items()})
    n = len(comps)
    grads = [[derivative(p, ax) for p in comps] for ax in range(3)]
    fwd_monos = _collect(comps)
    bwd_monos = _collect([g for ax in range(3) for g in grads[ax]])
    one = "1.0f" if dt == "f32" else "1.0"
    eps = "1e-12f" if dt == "f32" else "1e-12"
    load = f"""    T x = v[3 * e], y = v[3 * e + 1], z = v[3 * e + 2];
    T inv = {one};
    if (NORMALIZE) {{ const T r = sqrt(x * x + y * y + z * z); inv = {one} / (r > {eps} ? r : {eps}); x *= inv; y *= inv; z *= inv; }}"""
    src = [f"""// Generated by fasteq_b200.codegen.sh -- do not edit.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "fasteq_b200.h"
typedef {ctype} T;
constexpr int NOUT = {n};
constexpr bool NORMALIZE = {str(normalize).lower()};
static thread_local char g_err[256];
static int cuda_fail(cudaError_t e) {{ snprintf(g_err, sizeof(g_err), "%s", cudaGetErrorString(e)); return FASTEQ_CUDA_ERROR; }}
extern "C" const char* fasteq_last_cuda_error(void) {{ return g_err; }}
extern "C" int fasteq_sh_num_outputs(void) {{ return NOUT; }}

__global__ void __launch_bounds__(256) fasteq_sh_fwd_kernel(const T* __restrict__ v, long long n, T* __restrict__ out) {{
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {{
{load}"""]
    src += _emit_monomials(fwd_monos, "    ")
    src.append("    T* o = out + e * NOUT;")
    for i, p in enumerate(comps):
        src.append(f"    o[{i}] = {_poly_expr(p, dt)};")
    src.append("  }\n}")
    src.append(f"""
__global__ void __launch_bounds__(256) fasteq_sh_bwd_kernel(const T* __restrict__ v, const T* __restrict__ gout, long long n,
                                                           T* __restrict__ gv) {{
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {{
{load}""")
    src += _emit_monomials(bwd_monos, "    ")
    src.append("    const T* g = gout + e * NOUT;")
    src.append("    T gx = T(0), gy = T(0), gz = T(0);")
    for i in range(n):
        parts = []
        for ax, name in enumerate(("gx", "gy", "gz")):
            if grads[ax][i]:
                parts.append(f"{name} += gi * ({_poly_expr(grads[ax][i], dt)});")
        if parts:
            src.append(f"    {{ const T gi = g[{i}]; " + " ".join(parts) + " }")
    dbwd = _emit_double_backward(ls, comps, grads, load, dt)
    src.append("""    if (NORMALIZE) {
      // d(r/|r|)/dr = (I - u u^T) / |r| ; below the clamp the map is linear with slope 1/eps
      const T dot = gx * x + gy * y + gz * z;
      const T r2 = x * x + y * y + z * z;        // 1 when |r| was above the clamp
      if (r2 > T(0.5)) { gx -= x * dot; gy -= y * dot; gz -= z * dot; }
      gx *= inv; gy *= inv; gz *= inv;
    }
    gv[3 * e] = gx; gv[3 * e + 1] = gy; gv[3 * e + 2] = gz;
  }
}
""" + dbwd + """
extern "C" int fasteq_sh_double_backward(const void* vec, const void* grad_out, const void* ggvec, int64_t n, void* d_grad_out,
                                         void* d_vec, fasteq_stream_t stream) {
  if (n < 0) return FASTEQ_INVALID;
  if (n == 0) return FASTEQ_OK;
  if (!vec || !grad_out || !ggvec || !d_grad_out || !d_vec) return FASTEQ_INVALID;
  long long blocks = (n + 255) / 256; if (blocks > 148 * 32) blocks = 148 * 32;
  fasteq_sh_dbwd_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const T*)vec, (const T*)grad_out, (const T*)ggvec, n,
                                                                          (T*)d_grad_out, (T*)d_vec);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

extern "C" int fasteq_sh_forward(const void* vec, int64_t n, void* out, fasteq_stream_t stream) {
  if (n < 0) return FASTEQ_INVALID;
  if (n == 0) return FASTEQ_OK;
  if (!vec || !out) return FASTEQ_INVALID;
  long long blocks = (n + 255) / 256; if (blocks > 148 * 32) blocks = 148 * 32;
  fasteq_sh_fwd_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const T*)vec, n, (T*)out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}

extern "C" int fasteq_sh_backward(const void* vec, const void* grad_out, int64_t n, void* grad_vec, fasteq_stream_t stream) {
  if (n < 0) return FASTEQ_INVALID;
  if (n == 0) return FASTEQ_OK;
  if (!vec || !grad_out || !grad_vec) return FASTEQ_INVALID;
  long long blocks = (n + 255) / 256; if (blocks > 148 * 32) blocks = 148 * 32;
  fasteq_sh_bwd_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const T*)vec, (const T*)grad_out, n, (T*)grad_vec);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTEQ_OK : cuda_fail(e);
}
""")
    return "\n".join(src)


def emit_sh_device(ls: Tuple[int, ...], dtype: str, normalize: bool, normalization: str) -> str:
    """``fasteq_sh::eval`` / ``fasteq_sh::vjp`` device functions (same polynomials and Jacobian as the
    stand-alone kernels) for kernels that evaluate the harmonics of an edge vector in place."""
    dt = dtype
    lmax = max(ls)
    table = sh_polynomials(lmax)
    comps: List[Poly] = []
    for l in ls:
        scale = {"component": 1.0, "norm": 1.0 / sqrt(2 * l + 1), "integral": 1.0 / sqrt(4 * pi)}[normalization]
        for p in table[l]:
            comps.append({e: c * scale for e, c in p.items()})
    n = len(comps)
    grads = [[derivative(p, ax) for p in comps] for ax in range(3)]
    one = "1.0f" if dt == "f32" else "1.0"
    eps = "1e-12f" if dt == "f32" else "1e-12"
    norm = f"""  T inv = {one};
  if (NORMALIZE) {{ const T r = sqrt(x * x + y * y + z * z); inv = {one} / (r > {eps} ? r : {eps}); x *= inv; y *= inv; z *= inv; }}"""
    L = [f"""namespace fasteq_sh {{
using T = cfg::T;
constexpr int NOUT = {n};
constexpr bool NORMALIZE = {str(normalize).lower()};
__device__ __forceinline__ void eval(T x, T y, T z, T* o) {{
{norm}
  (void)inv;"""]
    L += _emit_monomials(_collect(comps), "  ")
    for i, p in enumerate(comps):
        L.append(f"  o[{i}] = {_poly_expr(p, dt)};")
    L.append("}")
    L.append(f"""__device__ __forceinline__ void vjp(T x, T y, T z, const T* g, T* gv) {{
{norm}""")
    L += _emit_monomials(_collect([g for ax in range(3) for g in grads[ax]]), "  ")
    L.append("  T gx = T(0), gy = T(0), gz = T(0);")
    for i in range(n):
        parts = []
        for ax, name in enumerate(("gx", "gy", "gz")):
            if grads[ax][i]:
                parts.append(f"{name} += gi * ({_poly_expr(grads[ax][i], dt)});")
        if parts:
            L.append(f"  {{ const T gi = g[{i}]; " + " ".join(parts) + " }")
    L.append("""  if (NORMALIZE) {
    const T dot = gx * x + gy * y + gz * z;
    const T r2 = x * x + y * y + z * z;        // 1 when |r| was above the clamp
    if (r2 > T(0.5)) { gx -= x * dot; gy -= y * dot; gz -= z * dot; }
    gx *= inv; gy *= inv; gz *= inv;
  }
  gv[0] = gx; gv[1] = gy; gv[2] = gz;
}
}  // namespace fasteq_sh
""")
    return "\n".join(L)


SH_DEVICE_STUB = """namespace fasteq_sh {
using T = cfg::T;
__device__ __forceinline__ void eval(T, T, T, T*) {}
__device__ __forceinline__ void vjp(T, T, T, const T*, T*) {}
}  // namespace fasteq_sh
"""
