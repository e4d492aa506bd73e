// Device-side building blocks shared by the generated sm_100a kernels:
// mbarrier producer/consumer pipeline primitives with BOUNDED waits, 1-D bulk
// asynchronous copies (the TMA engine's untiled form), reductions.
//
// Every wait loop is bounded: when the limit is hit the waiter records an error
// code in a status word and falls through, so a broken pipeline yields a
// wrong-but-finite kernel and a non-zero status instead of a hung GPU (the same
// policy as the reference's FP32 TMA GEMM,
// fasteq/cuda/src/eqlinear/backends/fp32/simt_gemm.cu:85-107).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace fasteq {

enum DeviceStatus : int {
  kDevOk = 0,
  kDevWaitTimeout = 1,   // an mbarrier wait gave up
  kDevBadIndex = 2,      // a gather/scatter index was outside its tensor
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait: gives up after about two seconds of wall time (checked every 256 failed
// probes).  Returns false (and flags *status) if the phase never completed.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    // once any wait in this launch has failed, the rest give up at once so the kernel ends quickly
    if (*reinterpret_cast<volatile int*>(status) != 0) return false;
    if (global_timer_ns() - t0 > 2000000000ull) break;
  }
  atomicExch(status, (int)kDevWaitTimeout);
  return false;
}

// 1-D bulk copy global -> shared (TMA engine, no tensor map): both addresses
// 16-byte aligned, size a multiple of 16 bytes; completion is signalled on the
// mbarrier as transferred bytes.  The copy targets this CTA only.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Ask the TMA engine to bring [gmem_src, gmem_src + bytes) into L2 (no destination, no completion to wait for):
// 16-byte aligned address, size a multiple of 16 bytes.  Used by the producers to run ahead of their ring.
__device__ __forceinline__ void bulk_prefetch_l2(const void* gmem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gmem_src), "r"(bytes) : "memory");
}

// 1-D bulk copy shared -> global, tracked by the per-thread bulk async-group.
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

// generic-proxy writes to shared memory -> visible to the async proxy (bulk stores)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void red_add(float* p, float v) { asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory"); }
__device__ __forceinline__ void red_add(double* p, double v) { asm volatile("red.global.add.f64 [%0], %1;" ::"l"(p), "d"(v) : "memory"); }

// red.global.add of two adjacent floats in one instruction (8-byte aligned address)
__device__ __forceinline__ void red_add2(float* p, float2 v) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(v.x), "f"(v.y) : "memory");
}

// ---- value abstraction used by the generated arithmetic: a "value" is one channel (float or
// double) or two adjacent FP32 channels packed in a float2 and processed with the sm_100
// f32x2 instructions (one issue slot for two FMAs; literal multipliers become packed
// constant-bank operands).
__device__ __forceinline__ float vmul(float a, float b) { return a * b; }
__device__ __forceinline__ float vfma(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ float vadd(float a, float b) { return a + b; }
__device__ __forceinline__ double vmul(double a, double b) { return a * b; }
__device__ __forceinline__ double vfma(double a, double b, double c) { return fma(a, b, c); }
__device__ __forceinline__ double vadd(double a, double b) { return a + b; }
__device__ __forceinline__ unsigned long long f2_bits(float2 a) { return *reinterpret_cast<unsigned long long*>(&a); }
__device__ __forceinline__ float2 vmul(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(*reinterpret_cast<unsigned long long*>(&d)) : "l"(f2_bits(a)), "l"(f2_bits(b)));
  return d;
}
__device__ __forceinline__ float2 vfma(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(f2_bits(a)), "l"(f2_bits(b)), "l"(f2_bits(c)));
  return d;
}
__device__ __forceinline__ float2 vadd(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(*reinterpret_cast<unsigned long long*>(&d)) : "l"(f2_bits(a)), "l"(f2_bits(b)));
  return d;
}
template <typename V> struct VT;
template <> struct VT<float> {
  using S = float; static constexpr int N = 1;
  static __device__ __forceinline__ float bc(float s) { return s; }
  static __device__ __forceinline__ float zero() { return 0.f; }
  static __device__ __forceinline__ float hsum(float v) { return v; }
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ float ldg(const float* p) { return __ldg(p); }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
  static __device__ __forceinline__ void red(float* p, float v) { red_add(p, v); }
};
template <> struct VT<double> {
  using S = double; static constexpr int N = 1;
  static __device__ __forceinline__ double bc(double s) { return s; }
  static __device__ __forceinline__ double zero() { return 0.0; }
  static __device__ __forceinline__ double hsum(double v) { return v; }
  static __device__ __forceinline__ double ld(const double* p) { return *p; }
  static __device__ __forceinline__ double ldg(const double* p) { return __ldg(p); }
  static __device__ __forceinline__ void st(double* p, double v) { *p = v; }
  static __device__ __forceinline__ void red(double* p, double v) { red_add(p, v); }
};
template <> struct VT<float2> {
  using S = float; static constexpr int N = 2;
  static __device__ __forceinline__ float2 bc(float s) { return make_float2(s, s); }
  static __device__ __forceinline__ float2 zero() { return make_float2(0.f, 0.f); }
  static __device__ __forceinline__ float hsum(float2 v) { return v.x + v.y; }
  static __device__ __forceinline__ float2 ld(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ float2 ldg(const float* p) { return __ldg(reinterpret_cast<const float2*>(p)); }
  static __device__ __forceinline__ void st(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
  static __device__ __forceinline__ void red(float* p, float2 v) { red_add2(p, v); }
};

// ---- tensor memory as per-thread scratch.  A thread of warp w can reach lanes 32 * (w % 4) .. + 31 of tensor memory,
// one lane per thread and up to 512 32-bit columns in it: values a thread parks there come back to the same thread, so no
// ordering against other threads is needed beyond the wait on its own stores / loads.  All of these are warp-collective.
__device__ __forceinline__ void scratch_tmem_alloc(uint32_t* smem_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void scratch_tmem_free(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void scratch_tmem_st(uint32_t addr, float v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(addr), "r"(__float_as_uint(v)) : "memory");
}
__device__ __forceinline__ void scratch_tmem_st(uint32_t addr, float2 v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(__float_as_uint(v.x)), "r"(__float_as_uint(v.y)) : "memory");
}
__device__ __forceinline__ void scratch_tmem_st(uint32_t addr, double v) {
  const unsigned long long b = (unsigned long long)__double_as_longlong(v);
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(addr), "r"((uint32_t)b), "r"((uint32_t)(b >> 32)) : "memory");
}
__device__ __forceinline__ void scratch_tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// the loaded registers are valid only after scratch_tmem_wait_ld(...) has been given them
__device__ __forceinline__ void scratch_tmem_ld(uint32_t addr, float& v) {
  uint32_t r;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(addr) : "memory");
  v = __uint_as_float(r);
}
__device__ __forceinline__ void scratch_tmem_ld(uint32_t addr, float2& v) {
  uint32_t r0, r1;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr) : "memory");
  v = make_float2(__uint_as_float(r0), __uint_as_float(r1));
}
__device__ __forceinline__ void scratch_tmem_ld(uint32_t addr, double& v) {
  uint32_t r0, r1;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr) : "memory");
  v = __longlong_as_double((long long)(((unsigned long long)r1 << 32) | r0));
}
// the wait names the values it releases, so that no use of them can be scheduled ahead of it
__device__ __forceinline__ void scratch_tmem_wait_ld(float& a) { asm volatile("tcgen05.wait::ld.sync.aligned;" : "+f"(a)::"memory"); }
__device__ __forceinline__ void scratch_tmem_wait_ld(float2& a) { asm volatile("tcgen05.wait::ld.sync.aligned;" : "+f"(a.x), "+f"(a.y)::"memory"); }
__device__ __forceinline__ void scratch_tmem_wait_ld(double& a) { asm volatile("tcgen05.wait::ld.sync.aligned;" : "+d"(a)::"memory"); }
__device__ __forceinline__ void scratch_tmem_pin(double& a) { asm volatile("" : "+d"(a)::"memory"); }
__device__ __forceinline__ void scratch_tmem_pin(float& a) { asm volatile("" : "+f"(a)::"memory"); }
__device__ __forceinline__ void scratch_tmem_pin(float2& a) { asm volatile("" : "+f"(a.x), "+f"(a.y)::"memory"); }

template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace fasteq
