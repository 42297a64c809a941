// Shared device helpers: storage-type conversion, 16-byte vector loads, warp
// reductions and the exact (erf) GELU the reference's nn.GELU computes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace wdz {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

// Elements of T in one 16-byte vector.
template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); };

// Load 16 bytes at p (16-byte aligned) and widen to float.
__device__ __forceinline__ void load_vec(const float* p, float (&v)[4]) {
  float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load_vec(const bf16* p, float (&v)[8]) {
  uint4 t = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
// Same through the read-only path, for streamed weights.
__device__ __forceinline__ void load_vec_nc(const float* p, float (&v)[4]) {
  float4 t = __ldg(reinterpret_cast<const float4*>(p));
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load_vec_nc(const bf16* p, float (&v)[8]) {
  uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}

// The same GELU, branch-free and with ONE special-function instruction, for the bf16 tensor-core epilogues (which are
// bound by the transcendental pipe: the library erff costs ~50 instructions with both of its branches taken in a warp,
// and a reciprocal + exponential form still saturated that pipe):
//   erf(z) = 1 - 2^(-q(z)),  z in [0, 4],  q = the degree-7 polynomial below (no constant term), fitted here by
//   weighted least squares to -log2(erfc(z)); beyond 4, erf is 1 to fp32 precision.
// Absolute error of erf: 1.6e-7 with an exact 2^x, about 4e-7 with ex2.approx - the size of fp32 rounding in the
// reference's own evaluation - so the GELU value is off by less than 1e-6 for every input, before it is rounded to
// bf16 (2^-9 relative) or added to an O(1) fp32 stream.
__device__ __forceinline__ float gelu_fast(float x) {
  const float z = x * 0.70710678118654752440f;
  const float a = fminf(fabsf(z), 4.0f);
  float q = -1.0020713708352587e-4f;
  q = fmaf(q, a, 4.6149219114128025e-4f);
  q = fmaf(q, a, 2.3024143134139e-3f);
  q = fmaf(q, a, -2.9452696402427522e-2f);
  q = fmaf(q, a, 1.489637594409859e-1f);
  q = fmaf(q, a, 9.183286244618459e-1f);
  q = fmaf(q, a, 1.6279137332204003f);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-q * a));
  const float er = copysignf(1.0f - e, z);
  const float h = 0.5f * x;
  return fmaf(h, er, h);
}

// Programmatic dependent launch: a kernel launched with the programmatic
// stream-serialization attribute may start while its predecessor is still
// running; pdl_wait() blocks until the predecessor has completed and its
// writes are visible (a no-op under a normal launch), pdl_trigger() lets the
// successor begin its own launch.  Every kernel of the decode step calls
// pdl_wait() before touching global memory, so ordering is preserved while
// launch latency and prologues overlap.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Device-side error word shared by all kernels of an engine (0 = fine).
struct DevStatus {
  int code;
  int detail;
};

}  // namespace wdz
