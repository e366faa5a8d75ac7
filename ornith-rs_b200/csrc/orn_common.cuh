// Shared device/host helpers for the sm_100a decode library.
//
// Numerical contract of the whole library: every float operation below is a
// single IEEE-754 binary32 operation (add, mul, fma, div, sqrt) written out
// explicitly.  The translation units are compiled with `-fmad=false`, so the
// compiler never contracts a mul+add into an fma on its own; an fma happens
// exactly where `fmaf` is written.  A CPU restatement that performs the same
// operations in the same order therefore reproduces every result bit for bit,
// which is what lets routing indices and greedy token ids be compared exactly.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>

#define ORN_HD __host__ __device__ __forceinline__
#define ORN_D __device__ __forceinline__

#define ORN_OK 0
#define ORN_ERR_ARG (-1)
#define ORN_ERR_ALLOC (-2)
#define ORN_ERR_CUDA (-3)
#define ORN_ERR_TIMEOUT (-4)
#define ORN_ERR_IO (-5)
#define ORN_ERR_STATE (-6)

// ---------------------------------------------------------------------------
// bit casts
// ---------------------------------------------------------------------------
ORN_HD uint32_t orn_f2u(float f) {
#ifdef __CUDA_ARCH__
  return __float_as_uint(f);
#else
  union { float f; uint32_t u; } v; v.f = f; return v.u;
#endif
}
ORN_HD float orn_u2f(uint32_t u) {
#ifdef __CUDA_ARCH__
  return __uint_as_float(u);
#else
  union { float f; uint32_t u; } v; v.u = u; return v.f;
#endif
}

// bfloat16 as raw uint16.  Rounding: nearest, ties to even (the reference
// states the same rule in src/array.rs:229-237).
typedef uint16_t bf16_t;

ORN_HD float bf2f(bf16_t h) { return orn_u2f(((uint32_t)h) << 16); }
ORN_HD bf16_t f2bf(float f) {
#ifdef __CUDA_ARCH__
  // one instruction on the device; equal to the integer form below for every input that is not
  // a NaN (a NaN comes back as the canonical quiet NaN instead of keeping its payload)
  unsigned short r;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
  return r;
#endif
  uint32_t u = orn_f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_t)((u >> 16) | 0x40);  // NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return (bf16_t)(u >> 16);
}
// round a float to the nearest bfloat16 value, kept as float
ORN_HD float bfr(float f) { return bf2f(f2bf(f)); }

// IEEE half -> float, subnormals included (k-quant super-scales at the 1e-3
// scale of the synthetic artifacts are often subnormal halves).
ORN_HD float h2f(uint16_t h) {
#ifdef __CUDA_ARCH__
  float r;  // the hardware conversion is exact for every half, subnormals included
  asm("cvt.f32.f16 %0, %1;" : "=f"(r) : "h"(h));
  return r;
#endif
  uint32_t s = ((uint32_t)(h & 0x8000u)) << 16;
  uint32_t e = (h >> 10) & 0x1fu;
  uint32_t m = h & 0x3ffu;
  if (e == 0) {
    float v = (float)m * 5.9604644775390625e-08f;  // m * 2^-24, exact
    return s ? -v : v;
  }
  if (e == 31) return orn_u2f(s | 0x7f800000u | (m << 13));
  return orn_u2f(s | ((e + 112u) << 23) | (m << 13));
}

// ---------------------------------------------------------------------------
// elementary functions, written once for device and host
// ---------------------------------------------------------------------------
#define ORN_LN2_HI 0.693145751953125f
#define ORN_LN2_LO 1.42860682030941723212e-6f

// e^x, about 1 ulp.  n = rint(x*log2 e); r = x - n ln2 (two parts); degree-7
// Horner polynomial in fma form; scaled by 2^n through the exponent field.
ORN_HD float orn_expf(float x) {
  if (x < -87.0f) return 0.0f;
  if (x > 88.5f) return orn_u2f(0x7f800000u);
  float n = rintf(x * 1.44269504088896341f);
  float r = fmaf(n, -ORN_LN2_HI, x);
  r = fmaf(n, -ORN_LN2_LO, r);
  float p = 1.9841269841e-4f;         // 1/5040
  p = fmaf(p, r, 1.3888888889e-3f);    // 1/720
  p = fmaf(p, r, 8.3333333333e-3f);    // 1/120
  p = fmaf(p, r, 4.1666666667e-2f);    // 1/24
  p = fmaf(p, r, 1.6666666667e-1f);    // 1/6
  p = fmaf(p, r, 0.5f);
  p = fmaf(p, r, 1.0f);
  p = fmaf(p, r, 1.0f);
  int ni = (int)n;  // in [-126, 128]
  if (ni > 127) {   // keep the scale factor a finite normal number
    p = p * 2.0f;
    ni -= 1;
  }
  return p * orn_u2f((uint32_t)(ni + 127) << 23);
}

// natural log of a finite x > 0, about 1-2 ulp.  x = m 2^e with m in
// [sqrt(1/2), sqrt 2); log m = 2 atanh(s), s = (m-1)/(m+1), odd series in s.
ORN_HD float orn_logf(float x) {
  int e = 0;
  uint32_t u = orn_f2u(x);
  if (u < 0x00800000u) {
    x = x * 8388608.0f;
    u = orn_f2u(x);
    e = -23;
  }
  int32_t t = (int32_t)(u - 0x3f3504f3u);
  e += (int)(t >> 23);
  float m = orn_u2f((uint32_t)(t & 0x007fffff) + 0x3f3504f3u);
  float f = m - 1.0f;
  float s = f / (2.0f + f);
  float z = s * s;
  float p = 0.1111111111f;         // 1/9
  p = fmaf(p, z, 0.1428571429f);   // 1/7
  p = fmaf(p, z, 0.2f);            // 1/5
  p = fmaf(p, z, 0.3333333333f);   // 1/3
  p = p * z;
  float s2 = s + s;
  float lm = fmaf(s2, p, s2);
  float fe = (float)e;
  return fmaf(fe, ORN_LN2_HI, fmaf(fe, ORN_LN2_LO, lm));
}

// log(1 + x) for x >= 0
ORN_HD float orn_log1pf(float x) {
  float u = 1.0f + x;
  if (u == 1.0f) return x;
  return orn_logf(u) * (x / (u - 1.0f));
}

// sin and cos of a finite angle up to about 1e5 rad: three-part Cody-Waite
// reduction by pi/2, then the usual minimax-style polynomials on [-pi/4, pi/4].
ORN_HD void orn_sincosf(float a, float* sn, float* cs) {
  float k = rintf(a * 0.636619772367581343f);
  float r = fmaf(k, -1.5703125f, a);                       // pi/2 high bits
  r = fmaf(k, -4.8375129699707031e-4f, r);                  // middle bits
  r = fmaf(k, -7.5497899548918821e-8f, r);                  // low bits
  float z = r * r;
  float ps = -1.9515295891e-4f;
  ps = fmaf(ps, z, 8.3321608736e-3f);
  ps = fmaf(ps, z, -1.6666654611e-1f);
  float s = fmaf(ps * z, r, r);
  float pc = 2.443315711809948e-5f;
  pc = fmaf(pc, z, -1.388731625493765e-3f);
  pc = fmaf(pc, z, 4.166664568298827e-2f);
  float c = fmaf(pc * z, z, fmaf(-0.5f, z, 1.0f));
  int q = ((int)k) & 3;
  float so = (q & 1) ? c : s;
  float co = (q & 1) ? s : c;
  if (q == 1 || q == 2) co = -co;
  if (q >= 2) so = -so;
  *sn = so;
  *cs = co;
}

// 1/sqrt(x) as one IEEE sqrt and one IEEE division
ORN_HD float orn_rsqrtf(float x) { return 1.0f / sqrtf(x); }

// Sigmoid of a bfloat16 value evaluated in bfloat16, every intermediate
// rounded: y = 1/(1+exp(|x|)); x<0 ? y : 1-y  (kernels/ornith_sigmoid.h:17-22
// of the reference; the reference's "fast" and "precise" flavours differ on a
// single input and share one exponential here).
ORN_HD float orn_sigmoid_bf(float x /* a bf16 value */) {
  float e = bfr(orn_expf(fabsf(x)));
  float d = bfr(1.0f + e);
  float y = bfr(1.0f / d);
  return (x < 0.0f) ? y : bfr(1.0f - y);
}
// the same form evaluated in float (rms_norm_gated's gate)
ORN_HD float orn_sigmoid_f32(float x) {
  float y = 1.0f / (1.0f + orn_expf(fabsf(x)));
  return (x < 0.0f) ? y : 1.0f - y;
}
// silu in bfloat16: bf(x * sigmoid_bf(x))
ORN_HD float orn_silu_bf(float x) { return bfr(x * orn_sigmoid_bf(x)); }
// swiglu in bfloat16: bf( bf(g*sigmoid(g)) * u )   (ornith_elementwise.metal:94-105)
ORN_HD float orn_swiglu_bf(float g, float u) { return bfr(orn_silu_bf(g) * u); }

// softplus evaluated in bfloat16 as logaddexp(x, 0) = max + log1p(exp(min-max))
// (kernels/ornith_logaddexp.h:13-23)
ORN_HD float orn_softplus_bf(float x /* bf16 value */) {
  float mx = x > 0.0f ? x : 0.0f;
  float mn = x > 0.0f ? 0.0f : x;
  float d = bfr(mn - mx);
  float e = bfr(orn_expf(d));
  float l = bfr(orn_log1pf(e));
  return bfr(mx + l);
}

#ifdef __CUDACC__
// ---------------------------------------------------------------------------
// warp helpers (device only)
// ---------------------------------------------------------------------------
// Butterfly sum over the 32 lanes: xor 16, 8, 4, 2, 1.  Every lane ends with
// the same value; the CPU restatement folds a 32-entry array the same way.
// programmatic dependent launch: let the next kernel of the stream start / wait for the previous ones
ORN_D void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
ORN_D void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

ORN_D float warp_sum(float v) {
  v = v + __shfl_xor_sync(0xffffffffu, v, 16);
  v = v + __shfl_xor_sync(0xffffffffu, v, 8);
  v = v + __shfl_xor_sync(0xffffffffu, v, 4);
  v = v + __shfl_xor_sync(0xffffffffu, v, 2);
  v = v + __shfl_xor_sync(0xffffffffu, v, 1);
  return v;
}
ORN_D float warp_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return v;
}
ORN_D uint32_t warp_max_u32(uint32_t v) {
  v = max(v, __shfl_xor_sync(0xffffffffu, v, 16));
  v = max(v, __shfl_xor_sync(0xffffffffu, v, 8));
  v = max(v, __shfl_xor_sync(0xffffffffu, v, 4));
  v = max(v, __shfl_xor_sync(0xffffffffu, v, 2));
  v = max(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return v;
}
ORN_D uint32_t warp_min_u32(uint32_t v) {
  v = min(v, __shfl_xor_sync(0xffffffffu, v, 16));
  v = min(v, __shfl_xor_sync(0xffffffffu, v, 8));
  v = min(v, __shfl_xor_sync(0xffffffffu, v, 4));
  v = min(v, __shfl_xor_sync(0xffffffffu, v, 2));
  v = min(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return v;
}

ORN_D uint4 ldg128(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
// streaming 16-byte load for weights that are read once per step
ORN_D uint4 ldg128_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
ORN_D uint32_t ldg32_stream(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
#endif  // __CUDACC__
