/* TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Scalar CPU restatement of the arithmetic of ornith-rs's decode hot path.
 * Only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark may load this; the CUDA library never does.
 *
 * Parity status: the reference (Rust + Metal) cannot be built or run on Linux,
 * and its golden tensors (refs/) are not distributed with it.  What is pinned:
 * Q4_K decode, field packing and the plain quantiser against the reference's
 * own numpy port tools/q4k.py, and 8-bit affine quantise/pack against
 * tools/aq.py (fixtures under tests/golden/).  Everything else follows the
 * reference's kernels by reading and is "parity unpinned" against the
 * reference's GPU output.  Metal leaves the order of simd_sum unspecified and
 * its fast:: exp/sin/cos have no bit-exact CUDA twin, so this file DEFINES the
 * reduction orders and elementary functions; the CUDA kernels mirror them.
 *
 * Build: gcc -O2 -ffp-contract=off -mfma (no fast-math).  With contraction off
 * an fma happens exactly where fmaf() is written, as in the CUDA code.
 */
#ifndef ORN_ORACLE_MATH_H
#define ORN_ORACLE_MATH_H

#include <math.h>
#include <stdint.h>
#include <string.h>

typedef uint16_t bf16;

static inline uint32_t o_f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float o_u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* bfloat16: round to nearest, ties to even (src/array.rs:229-237) */
static inline float o_bf2f(bf16 h) { return o_u2f(((uint32_t)h) << 16); }
static inline bf16 o_f2bf(float f) {
  uint32_t u = o_f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (bf16)(u >> 16);
}
static inline float o_bfr(float f) { return o_bf2f(o_f2bf(f)); }

/* IEEE half -> float (src/array.rs:279-284 lists known values) */
static inline float o_h2f(uint16_t h) {
  uint32_t s = ((uint32_t)(h & 0x8000u)) << 16;
  uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
  if (e == 0) { float v = (float)m * 5.9604644775390625e-08f; return s ? -v : v; }
  if (e == 31) return o_u2f(s | 0x7f800000u | (m << 13));
  return o_u2f(s | ((e + 112u) << 23) | (m << 13));
}

#define O_LN2_HI 0.693145751953125f
#define O_LN2_LO 1.42860682030941723212e-6f

static inline float o_expf(float x) {
  if (x < -87.0f) return 0.0f;
  if (x > 88.5f) return o_u2f(0x7f800000u);
  float n = rintf(x * 1.44269504088896341f);
  float r = fmaf(n, -O_LN2_HI, x);
  r = fmaf(n, -O_LN2_LO, r);
  float p = 1.9841269841e-4f;
  p = fmaf(p, r, 1.3888888889e-3f);
  p = fmaf(p, r, 8.3333333333e-3f);
  p = fmaf(p, r, 4.1666666667e-2f);
  p = fmaf(p, r, 1.6666666667e-1f);
  p = fmaf(p, r, 0.5f);
  p = fmaf(p, r, 1.0f);
  p = fmaf(p, r, 1.0f);
  int ni = (int)n;
  if (ni > 127) { p = p * 2.0f; ni -= 1; }
  return p * o_u2f((uint32_t)(ni + 127) << 23);
}

static inline float o_logf(float x) {
  int e = 0;
  uint32_t u = o_f2u(x);
  if (u < 0x00800000u) { x = x * 8388608.0f; u = o_f2u(x); e = -23; }
  int32_t t = (int32_t)(u - 0x3f3504f3u);
  e += (int)(t >> 23);
  float m = o_u2f((uint32_t)(t & 0x007fffff) + 0x3f3504f3u);
  float f = m - 1.0f;
  float s = f / (2.0f + f);
  float z = s * s;
  float p = 0.1111111111f;
  p = fmaf(p, z, 0.1428571429f);
  p = fmaf(p, z, 0.2f);
  p = fmaf(p, z, 0.3333333333f);
  p = p * z;
  float s2 = s + s;
  float lm = fmaf(s2, p, s2);
  float fe = (float)e;
  return fmaf(fe, O_LN2_HI, fmaf(fe, O_LN2_LO, lm));
}

static inline float o_log1pf(float x) {
  float u = 1.0f + x;
  if (u == 1.0f) return x;
  return o_logf(u) * (x / (u - 1.0f));
}

static inline void o_sincosf(float a, float* sn, float* cs) {
  float k = rintf(a * 0.636619772367581343f);
  float r = fmaf(k, -1.5703125f, a);
  r = fmaf(k, -4.8375129699707031e-4f, r);
  r = fmaf(k, -7.5497899548918821e-8f, r);
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
  *sn = so; *cs = co;
}

static inline float o_rsqrtf(float x) { return 1.0f / sqrtf(x); }

/* kernels/ornith_sigmoid.h:17-22, evaluated in bfloat16 step by step */
static inline float o_sigmoid_bf(float x) {
  float e = o_bfr(o_expf(fabsf(x)));
  float d = o_bfr(1.0f + e);
  float y = o_bfr(1.0f / d);
  return (x < 0.0f) ? y : o_bfr(1.0f - y);
}
static inline float o_sigmoid_f32(float x) {
  float y = 1.0f / (1.0f + o_expf(fabsf(x)));
  return (x < 0.0f) ? y : 1.0f - y;
}
static inline float o_silu_bf(float x) { return o_bfr(x * o_sigmoid_bf(x)); }
/* kernels/ornith_elementwise.metal:94-105 */
static inline float o_swiglu_bf(float g, float u) { return o_bfr(o_silu_bf(g) * u); }
/* kernels/ornith_logaddexp.h:13-23 with y = 0, in bfloat16 */
static inline float o_softplus_bf(float x) {
  float mx = x > 0.0f ? x : 0.0f;
  float mn = x > 0.0f ? 0.0f : x;
  float d = o_bfr(mn - mx);
  float e = o_bfr(o_expf(d));
  float l = o_bfr(o_log1pf(e));
  return o_bfr(mx + l);
}

/* The 32-lane butterfly (xor 16,8,4,2,1) as seen by lane 0; `a` is clobbered. */
static inline float o_fold32(float* a) {
  for (int off = 16; off >= 1; off >>= 1)
    for (int i = 0; i < off; ++i) a[i] = a[i] + a[i + off];
  return a[0];
}

#endif
