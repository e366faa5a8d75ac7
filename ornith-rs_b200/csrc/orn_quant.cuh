// Device helpers shared by the dequant mat-vec kernels: exact byte -> float
// conversion, bfloat16 widening, the Q4_K scale/min unpack.
#pragma once

#include "orn_common.cuh"

// float(byte I of w), exact: 0x4B0000bb is 2^23 + bb
template <int I>
ORN_D float byte_f(uint32_t w) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + I)) - 8388608.0f;
}
// float(byte I of w) - 32, exact
template <int I>
ORN_D float byte_m32_f(uint32_t w) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + I)) - 8388640.0f;
}
// ---- packed pairs of floats: fma.rn.f32x2 / add.rn.f32x2 do two IEEE operations per issue slot.
// A unit's products accumulate in two chains (even and odd elements), which is what one packed
// fma over (x[2i], x[2i+1]) x (q[2i], q[2i+1]) + (even, odd) computes.
ORN_D uint64_t pk2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
ORN_D float pk2_sum(uint64_t v) {  // even chain + odd chain
  float a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
  return a + b;
}
ORN_D uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
ORN_D uint64_t fadd2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// float(byte I of w), float(byte I+1 of w), each minus `bias` (given as the packed pair of
// -(2^23 + bias)): exact
template <int I>
ORN_D uint64_t byte2_f(uint32_t w, uint64_t neg_magic) {
  const float f0 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + I));
  const float f1 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + I + 1));
  return fadd2(pk2(f0, f1), neg_magic);
}

ORN_D float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
ORN_D float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// 8 bf16 -> 8 floats
ORN_D void widen8(const uint4& v, float* f) {
  f[0] = bf_lo(v.x); f[1] = bf_hi(v.x);
  f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
  f[4] = bf_lo(v.z); f[5] = bf_hi(v.z);
  f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
}

// kernels/q4k.metal:43-56 (get_scale_min_k4) on the 12 scale bytes held as
// three words (bytes 0-3, 4-7, 8-11).  Branch-free: neighbouring lanes ask for
// different sub-blocks, so a branch on j would run both sides one after the other.
ORN_D void q4k_scale_min(int j, uint32_t s0, uint32_t s1, uint32_t s2, float* sc, float* mn) {
  const int sh = 8 * (j & 3);
  const uint32_t a = (s0 >> sh) & 0xff;  // q[j & 3]
  const uint32_t b = (s1 >> sh) & 0xff;  // q[(j & 3) + 4]
  const uint32_t c = (s2 >> sh) & 0xff;  // q[(j & 3) + 8]
  const bool low = j < 4;
  const uint32_t scv = low ? (a & 63) : ((c & 0xF) | ((a >> 6) << 4));
  const uint32_t mnv = low ? (b & 63) : ((c >> 4) | ((b >> 6) << 4));
  *sc = (float)scv;
  *mn = (float)mnv;
}
