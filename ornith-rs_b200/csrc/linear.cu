// Dequant mat-vec kernels for the four weight formats of the decode path
// (Q4_K, Q6_K, 8-bit affine group 64, bf16), their routed (expert-gathered)
// forms, block dequantisation and the embedding gather.
//
// Replaces kernels/q4k.metal (q4k_qmv, q4k_qmv_m*, q4k_gather_qmv,
// q4k_dequantize), kernels/q6k.metal, the 8-bit affine_qmv_fast of
// kernels/mlx/.../quantized.h:756-822 and the bf16 gemv / gemv_gather of
// kernels/mlx/.../gemv.h, as dispatched by src/ops/kquant.rs:539-595,741-770,
// src/ops/quantized.rs:249-333 and src/ops/matmul.rs:334-437,649-711.
//
// Shape of every kernel here: one warp owns R output rows.  A row of K weights
// is cut into units (Q4_K: 16 bytes = 32 weights, Q6_K: 3 x 4 bytes = 16
// weights, A8: 16 bytes = 16 weights, BF16: 16 bytes = 8 weights); unit u
// belongs to lane u mod 32, so consecutive lanes read consecutive 16-byte
// pieces of the row (fully coalesced 128-bit loads).  Dequantisation happens in
// registers; a lane folds its units in ascending order into one float per
// (row, activation row), the products of a unit in two fma chains (even and odd
// elements: the two halves of a packed fma.rn.f32x2 in the fused kernels);
// lanes are folded by the xor-16..1 shuffle butterfly.
// The M activation rows of a verify window share each weight load and each get
// exactly the arithmetic a single row gets, so a row's bits do not depend on M
// (the property src/ops/invariant.rs:78-116 asks for).
//
// The kernels are HBM-bound (at most ~8 flop per weight byte), so no tensor
// cores: the work per weight is one byte-permute, one add and M fmas.
#include <cuda_fp16.h>

#include "orn_internal.h"
#include "orn_quant.cuh"

namespace {

constexpr int kWarpsPerBlock = 4;

// ---------------------------------------------------------------------------
// per-format unit: activation registers + weight registers + fold
// ---------------------------------------------------------------------------
template <int KIND>
struct Fmt;

// activation loads: from global memory through the read-only path, or from shared memory
template <bool SH> ORN_D uint4 ldx128(const void* p) {
  if constexpr (SH) return *reinterpret_cast<const uint4*>(p);
  else return ldg128(p);
}
template <bool SH> ORN_D uint2 ldx64(const void* p) {
  if constexpr (SH) return *reinterpret_cast<const uint2*>(p);
  else return __ldg(reinterpret_cast<const uint2*>(p));
}

template <>
struct Fmt<ORN_Q4K> {
  static constexpr int kWeightsPerUnit = 32;
  struct X { float lo[16], hi[16], slo, shi; };
  struct W { uint4 q; uint4 meta; };
  ORN_D static void load_x(const bf16_t* x, int u, X& r) { load_x_t<false>(x, u, r); }
  template <bool SH>
  ORN_D static void load_x_t(const bf16_t* x, int u, X& r) {
    int blk = u >> 3, j = u & 7, g = j >> 1, h = j & 1;
    const bf16_t* p = x + blk * 256 + 64 * g + 16 * h;
    uint4 a = ldx128<SH>(p), b = ldx128<SH>(p + 8), c = ldx128<SH>(p + 32), d = ldx128<SH>(p + 40);
    widen8(a, r.lo); widen8(b, r.lo + 8); widen8(c, r.hi); widen8(d, r.hi + 8);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) { s0 = s0 + r.lo[i]; s1 = s1 + r.hi[i]; }
    r.slo = s0; r.shi = s1;
  }
  ORN_D static void load_w(const LinDev& L, int64_t row, int u, W& w) {
    int blk = u >> 3, j = u & 7;
    w.q = ldg128_stream(L.w + row * L.rec + blk * 128 + 16 * j);
    w.meta = ldg128(L.s + row * L.rec + blk * 16);
  }
  ORN_D static float fold(const W& w, const X& x, int u, float acc) {
    int g = (u & 7) >> 1;
    const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
    // two chains per sum (even / odd elements), added at the end
    float le = 0.f, lod = 0.f, he = 0.f, hod = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t l4 = qw[k] & 0x0F0F0F0Fu, h4 = (qw[k] >> 4) & 0x0F0F0F0Fu;
      le = fmaf(x.lo[4 * k + 0], byte_f<0>(l4), le);
      lod = fmaf(x.lo[4 * k + 1], byte_f<1>(l4), lod);
      le = fmaf(x.lo[4 * k + 2], byte_f<2>(l4), le);
      lod = fmaf(x.lo[4 * k + 3], byte_f<3>(l4), lod);
      he = fmaf(x.hi[4 * k + 0], byte_f<0>(h4), he);
      hod = fmaf(x.hi[4 * k + 1], byte_f<1>(h4), hod);
      he = fmaf(x.hi[4 * k + 2], byte_f<2>(h4), he);
      hod = fmaf(x.hi[4 * k + 3], byte_f<3>(h4), hod);
    }
    const float lo = le + lod, hi = he + hod;
    float d = h2f((uint16_t)(w.meta.x & 0xffff)), dmin = h2f((uint16_t)(w.meta.x >> 16));
    float s1, m1, s2, m2;
    q4k_scale_min(2 * g, w.meta.y, w.meta.z, w.meta.w, &s1, &m1);
    q4k_scale_min(2 * g + 1, w.meta.y, w.meta.z, w.meta.w, &s2, &m2);
    float t = s1 * lo;
    t = fmaf(s2, hi, t);
    float mt = m1 * x.slo;
    mt = fmaf(m2, x.shi, mt);
    acc = fmaf(d, t, acc);
    acc = fmaf(-dmin, mt, acc);
    return acc;
  }
};

template <>
struct Fmt<ORN_Q6K> {
  static constexpr int kWeightsPerUnit = 16;
  struct X { float v[4][4]; };  // [quadrant][i]
  struct W { uint32_t qa, qb, qh; uint32_t sc4; float d; };
  ORN_D static void load_x(const bf16_t* x, int u, X& r) { load_x_t<false>(x, u, r); }
  template <bool SH>
  ORN_D static void load_x_t(const bf16_t* x, int u, X& r) {
    int blk = u >> 4, j = u & 15, half = j >> 3, l0 = 4 * (j & 7);
    const bf16_t* p = x + blk * 256 + 128 * half + l0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint2 v = ldx64<SH>(p + 32 * c);
      r.v[c][0] = bf_lo(v.x); r.v[c][1] = bf_hi(v.x);
      r.v[c][2] = bf_lo(v.y); r.v[c][3] = bf_hi(v.y);
    }
  }
  ORN_D static void load_w(const LinDev& L, int64_t row, int u, W& w) {
    int blk = u >> 4, j = u & 15, half = j >> 3, l0 = 4 * (j & 7);
    const uint8_t* base = L.w + row * L.rec + blk * 192;
    w.qa = ldg32_stream(base + 64 * half + l0);
    w.qb = ldg32_stream(base + 64 * half + 32 + l0);
    w.qh = ldg32_stream(base + 128 + 32 * half + l0);
    // scales sc[8*half + is + {0,2,4,6}], is = l0/16: read the 8 bytes of this
    // half as two words and pick bytes is, is+2 | is+4, is+6
    const uint8_t* sp = L.s + row * L.rec + blk * 16 + 8 * half;
    uint2 s8 = __ldg(reinterpret_cast<const uint2*>(sp));
    int is = l0 >> 4;
    uint32_t lo = s8.x >> (8 * is), hi = s8.y >> (8 * is);
    w.sc4 = (lo & 0xff) | (((lo >> 16) & 0xff) << 8) | ((hi & 0xff) << 16) |
            (((hi >> 16) & 0xff) << 24);
    w.d = h2f(__ldg(reinterpret_cast<const uint16_t*>(L.b + row * L.rec) + blk));
  }
  ORN_D static float fold(const W& w, const X& x, int, float acc) {
    uint32_t q1 = (w.qa & 0x0F0F0F0Fu) | ((w.qh & 0x03030303u) << 4);
    uint32_t q2 = (w.qb & 0x0F0F0F0Fu) | ((w.qh & 0x0C0C0C0Cu) << 2);
    uint32_t q3 = ((w.qa >> 4) & 0x0F0F0F0Fu) | (w.qh & 0x30303030u);
    uint32_t q4 = ((w.qb >> 4) & 0x0F0F0F0Fu) | ((w.qh & 0xC0C0C0C0u) >> 2);
    // two chains per quadrant sum (even / odd elements), added at the end
    float e0 = fmaf(x.v[0][0], byte_m32_f<0>(q1), 0.f), o0 = fmaf(x.v[0][1], byte_m32_f<1>(q1), 0.f);
    e0 = fmaf(x.v[0][2], byte_m32_f<2>(q1), e0); o0 = fmaf(x.v[0][3], byte_m32_f<3>(q1), o0);
    float e1 = fmaf(x.v[1][0], byte_m32_f<0>(q2), 0.f), o1 = fmaf(x.v[1][1], byte_m32_f<1>(q2), 0.f);
    e1 = fmaf(x.v[1][2], byte_m32_f<2>(q2), e1); o1 = fmaf(x.v[1][3], byte_m32_f<3>(q2), o1);
    float e2 = fmaf(x.v[2][0], byte_m32_f<0>(q3), 0.f), o2 = fmaf(x.v[2][1], byte_m32_f<1>(q3), 0.f);
    e2 = fmaf(x.v[2][2], byte_m32_f<2>(q3), e2); o2 = fmaf(x.v[2][3], byte_m32_f<3>(q3), o2);
    float e3 = fmaf(x.v[3][0], byte_m32_f<0>(q4), 0.f), o3 = fmaf(x.v[3][1], byte_m32_f<1>(q4), 0.f);
    e3 = fmaf(x.v[3][2], byte_m32_f<2>(q4), e3); o3 = fmaf(x.v[3][3], byte_m32_f<3>(q4), o3);
    const float s0 = e0 + o0, s1 = e1 + o1, s2 = e2 + o2, s3 = e3 + o3;
    float c0 = (float)(int8_t)(w.sc4 & 0xff), c1 = (float)(int8_t)((w.sc4 >> 8) & 0xff);
    float c2 = (float)(int8_t)((w.sc4 >> 16) & 0xff), c3 = (float)(int8_t)(w.sc4 >> 24);
    float t = c0 * s0;
    t = fmaf(c1, s1, t);
    t = fmaf(c2, s2, t);
    t = fmaf(c3, s3, t);
    return fmaf(w.d, t, acc);
  }
};

template <>
struct Fmt<ORN_A8> {
  static constexpr int kWeightsPerUnit = 16;
  struct X { float v[16]; float sum; };
  struct W { uint4 q; uint32_t sb; };
  ORN_D static void load_x(const bf16_t* x, int u, X& r) { load_x_t<false>(x, u, r); }
  template <bool SH>
  ORN_D static void load_x_t(const bf16_t* x, int u, X& r) {
    const bf16_t* p = x + 16 * u;
    uint4 a = ldx128<SH>(p), b = ldx128<SH>(p + 8);
    widen8(a, r.v); widen8(b, r.v + 8);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) s = s + r.v[i];
    r.sum = s;
  }
  ORN_D static void load_w(const LinDev& L, int64_t row, int u, W& w) {
    w.q = ldg128_stream(L.w + row * L.rec + 16 * u);
    w.sb = __ldg(reinterpret_cast<const uint32_t*>(L.s + row * L.rec) + (u >> 2));
  }
  ORN_D static float fold(const W& w, const X& x, int, float acc) {
    const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
    float se = 0.f, so = 0.f;  // even / odd chains, added at the end
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      se = fmaf(x.v[4 * k + 0], byte_f<0>(qw[k]), se);
      so = fmaf(x.v[4 * k + 1], byte_f<1>(qw[k]), so);
      se = fmaf(x.v[4 * k + 2], byte_f<2>(qw[k]), se);
      so = fmaf(x.v[4 * k + 3], byte_f<3>(qw[k]), so);
    }
    const float s1 = se + so;
    acc = fmaf(bf_lo(w.sb), s1, acc);
    acc = fmaf(bf_hi(w.sb), x.sum, acc);
    return acc;
  }
};

// mlx affine 4-bit, group 32 (quantized.h:756-822 at bits = 4): a unit is one group, 16 code bytes;
// byte b holds weights 2b (low nibble) and 2b+1 (high nibble)
template <>
struct Fmt<ORN_A4> {
  static constexpr int kWeightsPerUnit = 32;
  struct X { float v[32]; float sum; };
  struct W { uint4 q; uint32_t sb; };
  ORN_D static void load_x(const bf16_t* x, int u, X& r) { load_x_t<false>(x, u, r); }
  template <bool SH>
  ORN_D static void load_x_t(const bf16_t* x, int u, X& r) {
    const bf16_t* p = x + 32 * u;
#pragma unroll
    for (int i = 0; i < 4; ++i) widen8(ldx128<SH>(p + 8 * i), r.v + 8 * i);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) s = s + r.v[i];
    r.sum = s;
  }
  ORN_D static void load_w(const LinDev& L, int64_t row, int u, W& w) {
    w.q = ldg128_stream(L.w + row * L.rec + 16 * u);
    w.sb = __ldg(reinterpret_cast<const uint32_t*>(L.s + row * L.rec) + u);
  }
  ORN_D static float fold(const W& w, const X& x, int, float acc) {
    const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
    float se = 0.f, so = 0.f;  // even (low nibbles) / odd (high nibbles) chains, added at the end
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t l4 = qw[k] & 0x0F0F0F0Fu, h4 = (qw[k] >> 4) & 0x0F0F0F0Fu;
      se = fmaf(x.v[8 * k + 0], byte_f<0>(l4), se);
      so = fmaf(x.v[8 * k + 1], byte_f<0>(h4), so);
      se = fmaf(x.v[8 * k + 2], byte_f<1>(l4), se);
      so = fmaf(x.v[8 * k + 3], byte_f<1>(h4), so);
      se = fmaf(x.v[8 * k + 4], byte_f<2>(l4), se);
      so = fmaf(x.v[8 * k + 5], byte_f<2>(h4), so);
      se = fmaf(x.v[8 * k + 6], byte_f<3>(l4), se);
      so = fmaf(x.v[8 * k + 7], byte_f<3>(h4), so);
    }
    const float s1 = se + so;
    acc = fmaf(bf_lo(w.sb), s1, acc);
    acc = fmaf(bf_hi(w.sb), x.sum, acc);
    return acc;
  }
};

template <>
struct Fmt<ORN_BF16> {
  static constexpr int kWeightsPerUnit = 8;
  struct X { float v[8]; };
  struct W { uint4 q; };
  ORN_D static void load_x(const bf16_t* x, int u, X& r) { load_x_t<false>(x, u, r); }
  template <bool SH>
  ORN_D static void load_x_t(const bf16_t* x, int u, X& r) { widen8(ldx128<SH>(x + 8 * u), r.v); }
  ORN_D static void load_w(const LinDev& L, int64_t row, int u, W& w) {
    w.q = ldg128_stream(L.w + row * L.rec + 16 * u);
  }
  ORN_D static float fold(const W& w, const X& x, int, float acc) {
    float f[8];
    widen8(w.q, f);
    float se = 0.f, so = 0.f;  // the unit's even / odd chains; their sum joins the lane's total
#pragma unroll
    for (int i = 0; i < 8; i += 2) { se = fmaf(x.v[i], f[i], se); so = fmaf(x.v[i + 1], f[i + 1], so); }
    return acc + (se + so);
  }
};

// ---------------------------------------------------------------------------
// the mat-vec kernel: dense (blockIdx.y == 0, M rows of x share the weights)
// and routed (blockIdx.y = routed row, M == 1)
// ---------------------------------------------------------------------------
template <int KIND, int M, int R, int SU>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
gemv_kernel(LinDev L, const bf16_t* __restrict__ x, void* __restrict__ y, int out_f32,
            const uint32_t* __restrict__ lhs, const uint32_t* __restrict__ rhs) {
  using F = Fmt<KIND>;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row0 = (blockIdx.x * kWarpsPerBlock + warp) * R;
  if (row0 >= L.O) return;
  int64_t rowbase = row0;
  int64_t ybase = 0;
  if (rhs != nullptr) {
    const int r = blockIdx.y;
    rowbase += (int64_t)rhs[r] * L.O;
    x += (int64_t)lhs[r] * L.K;
    ybase = (int64_t)r * L.O;
  }
  const int units = L.K / F::kWeightsPerUnit;
  float acc[R][M];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.f;

  for (int u0 = lane; u0 < units; u0 += 32 * SU) {
    typename F::W w[SU][R];
    // all weight loads of this batch first, so that SU*R 16-byte requests per
    // lane are in flight before any of them is consumed
#pragma unroll
    for (int s = 0; s < SU; ++s) {
      const int u = u0 + 32 * s;
      if (u < units) {
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (row0 + r < L.O) F::load_w(L, rowbase + r, u, w[s][r]);
      }
    }
#pragma unroll
    for (int s = 0; s < SU; ++s) {
      const int u = u0 + 32 * s;
      if (u < units) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          typename F::X xr;
          F::load_x(x + (int64_t)m * L.K, u, xr);
#pragma unroll
          for (int r = 0; r < R; ++r)
            if (row0 + r < L.O) acc[r][m] = F::fold(w[s][r], xr, u, acc[r][m]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = warp_sum(acc[r][m]);
      if (lane == 0 && row0 + r < L.O) {
        int64_t idx = ybase + (int64_t)m * L.O + row0 + r;
        if (out_f32) reinterpret_cast<float*>(y)[idx] = v;
        else reinterpret_cast<bf16_t*>(y)[idx] = f2bf(v);
      }
    }
}

template <int KIND, int M, int R, int SU>
int launch_gemv(orn_ctx* ctx, cudaStream_t st, const orn_linear* L, const bf16_t* x, void* y,
                int out_f32, const uint32_t* lhs, const uint32_t* rhs, int rows) {
  const int warps = (L->O + R - 1) / R;
  dim3 grid((warps + kWarpsPerBlock - 1) / kWarpsPerBlock, rows > 0 ? rows : 1);
  gemv_kernel<KIND, M, R, SU><<<grid, kWarpsPerBlock * 32, 0, st>>>(lin_dev(L), x, y, out_f32,
                                                                     lhs, rhs);
  return orn_launch_check(ctx, "gemv_kernel");
}

// Rows per warp and step batch: enough warps to cover every SM several times
// for small matrices, more bytes in flight per lane for large ones.
template <int KIND, int M>
int dispatch_gemv(orn_ctx* ctx, cudaStream_t st, const orn_linear* L, const bf16_t* x, void* y,
                  int out_f32, const uint32_t* lhs, const uint32_t* rhs, int rows) {
  const int units = L->K / Fmt<KIND>::kWeightsPerUnit;
  const int steps = (units + 31) / 32;
  const int64_t total_rows = (int64_t)L->O * (rows > 0 ? rows : 1);
  const bool big = total_rows >= 16384;
  if (steps >= 4) {
    if (big) return launch_gemv<KIND, M, 2, 4>(ctx, st, L, x, y, out_f32, lhs, rhs, rows);
    return launch_gemv<KIND, M, 1, 4>(ctx, st, L, x, y, out_f32, lhs, rhs, rows);
  }
  if (steps >= 2) {
    if (big) return launch_gemv<KIND, M, 4, 2>(ctx, st, L, x, y, out_f32, lhs, rhs, rows);
    return launch_gemv<KIND, M, 2, 2>(ctx, st, L, x, y, out_f32, lhs, rhs, rows);
  }
  if (big) return launch_gemv<KIND, M, 4, 1>(ctx, st, L, x, y, out_f32, lhs, rhs, rows);
  return launch_gemv<KIND, M, 2, 1>(ctx, st, L, x, y, out_f32, lhs, rhs, rows);
}

template <int KIND>
int dispatch_m(orn_ctx* ctx, cudaStream_t st, const orn_linear* L, const bf16_t* x, int M, void* y,
               int out_f32) {
  switch (M) {
    case 1: return dispatch_gemv<KIND, 1>(ctx, st, L, x, y, out_f32, nullptr, nullptr, 0);
    case 2: return dispatch_gemv<KIND, 2>(ctx, st, L, x, y, out_f32, nullptr, nullptr, 0);
    case 3: return dispatch_gemv<KIND, 3>(ctx, st, L, x, y, out_f32, nullptr, nullptr, 0);
    default: return dispatch_gemv<KIND, 4>(ctx, st, L, x, y, out_f32, nullptr, nullptr, 0);
  }
}

}  // namespace

int k_gemv(orn_ctx* ctx, cudaStream_t st, const orn_linear* L, const bf16_t* x, int M, void* y,
           int out_f32) {
  // more than four rows: groups of four, each group re-reading the weights
  // (the decode path never has more; prefill chunks do)
  for (int m0 = 0; m0 < M; m0 += 4) {
    int mm = M - m0 < 4 ? M - m0 : 4;
    const bf16_t* xs = x + (int64_t)m0 * L->K;
    void* ys = out_f32 ? (void*)((float*)y + (int64_t)m0 * L->O)
                       : (void*)((bf16_t*)y + (int64_t)m0 * L->O);
    int rc;
    switch (L->kind) {
      case ORN_Q4K: rc = dispatch_m<ORN_Q4K>(ctx, st, L, xs, mm, ys, out_f32); break;
      case ORN_Q6K: rc = dispatch_m<ORN_Q6K>(ctx, st, L, xs, mm, ys, out_f32); break;
      case ORN_A8: rc = dispatch_m<ORN_A8>(ctx, st, L, xs, mm, ys, out_f32); break;
      case ORN_A4: rc = dispatch_m<ORN_A4>(ctx, st, L, xs, mm, ys, out_f32); break;
      default: rc = dispatch_m<ORN_BF16>(ctx, st, L, xs, mm, ys, out_f32); break;
    }
    if (rc != ORN_OK) return rc;
  }
  return ORN_OK;
}

int k_gather_gemv(orn_ctx* ctx, cudaStream_t st, const orn_linear* L, const bf16_t* x,
                  const uint32_t* lhs, const uint32_t* rhs, int rows, bf16_t* y) {
  if (rows <= 0) return ORN_OK;
  switch (L->kind) {
    case ORN_Q4K: return dispatch_gemv<ORN_Q4K, 1>(ctx, st, L, x, y, 0, lhs, rhs, rows);
    case ORN_Q6K: return dispatch_gemv<ORN_Q6K, 1>(ctx, st, L, x, y, 0, lhs, rhs, rows);
    case ORN_A8: return dispatch_gemv<ORN_A8, 1>(ctx, st, L, x, y, 0, lhs, rhs, rows);
    case ORN_A4: return dispatch_gemv<ORN_A4, 1>(ctx, st, L, x, y, 0, lhs, rhs, rows);
    default: return dispatch_gemv<ORN_BF16, 1>(ctx, st, L, x, y, 0, lhs, rhs, rows);
  }
}

// ---------------------------------------------------------------------------
// grouped mat-vec: rows sorted by expert (the sorted path of switch_glu_rows,
// src/ops/moe.rs:283-314, after counting_sort, :463-508).  Expert e owns the
// sorted rows seg[e] .. seg[e+1]-1; a warp takes R output rows of one expert and
// walks that expert's activation rows in groups of four, so the expert's
// records come from HBM once (later groups find them in L1/L2) and every row is
// computed with exactly the one-row arithmetic of gemv_kernel: the result bits
// do not depend on how the rows are grouped.
// ---------------------------------------------------------------------------
namespace {
constexpr int kGroupThreads = 256;  // 8 warps
constexpr int kGroupRows = 128;     // output rows of one expert a block owns (32 for one small dense matrix over many rows)
constexpr int kGroupBatch = 4;      // activation rows staged per pass (the mat-vec's row limit)

// One warp, R output rows starting at row0 of expert matrix rows `rowbase`, M staged activation
// rows in shared memory: the arithmetic of gemv_kernel (units in ascending order per lane, the
// xor butterfly), weights requested SU units ahead.
template <int KIND, int M, int R, int SU>
ORN_D void grouped_rows(const LinDev& L, int64_t rowbase, int row0, int row_end, const bf16_t* xsm, bf16_t* y,
                        const uint32_t* row_map, int first, int lane) {
  using F = Fmt<KIND>;
  const int units = L.K / F::kWeightsPerUnit;
  float acc[R][M];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
  for (int u0 = lane; u0 < units; u0 += 32 * SU) {
    typename F::W w[SU][R];
#pragma unroll
    for (int su = 0; su < SU; ++su) {
      const int u = u0 + 32 * su;
      if (u < units) {
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (row0 + r < row_end) F::load_w(L, rowbase + r, u, w[su][r]);
      }
    }
#pragma unroll
    for (int su = 0; su < SU; ++su) {
      const int u = u0 + 32 * su;
      if (u < units) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          typename F::X xr;
          F::template load_x_t<true>(xsm + (size_t)m * L.K, u, xr);
#pragma unroll
          for (int r = 0; r < R; ++r)
            if (row0 + r < row_end) acc[r][m] = F::fold(w[su][r], xr, u, acc[r][m]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float v = warp_sum(acc[r][m]);
      if (lane == 0 && row0 + r < row_end) {
        const int64_t orow = row_map != nullptr ? (int64_t)row_map[first + m] : (int64_t)(first + m);
        y[orow * L.O + row0 + r] = f2bf(v);
      }
    }
}

// grid (ceil(O / kGroupRows), E): a block owns kGroupRows output rows of one expert; it stages up
// to four of the expert's activation rows in shared memory per pass and streams its weight rows
// once per pass (the first pass from HBM, later passes from L2)
template <int KIND, int R, int SU>
__global__ void __launch_bounds__(kGroupThreads)
grouped_gemv_kernel(LinDev L, const bf16_t* __restrict__ xs, const int* __restrict__ seg, bf16_t* __restrict__ y,
                    const uint32_t* __restrict__ row_map, int rows_per_block, LinDev L2, bf16_t* __restrict__ y2, int blocks1) {
  extern __shared__ __align__(16) uint8_t gsm[];
  bf16_t* xsm = reinterpret_cast<bf16_t*>(gsm);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = blockIdx.y;
  const int first = seg[e], n = seg[e + 1] - first;
  if (n <= 0) return;
  // a second matrix over the same rows (same format and row length) rides in the blocks behind the first one's
  int bx = blockIdx.x;
  if (bx >= blocks1) { L = L2; y = y2; bx -= blocks1; }
  const int chunk0 = bx * rows_per_block;
  const int row_end = min(L.O, chunk0 + rows_per_block);
  // the expert's rows in passes of four; blockIdx.z takes every gridDim.z-th pass
  for (int m0 = kGroupBatch * blockIdx.z; m0 < n; m0 += kGroupBatch * gridDim.z) {
    const int M = min(kGroupBatch, n - m0);
    __syncthreads();  // the previous pass has read its rows
    const uint4* src = reinterpret_cast<const uint4*>(xs + (size_t)(first + m0) * L.K);
    for (int i = threadIdx.x; i < M * L.K / 8; i += blockDim.x) reinterpret_cast<uint4*>(xsm)[i] = __ldg(src + i);
    __syncthreads();
    for (int row0 = chunk0 + warp * R; row0 < row_end; row0 += (kGroupThreads / 32) * R) {
      const int64_t rowbase = (int64_t)e * L.O + row0;
      switch (M) {
        case 1: grouped_rows<KIND, 1, R, SU>(L, rowbase, row0, row_end, xsm, y, row_map, first + m0, lane); break;
        case 2: grouped_rows<KIND, 2, R, SU>(L, rowbase, row0, row_end, xsm, y, row_map, first + m0, lane); break;
        case 3: grouped_rows<KIND, 3, R, SU>(L, rowbase, row0, row_end, xsm, y, row_map, first + m0, lane); break;
        default: grouped_rows<KIND, 4, R, SU>(L, rowbase, row0, row_end, xsm, y, row_map, first + m0, lane); break;
      }
    }
  }
}

template <int KIND>
int launch_grouped(orn_ctx* ctx, cudaStream_t st, const orn_linear* L, const bf16_t* xs, const int* seg, bf16_t* y,
                   const uint32_t* row_map, int max_rows, const orn_linear* L2 = nullptr, bf16_t* y2 = nullptr) {
  const size_t smem = (size_t)kGroupBatch * L->K * sizeof(bf16_t);
  if (smem > 48 * 1024) ORN_FAIL(ctx, ORN_ERR_ARG, "grouped gemv: rows longer than 6144 weights");
  // passes of four rows spread over blockIdx.z: all of them for one dense matrix over many rows,
  // a few for routed experts (an expert with more rows than that loops)
  int z = L->E == 1 ? (max_rows + kGroupBatch - 1) / kGroupBatch : 4;
  if (z < 1) z = 1;
  if (z > 64) z = 64;
  // one small dense matrix (a router) over many rows: narrower blocks so that the launch fills the part
  const int rpb = (L->E == 1 && L->O <= 1024) ? 32 : kGroupRows;
  const int blocks1 = (L->O + rpb - 1) / rpb, blocks2 = L2 ? (L2->O + rpb - 1) / rpb : 0;
  dim3 grid(blocks1 + blocks2, L->E, z);
  const int units = L->K / Fmt<KIND>::kWeightsPerUnit;
  const LinDev d1 = lin_dev(L), d2 = L2 ? lin_dev(L2) : d1;
  if (units > 32) grouped_gemv_kernel<KIND, 2, 2><<<grid, kGroupThreads, smem, st>>>(d1, xs, seg, y, row_map, rpb, d2, y2, blocks1);
  else grouped_gemv_kernel<KIND, 4, 1><<<grid, kGroupThreads, smem, st>>>(d1, xs, seg, y, row_map, rpb, d2, y2, blocks1);
  return orn_launch_check(ctx, "grouped_gemv");
}
}  // namespace

// y[row_map ? row_map[p] : p] = W[expert of sorted row p] . xs[p] for every sorted row p
int k_grouped_gemv(orn_ctx* ctx, cudaStream_t st, const orn_linear* L, const bf16_t* xs, const int* seg, bf16_t* y,
                   const uint32_t* row_map, int max_rows) {
  if (L->E > 65535) ORN_FAIL(ctx, ORN_ERR_ARG, "grouped gemv: more than 65535 experts");
  switch (L->kind) {
    case ORN_Q4K: return launch_grouped<ORN_Q4K>(ctx, st, L, xs, seg, y, row_map, max_rows);
    case ORN_Q6K: return launch_grouped<ORN_Q6K>(ctx, st, L, xs, seg, y, row_map, max_rows);
    case ORN_A8: return launch_grouped<ORN_A8>(ctx, st, L, xs, seg, y, row_map, max_rows);
    case ORN_A4: return launch_grouped<ORN_A4>(ctx, st, L, xs, seg, y, row_map, max_rows);
    default: return launch_grouped<ORN_BF16>(ctx, st, L, xs, seg, y, row_map, max_rows);
  }
}

// two dense matrices of one format and row length over the same rows in one launch (the router and the
// shared expert's gate): each output has the bits of its own launch
int k_grouped_gemv2(orn_ctx* ctx, cudaStream_t st, const orn_linear* L1, bf16_t* y1, const orn_linear* L2, bf16_t* y2,
                    const bf16_t* xs, const int* seg, int max_rows) {
  if (L1->kind != L2->kind || L1->K != L2->K || L1->E != 1 || L2->E != 1) {
    int rc = k_grouped_gemv(ctx, st, L1, xs, seg, y1, nullptr, max_rows);
    return rc != ORN_OK ? rc : k_grouped_gemv(ctx, st, L2, xs, seg, y2, nullptr, max_rows);
  }
  switch (L1->kind) {
    case ORN_Q4K: return launch_grouped<ORN_Q4K>(ctx, st, L1, xs, seg, y1, nullptr, max_rows, L2, y2);
    case ORN_Q6K: return launch_grouped<ORN_Q6K>(ctx, st, L1, xs, seg, y1, nullptr, max_rows, L2, y2);
    case ORN_A8: return launch_grouped<ORN_A8>(ctx, st, L1, xs, seg, y1, nullptr, max_rows, L2, y2);
    case ORN_A4: return launch_grouped<ORN_A4>(ctx, st, L1, xs, seg, y1, nullptr, max_rows, L2, y2);
    default: return launch_grouped<ORN_BF16>(ctx, st, L1, xs, seg, y1, nullptr, max_rows, L2, y2);
  }
}

// ---------------------------------------------------------------------------
// block dequantisation (test/oracle surface of the reference:
// kernels/q4k.metal:64-96, kernels/q6k.metal:47-77)
// ---------------------------------------------------------------------------
namespace {
__global__ void q4k_dequant_kernel(LinDev L, int e, float* out) {
  int64_t nblocks = (int64_t)L.O * (L.K >> 8);
  int64_t ib = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (ib >= nblocks) return;
  const int nb = L.K >> 8;
  const int64_t row = (int64_t)e * L.O + ib / nb;
  const int blk = (int)(ib % nb);
  const uint8_t* q = L.w + row * L.rec + blk * 128;
  uint4 meta = ldg128(L.s + row * L.rec + blk * 16);
  float d = h2f((uint16_t)(meta.x & 0xffff)), dmin = h2f((uint16_t)(meta.x >> 16));
  float* y = out + ib * 256;
  for (int g = 0; g < 4; ++g) {
    float s1, m1, s2, m2;
    q4k_scale_min(2 * g, meta.y, meta.z, meta.w, &s1, &m1);
    q4k_scale_min(2 * g + 1, meta.y, meta.z, meta.w, &s2, &m2);
    float d1 = d * s1, o1 = dmin * m1, d2 = d * s2, o2 = dmin * m2;
    for (int l = 0; l < 32; ++l) {
      uint8_t b = q[32 * g + l];
      y[64 * g + l] = d1 * (float)(b & 0xF) - o1;
      y[64 * g + 32 + l] = d2 * (float)(b >> 4) - o2;
    }
  }
}

__global__ void q6k_dequant_kernel(LinDev L, int e, float* out) {
  int64_t nblocks = (int64_t)L.O * (L.K >> 8);
  int64_t ib = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (ib >= nblocks) return;
  const int nb = L.K >> 8;
  const int64_t row = (int64_t)e * L.O + ib / nb;
  const int blk = (int)(ib % nb);
  const uint8_t* ql = L.w + row * L.rec + blk * 192;
  const uint8_t* qh = ql + 128;
  const int8_t* sc = reinterpret_cast<const int8_t*>(L.s + row * L.rec) + blk * 16;
  float d = h2f(reinterpret_cast<const uint16_t*>(L.b + row * L.rec)[blk]);
  float* y = out + ib * 256;
  for (int n = 0; n < 2; ++n) {
    for (int l = 0; l < 32; ++l) {
      int is = l / 16;
      int q1 = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
      int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
      int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      y[l + 0] = d * (float)sc[is + 0] * (float)q1;
      y[l + 32] = d * (float)sc[is + 2] * (float)q2;
      y[l + 64] = d * (float)sc[is + 4] * (float)q3;
      y[l + 96] = d * (float)sc[is + 6] * (float)q4;
    }
    y += 128; ql += 64; qh += 32; sc += 8;
  }
}

// src/ops/embedding.rs:18-47: value = bf(f32(scale)*q + f32(bias)), one fma
__global__ void embedding_a8_kernel(LinDev L, const uint32_t* ids, bf16_t* out) {
  int t = blockIdx.y;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= L.K) return;
  int64_t row = ids[t];
  if (row >= L.O) row = L.O - 1;  // an id outside the table must not fault
  uint32_t sb = reinterpret_cast<const uint32_t*>(L.s + row * L.rec)[i >> 6];
  float q = (float)L.w[row * L.rec + i];
  out[(int64_t)t * L.K + i] = f2bf(fmaf(bf_lo(sb), q, bf_hi(sb)));
}
}  // namespace

int k_kq_dequantize(orn_ctx* ctx, cudaStream_t st, const orn_linear* L, int e, float* out) {
  int64_t nblocks = (int64_t)L->O * (L->K >> 8);
  int grid = (int)((nblocks + 127) / 128);
  if (L->kind == ORN_Q4K) q4k_dequant_kernel<<<grid, 128, 0, st>>>(lin_dev(L), e, out);
  else if (L->kind == ORN_Q6K) q6k_dequant_kernel<<<grid, 128, 0, st>>>(lin_dev(L), e, out);
  else ORN_FAIL(ctx, ORN_ERR_ARG, "orn_kq_dequantize: not a k-quant matrix");
  return orn_launch_check(ctx, "kq_dequant");
}

int k_embedding(orn_ctx* ctx, cudaStream_t st, const orn_linear* L, const uint32_t* ids, int T,
                bf16_t* out) {
  if (L->kind != ORN_A8) ORN_FAIL(ctx, ORN_ERR_ARG, "orn_embedding: table must be affine-8");
  dim3 grid((L->K + 255) / 256, T);
  embedding_a8_kernel<<<grid, 256, 0, st>>>(lin_dev(L), ids, out);
  return orn_launch_check(ctx, "embedding");
}

// ---------------------------------------------------------------------------
// layout: artifact tensors <-> HBM layout
// ---------------------------------------------------------------------------
void linear_artifact_sizes(int kind, int E, int O, int K, size_t* w, size_t* s, size_t* b) {
  size_t rows = (size_t)E * O;
  switch (kind) {
    case ORN_Q4K: *w = rows * (K / 2); *s = rows * (K / 256) * 12; *b = rows * (K / 256) * 4; break;
    case ORN_Q6K: *w = rows * (K / 256) * 192; *s = rows * (K / 256) * 16; *b = rows * (K / 256) * 2; break;
    case ORN_A8: *w = rows * K; *s = rows * (K / 64) * 2; *b = rows * (K / 64) * 2; break;
    case ORN_A4: *w = rows * (K / 2); *s = rows * (K / 32) * 2; *b = rows * (K / 32) * 2; break;
    default: *w = rows * K * 2; *s = 0; *b = 0; break;
  }
}
namespace {
// stream `off` of every row record <- / -> a dense [rows][row_bytes] tensor (row_bytes even)
__global__ void rows_scatter_kernel(const uint8_t* dense, size_t row_bytes, uint8_t* recs, size_t rec, size_t off) {
  const size_t r = blockIdx.x;
  const uint16_t* s = reinterpret_cast<const uint16_t*>(dense + r * row_bytes);
  uint16_t* d = reinterpret_cast<uint16_t*>(recs + r * rec + off);
  for (size_t i = threadIdx.x; i < row_bytes / 2; i += blockDim.x) d[i] = s[i];
}
__global__ void rows_gather_kernel(const uint8_t* recs, size_t rec, size_t off, size_t row_bytes, uint8_t* dense) {
  const size_t r = blockIdx.x;
  const uint16_t* s = reinterpret_cast<const uint16_t*>(recs + r * rec + off);
  uint16_t* d = reinterpret_cast<uint16_t*>(dense + r * row_bytes);
  for (size_t i = threadIdx.x; i < row_bytes / 2; i += blockDim.x) d[i] = s[i];
}
// Q4_K: {dm[4], scales[12]} <-> one 16-byte header per block inside the record
__global__ void q4k_pack_meta(const uint8_t* scales, const uint8_t* dm, int64_t nblocks, int nb, uint8_t* s1, size_t rec) {
  int64_t ib = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (ib >= nblocks) return;
  uint8_t* meta = s1 + (ib / nb) * rec + (ib % nb) * 16;
  for (int i = 0; i < 4; ++i) meta[i] = dm[ib * 4 + i];
  for (int i = 0; i < 12; ++i) meta[4 + i] = scales[ib * 12 + i];
}
__global__ void q4k_unpack_meta(const uint8_t* s1, size_t rec, int64_t nblocks, int nb, uint8_t* scales, uint8_t* dm) {
  int64_t ib = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (ib >= nblocks) return;
  const uint8_t* meta = s1 + (ib / nb) * rec + (ib % nb) * 16;
  for (int i = 0; i < 4; ++i) dm[ib * 4 + i] = meta[i];
  for (int i = 0; i < 12; ++i) scales[ib * 12 + i] = meta[4 + i];
}
// A8: scales bf16 + biases bf16 <-> u32 {scale, bias} inside the record
__global__ void a8_pack_sb(const uint16_t* s, const uint16_t* b, int64_t n, int ng, uint8_t* s1, size_t rec) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) reinterpret_cast<uint32_t*>(s1 + (i / ng) * rec)[i % ng] = (uint32_t)s[i] | ((uint32_t)b[i] << 16);
}
__global__ void a8_unpack_sb(const uint8_t* s1, size_t rec, int64_t n, int ng, uint16_t* s, uint16_t* b) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) {
    const uint32_t v = reinterpret_cast<const uint32_t*>(s1 + (i / ng) * rec)[i % ng];
    s[i] = (uint16_t)(v & 0xffff);
    b[i] = (uint16_t)(v >> 16);
  }
}
__global__ void gather_records_kernel(const uint8_t* src, const uint32_t* ids, size_t rec, uint8_t* dst) {
  const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)ids[blockIdx.x] * rec);
  uint4* d = reinterpret_cast<uint4*>(dst + (size_t)blockIdx.x * rec);
  for (size_t i = threadIdx.x; i < rec / 16; i += blockDim.x) d[i] = s[i];
}
}  // namespace

// dw/ds/db: device copies of the artifact tensors -> row records
int k_linear_pack(orn_ctx* ctx, cudaStream_t st, orn_linear* L, const uint8_t* dw, const uint8_t* ds,
                  const uint8_t* db) {
  const RecGeom g = rec_geom(L->kind, L->K);
  const size_t rows = (size_t)L->E * L->O;
  rows_scatter_kernel<<<(unsigned)rows, 128, 0, st>>>(dw, g.b0, L->w, g.rec, 0);
  int rc = orn_launch_check(ctx, "rows_scatter");
  if (rc != ORN_OK) return rc;
  if (L->kind == ORN_Q4K) {
    const int nb = L->K / 256;
    const int64_t n = (int64_t)rows * nb;
    q4k_pack_meta<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ds, db, n, nb, L->s, g.rec);
    return orn_launch_check(ctx, "q4k_pack_meta");
  }
  if (L->kind == ORN_Q6K) {
    rows_scatter_kernel<<<(unsigned)rows, 64, 0, st>>>(ds, g.b1, L->w, g.rec, g.b0);
    rows_scatter_kernel<<<(unsigned)rows, 32, 0, st>>>(db, g.b2, L->w, g.rec, g.b0 + g.b1);
    return orn_launch_check(ctx, "rows_scatter");
  }
  if (L->kind == ORN_A8 || L->kind == ORN_A4) {
    const int ng = L->kind == ORN_A8 ? L->K / 64 : L->K / 32;
    const int64_t n = (int64_t)rows * ng;
    a8_pack_sb<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const uint16_t*)ds, (const uint16_t*)db, n, ng, L->s, g.rec);
    return orn_launch_check(ctx, "a8_pack_sb");
  }
  return ORN_OK;
}

int k_linear_unpack(orn_ctx* ctx, cudaStream_t st, const orn_linear* L, uint8_t* dw, uint8_t* ds, uint8_t* db) {
  const RecGeom g = rec_geom(L->kind, L->K);
  const size_t rows = (size_t)L->E * L->O;
  rows_gather_kernel<<<(unsigned)rows, 128, 0, st>>>(L->w, g.rec, 0, g.b0, dw);
  int rc = orn_launch_check(ctx, "rows_gather");
  if (rc != ORN_OK) return rc;
  if (L->kind == ORN_Q4K) {
    const int nb = L->K / 256;
    const int64_t n = (int64_t)rows * nb;
    q4k_unpack_meta<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(L->s, g.rec, n, nb, ds, db);
    return orn_launch_check(ctx, "q4k_unpack_meta");
  }
  if (L->kind == ORN_Q6K) {
    rows_gather_kernel<<<(unsigned)rows, 64, 0, st>>>(L->w, g.rec, g.b0, g.b1, ds);
    rows_gather_kernel<<<(unsigned)rows, 32, 0, st>>>(L->w, g.rec, g.b0 + g.b1, g.b2, db);
    return orn_launch_check(ctx, "rows_gather");
  }
  if (L->kind == ORN_A8 || L->kind == ORN_A4) {
    const int ng = L->kind == ORN_A8 ? L->K / 64 : L->K / 32;
    const int64_t n = (int64_t)rows * ng;
    a8_unpack_sb<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(L->s, g.rec, n, ng, (uint16_t*)ds, (uint16_t*)db);
    return orn_launch_check(ctx, "a8_unpack_sb");
  }
  return ORN_OK;
}

int k_linear_gather_rows(orn_ctx* ctx, cudaStream_t st, const orn_linear* L, const uint32_t* ids, int n,
                         orn_linear* out) {
  gather_records_kernel<<<n, 128, 0, st>>>(L->w, ids, L->rec, out->w);
  return orn_launch_check(ctx, "gather_rows");
}

// ---------------------------------------------------------------------------
// seeded synthetic weights: w ~ approx N(0, std) from a counter hash, then the
// plain round-to-nearest quantiser of each format (min/max per sub-block for
// Q4_K as in tools/q4k.py:122-161, abs-max for Q6_K, min/max per group of 64
// for affine-8 as in tools/aq.py:34-72).
// ---------------------------------------------------------------------------
namespace {
ORN_D uint64_t mix64(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}
// sum of four uniforms on (-1,1), scaled to unit variance (Irwin-Hall, n = 4)
ORN_D float approx_normal(uint64_t seed, uint64_t idx) {
  uint64_t h = mix64(seed ^ (idx * 0xd1342543de82ef95ull));
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t v = (uint32_t)(h >> (16 * i)) & 0xffff;
    s += ((float)v + 0.5f) * (1.0f / 32768.0f) - 1.0f;
  }
  return s * 0.8660254f;  // var of sum = 4/3
}
ORN_D uint16_t f2h_rn(float f) { return __half_as_ushort(__float2half_rn(f)); }

__global__ void random_bf16_kernel(bf16_t* p, size_t n, uint64_t seed, float mean, float std) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i < n) p[i] = f2bf(mean + std * approx_normal(seed, i));
}

__global__ void random_q4k_kernel(LinDev L, uint64_t seed, float std) {
  int64_t nblocks = (int64_t)L.E * L.O * (L.K >> 8);
  int64_t ib = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (ib >= nblocks) return;
  float scale[8], mn[8];
  float smax = 0.f, mmax = 0.f;
  for (int j = 0; j < 8; ++j) {
    float lo = 0.f, hi = -1e30f;
    for (int i = 0; i < 32; ++i) {
      float v = std * approx_normal(seed, ib * 256 + j * 32 + i);
      lo = fminf(lo, v); hi = fmaxf(hi, v);
    }
    scale[j] = (hi - lo) / 15.0f;
    mn[j] = -lo;
    smax = fmaxf(smax, scale[j]); mmax = fmaxf(mmax, mn[j]);
  }
  uint16_t dh = f2h_rn(smax / 63.0f), dmh = f2h_rn(mmax / 63.0f);
  float d = h2f(dh), dm = h2f(dmh);
  uint8_t sc[8], m[8];
  for (int j = 0; j < 8; ++j) {
    sc[j] = d > 0.f ? (uint8_t)fminf(63.f, fmaxf(0.f, rintf(scale[j] / d))) : 0;
    m[j] = dm > 0.f ? (uint8_t)fminf(63.f, fmaxf(0.f, rintf(mn[j] / dm))) : 0;
  }
  const int nbr = L.K >> 8;
  const int64_t rrow = ib / nbr;
  const int rblk = (int)(ib % nbr);
  uint8_t* meta = const_cast<uint8_t*>(L.s) + rrow * L.rec + rblk * 16;
  meta[0] = dh & 0xff; meta[1] = dh >> 8; meta[2] = dmh & 0xff; meta[3] = dmh >> 8;
  uint8_t* p = meta + 4;
  for (int i = 0; i < 12; ++i) p[i] = 0;
  for (int j = 0; j < 4; ++j) { p[j] = sc[j] & 63; p[j + 4] = m[j] & 63; }
  for (int j = 4; j < 8; ++j) {
    p[j + 4] = (sc[j] & 0xF) | ((m[j] & 0xF) << 4);
    p[j - 4] |= (sc[j] >> 4) << 6;
    p[j] |= (m[j] >> 4) << 6;
  }
  uint8_t* q = const_cast<uint8_t*>(L.w) + rrow * L.rec + rblk * 128;
  for (int g = 0; g < 4; ++g) {
    float ds0 = d * sc[2 * g], ms0 = dm * m[2 * g], ds1 = d * sc[2 * g + 1], ms1 = dm * m[2 * g + 1];
    for (int l = 0; l < 32; ++l) {
      float a = std * approx_normal(seed, ib * 256 + 64 * g + l);
      float b = std * approx_normal(seed, ib * 256 + 64 * g + 32 + l);
      int qa = ds0 > 0.f ? (int)fminf(15.f, fmaxf(0.f, rintf((a + ms0) / ds0))) : 0;
      int qb = ds1 > 0.f ? (int)fminf(15.f, fmaxf(0.f, rintf((b + ms1) / ds1))) : 0;
      q[32 * g + l] = (uint8_t)(qa | (qb << 4));
    }
  }
}

__global__ void random_q6k_kernel(LinDev L, uint64_t seed, float std) {
  int64_t nblocks = (int64_t)L.E * L.O * (L.K >> 8);
  int64_t ib = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (ib >= nblocks) return;
  // 16 sub-blocks of 16 weights; sub-block scale = absmax/31, super scale d = max|scale|/127
  float sub[16];
  float smax = 0.f;
  for (int j = 0; j < 16; ++j) {
    float am = 0.f;
    for (int i = 0; i < 16; ++i) am = fmaxf(am, fabsf(std * approx_normal(seed, ib * 256 + j * 16 + i)));
    sub[j] = am / 31.0f;
    smax = fmaxf(smax, sub[j]);
  }
  uint16_t dh = f2h_rn(smax / 127.0f);
  float d = h2f(dh);
  int8_t sc[16];
  for (int j = 0; j < 16; ++j)
    sc[j] = d > 0.f ? (int8_t)fminf(127.f, fmaxf(1.f, rintf(sub[j] / d))) : 0;
  const int nbr = L.K >> 8;
  const int64_t rrow = ib / nbr;
  const int rblk = (int)(ib % nbr);
  int8_t* sp = reinterpret_cast<int8_t*>(const_cast<uint8_t*>(L.s) + rrow * L.rec) + rblk * 16;
  for (int j = 0; j < 16; ++j) sp[j] = sc[j];
  reinterpret_cast<uint16_t*>(const_cast<uint8_t*>(L.b) + rrow * L.rec)[rblk] = dh;
  uint8_t* ql = const_cast<uint8_t*>(L.w) + rrow * L.rec + rblk * 192;
  uint8_t* qh = ql + 128;
  for (int i = 0; i < 128; ++i) ql[i] = 0;
  for (int i = 0; i < 64; ++i) qh[i] = 0;
  for (int n = 0; n < 2; ++n)
    for (int c = 0; c < 4; ++c)
      for (int l = 0; l < 32; ++l) {
        int widx = 128 * n + 32 * c + l;
        float v = std * approx_normal(seed, ib * 256 + widx);
        float ds = d * (float)sc[widx / 16];
        int q = ds > 0.f ? (int)fminf(31.f, fmaxf(-32.f, rintf(v / ds))) + 32 : 32;
        int lo4 = q & 0xF, hi2 = q >> 4;
        int qli = 64 * n + l + ((c & 1) ? 32 : 0);
        if (c < 2) ql[qli] |= (uint8_t)lo4; else ql[qli] |= (uint8_t)(lo4 << 4);
        qh[32 * n + l] |= (uint8_t)(hi2 << (2 * c));
      }
}

__global__ void random_a8_kernel(LinDev L, uint64_t seed, float std) {
  int64_t ngroups = (int64_t)L.E * L.O * (L.K >> 6);
  int64_t ig = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (ig >= ngroups) return;
  float lo = 1e30f, hi = -1e30f;
  for (int i = 0; i < 64; ++i) {
    float v = std * approx_normal(seed, ig * 64 + i);
    lo = fminf(lo, v); hi = fmaxf(hi, v);
  }
  float scale = fmaxf((hi - lo) / 255.0f, 1e-8f);
  bf16_t sb = f2bf(scale), bb = f2bf(lo);
  float s = bf2f(sb), b = bf2f(bb);
  const int ngr = L.K >> 6;
  const int64_t rrow = ig / ngr;
  const int rgrp = (int)(ig % ngr);
  reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(L.s) + rrow * L.rec)[rgrp] = (uint32_t)sb | ((uint32_t)bb << 16);
  uint8_t* q = const_cast<uint8_t*>(L.w) + rrow * L.rec + rgrp * 64;
  for (int i = 0; i < 64; ++i) {
    float v = std * approx_normal(seed, ig * 64 + i);
    q[i] = (uint8_t)fminf(255.f, fmaxf(0.f, rintf((v - b) / s)));
  }
}
__global__ void random_a4_kernel(LinDev L, uint64_t seed, float std) {
  int64_t ngroups = (int64_t)L.E * L.O * (L.K >> 5);
  int64_t ig = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (ig >= ngroups) return;
  float lo = 1e30f, hi = -1e30f;
  for (int i = 0; i < 32; ++i) {
    float v = std * approx_normal(seed, ig * 32 + i);
    lo = fminf(lo, v); hi = fmaxf(hi, v);
  }
  float scale = fmaxf((hi - lo) / 15.0f, 1e-8f);
  bf16_t sb = f2bf(scale), bb = f2bf(lo);
  float s = bf2f(sb), b = bf2f(bb);
  const int ngr = L.K >> 5;
  const int64_t rrow = ig / ngr;
  const int rgrp = (int)(ig % ngr);
  reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(L.s) + rrow * L.rec)[rgrp] = (uint32_t)sb | ((uint32_t)bb << 16);
  uint8_t* q = const_cast<uint8_t*>(L.w) + rrow * L.rec + rgrp * 16;
  for (int i = 0; i < 16; ++i) {
    float v0 = std * approx_normal(seed, ig * 32 + 2 * i), v1 = std * approx_normal(seed, ig * 32 + 2 * i + 1);
    int q0 = (int)fminf(15.f, fmaxf(0.f, rintf((v0 - b) / s))), q1 = (int)fminf(15.f, fmaxf(0.f, rintf((v1 - b) / s)));
    q[i] = (uint8_t)(q0 | (q1 << 4));
  }
}
}  // namespace

int k_fill_bf16(orn_ctx* ctx, cudaStream_t st, bf16_t* p, size_t n, uint64_t seed, float mean,
                float std) {
  random_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(p, n, seed, mean, std);
  return orn_launch_check(ctx, "random_bf16");
}

int k_linear_random(orn_ctx* ctx, cudaStream_t st, orn_linear* L, uint64_t seed, float std) {
  LinDev d = lin_dev(L);
  if (L->kind == ORN_Q4K) {
    int64_t nb = (int64_t)L->E * L->O * (L->K / 256);
    random_q4k_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(d, seed, std);
  } else if (L->kind == ORN_Q6K) {
    int64_t nb = (int64_t)L->E * L->O * (L->K / 256);
    random_q6k_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(d, seed, std);
  } else if (L->kind == ORN_A8) {
    int64_t ng = (int64_t)L->E * L->O * (L->K / 64);
    random_a8_kernel<<<(unsigned)((ng + 127) / 128), 128, 0, st>>>(d, seed, std);
  } else if (L->kind == ORN_A4) {
    int64_t ng = (int64_t)L->E * L->O * (L->K / 32);
    random_a4_kernel<<<(unsigned)((ng + 127) / 128), 128, 0, st>>>(d, seed, std);
  } else {
    return k_fill_bf16(ctx, st, (bf16_t*)L->w, (size_t)L->E * L->O * L->K, seed, 0.f, std);
  }
  return orn_launch_check(ctx, "linear_random");
}
