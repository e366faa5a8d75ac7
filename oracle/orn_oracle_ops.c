/* TEST INFRASTRUCTURE, NOT PRODUCT CODE.  See orn_oracle_math.h for the parity
 * status ("parity unpinned" beyond Q4_K decode / packing / affine-8 packing).
 *
 * Op-level CPU restatement of the decode hot path of ornith-rs.  Each function
 * cites the reference file:line it follows.  Reduction orders are stated in
 * the comments; the CUDA kernels use the same orders.
 */
#include "orn_oracle.h"

#include <stdlib.h>

/* ------------------------------------------------------------------------- */
/* k-quant decode                                                             */
/* ------------------------------------------------------------------------- */

/* kernels/q4k.metal:43-56 (get_scale_min_k4); numpy twin tools/q4k.py:43-48 */
void orc_q4k_scale_min(int j, const uint8_t* q, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

/* kernels/q4k.metal:64-96 (q4k_dequantize); tools/q4k.py:98-119.
 * w = (d*sc)*q - (dmin*m), low nibbles of 32 bytes then their high nibbles. */
void orc_q4k_dequantize(const uint8_t* qs, const uint8_t* scales, const uint16_t* dm,
                        int64_t nblocks, float* out) {
  for (int64_t ib = 0; ib < nblocks; ++ib) {
    const uint8_t* q = qs + ib * 128;
    const uint8_t* sc = scales + ib * 12;
    float d = o_h2f(dm[ib * 2 + 0]), dmin = o_h2f(dm[ib * 2 + 1]);
    float* y = out + ib * 256;
    for (int g = 0; g < 4; ++g) {
      uint8_t s1, m1, s2, m2;
      orc_q4k_scale_min(2 * g, sc, &s1, &m1);
      orc_q4k_scale_min(2 * g + 1, sc, &s2, &m2);
      float d1 = d * (float)s1, o1 = dmin * (float)m1;
      float d2 = d * (float)s2, o2 = dmin * (float)m2;
      for (int l = 0; l < 32; ++l) y[64 * g + l] = d1 * (float)(q[32 * g + l] & 0xF) - o1;
      for (int l = 0; l < 32; ++l) y[64 * g + 32 + l] = d2 * (float)(q[32 * g + l] >> 4) - o2;
    }
  }
}

/* Integer fields only, for the bit-exact part of the contract: 8 scales, 8
 * mins and 256 codes per block. */
void orc_q4k_fields(const uint8_t* qs, const uint8_t* scales, int64_t nblocks,
                    uint8_t* sc_out, uint8_t* mn_out, uint8_t* q_out) {
  for (int64_t ib = 0; ib < nblocks; ++ib) {
    for (int j = 0; j < 8; ++j)
      orc_q4k_scale_min(j, scales + ib * 12, sc_out + ib * 8 + j, mn_out + ib * 8 + j);
    for (int g = 0; g < 4; ++g)
      for (int l = 0; l < 32; ++l) {
        uint8_t b = qs[ib * 128 + 32 * g + l];
        q_out[ib * 256 + 64 * g + l] = b & 0xF;
        q_out[ib * 256 + 64 * g + 32 + l] = b >> 4;
      }
  }
}

/* kernels/q6k.metal:47-77 (q6k_dequantize): w = d * int8 sc * (q - 32) */
void orc_q6k_dequantize(const uint8_t* w, const int8_t* scales, const uint16_t* dm,
                        int64_t nblocks, float* out) {
  for (int64_t ib = 0; ib < nblocks; ++ib) {
    const uint8_t* ql = w + ib * 192;
    const uint8_t* qh = ql + 128;
    const int8_t* sc = scales + ib * 16;
    float d = o_h2f(dm[ib]);
    float* y = out + ib * 256;
    for (int n = 0; n < 2; ++n) {
      for (int l = 0; l < 32; ++l) {
        int is = l / 16;
        int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
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
}

/* ------------------------------------------------------------------------- */
/* mat-vec: one output element                                               */
/* ------------------------------------------------------------------------- */
/* All four weight formats share one reduction shape.  A row of K weights is
 * cut into units of U consecutive storage elements (Q4_K: 16 bytes = 32
 * weights; Q6_K: 4 bytes of ql, 4 of ql+32, 4 of qh = 16 weights; affine-8:
 * 16 bytes = 16 weights; bf16: 8 weights).  Unit u belongs to lane u mod 32;
 * a lane folds its units in ascending order into one float (inside a unit the
 * products accumulate in two fma chains, even and odd elements, whose sum is
 * the unit's dot product); the 32 lane values are folded by the xor-16,8,4,2,1
 * butterfly.  The activation row is
 * bfloat16 widened to float. */

/* kernels/q4k.metal:158-221: y += d * sum_sub sc*(sum q x) - dmin * sum_sub m*(sum x) */
static float q4k_unit(const uint8_t* qs_row, const uint8_t* sc_row, const uint16_t* dm_row,
                      int u, const float* x, float acc) {
  int blk = u >> 3, j = u & 7, g = j >> 1, h = j & 1;
  const uint8_t* b = qs_row + blk * 128 + 32 * g + 16 * h;
  const float* xl = x + blk * 256 + 64 * g + 16 * h;
  const float* xh = xl + 32;
  /* products accumulate in two chains per sum, even and odd elements, added at the end */
  float lo2[2] = {0.f, 0.f}, hi2[2] = {0.f, 0.f}, sxl = 0.f, sxh = 0.f;
  for (int i = 0; i < 16; ++i) {
    lo2[i & 1] = fmaf(xl[i], (float)(b[i] & 0xF), lo2[i & 1]);
    hi2[i & 1] = fmaf(xh[i], (float)(b[i] >> 4), hi2[i & 1]);
    sxl = sxl + xl[i];
    sxh = sxh + xh[i];
  }
  const float lo = lo2[0] + lo2[1], hi = hi2[0] + hi2[1];
  uint8_t s1, m1, s2, m2;
  orc_q4k_scale_min(2 * g, sc_row + blk * 12, &s1, &m1);
  orc_q4k_scale_min(2 * g + 1, sc_row + blk * 12, &s2, &m2);
  float d = o_h2f(dm_row[blk * 2]), dmin = o_h2f(dm_row[blk * 2 + 1]);
  float t = (float)s1 * lo;
  t = fmaf((float)s2, hi, t);
  float mt = (float)m1 * sxl;
  mt = fmaf((float)m2, sxh, mt);
  acc = fmaf(d, t, acc);
  acc = fmaf(-dmin, mt, acc);
  return acc;
}

/* kernels/q6k.metal:126-168: y += d * sum_4 sc*(sum x (q-32)) */
static float q6k_unit(const uint8_t* w_row, const int8_t* sc_row, const uint16_t* dm_row,
                      int u, const float* x, float acc) {
  int blk = u >> 4, j = u & 15, half = j >> 3, l0 = 4 * (j & 7);
  const uint8_t* ql = w_row + blk * 192 + 64 * half + l0;
  const uint8_t* qh = w_row + blk * 192 + 128 + 32 * half + l0;
  const int8_t* sc = sc_row + blk * 16 + 8 * half + l0 / 16;
  const float* xx = x + blk * 256 + 128 * half + l0;
  /* two chains per quadrant sum (even and odd elements), added at the end */
  float p0[2] = {0.f, 0.f}, p1[2] = {0.f, 0.f}, p2[2] = {0.f, 0.f}, p3[2] = {0.f, 0.f};
  for (int i = 0; i < 4; ++i) {
    int q1 = (int)((ql[i] & 0xF) | ((qh[i] & 3) << 4)) - 32;
    int q2 = (int)((ql[i + 32] & 0xF) | (((qh[i] >> 2) & 3) << 4)) - 32;
    int q3 = (int)((ql[i] >> 4) | (((qh[i] >> 4) & 3) << 4)) - 32;
    int q4 = (int)((ql[i + 32] >> 4) | (((qh[i] >> 6) & 3) << 4)) - 32;
    p0[i & 1] = fmaf(xx[i], (float)q1, p0[i & 1]);
    p1[i & 1] = fmaf(xx[i + 32], (float)q2, p1[i & 1]);
    p2[i & 1] = fmaf(xx[i + 64], (float)q3, p2[i & 1]);
    p3[i & 1] = fmaf(xx[i + 96], (float)q4, p3[i & 1]);
  }
  const float s0 = p0[0] + p0[1], s1 = p1[0] + p1[1], s2 = p2[0] + p2[1], s3 = p3[0] + p3[1];
  float t = (float)sc[0] * s0;
  t = fmaf((float)sc[2], s1, t);
  t = fmaf((float)sc[4], s2, t);
  t = fmaf((float)sc[6], s3, t);
  return fmaf(o_h2f(dm_row[blk]), t, acc);
}

/* mlx quantized.h:756-822 (affine_qmv_fast) restated for 8 bits, group 64:
 * y += scale * sum(x q) + bias * sum(x)  (src/bin/cpu_row.rs:92-132) */
static float a8_unit(const uint8_t* w_row, const bf16* s_row, const bf16* b_row, int u,
                     const float* x, float acc) {
  const uint8_t* q = w_row + 16 * u;
  const float* xx = x + 16 * u;
  float p[2] = {0.f, 0.f}, s2 = 0.f; /* products: even and odd chains, added at the end */
  for (int i = 0; i < 16; ++i) {
    p[i & 1] = fmaf(xx[i], (float)q[i], p[i & 1]);
    s2 = s2 + xx[i];
  }
  const float s1 = p[0] + p[1];
  acc = fmaf(o_bf2f(s_row[u >> 2]), s1, acc);
  acc = fmaf(o_bf2f(b_row[u >> 2]), s2, acc);
  return acc;
}

/* mlx quantized.h:756-822 (affine_qmv_fast) restated for 4 bits, group 32 (the mode of
 * src/ops/quantized.rs:249-278 for the artifact's default modules): a unit is one group,
 * byte b of its 16 code bytes holds weights 2b (low nibble) and 2b+1 (high nibble);
 * y += scale * sum(x q) + bias * sum(x) */
static float a4_unit(const uint8_t* w_row, const bf16* s_row, const bf16* b_row, int u,
                     const float* x, float acc) {
  const uint8_t* q = w_row + 16 * u;
  const float* xx = x + 32 * u;
  float p[2] = {0.f, 0.f}, s2 = 0.f; /* products: even and odd chains, added at the end */
  for (int i = 0; i < 32; ++i) {
    const float code = (float)((i & 1) ? (q[i >> 1] >> 4) : (q[i >> 1] & 0xF));
    p[i & 1] = fmaf(xx[i], code, p[i & 1]);
    s2 = s2 + xx[i];
  }
  const float s1 = p[0] + p[1];
  acc = fmaf(o_bf2f(s_row[u]), s1, acc);
  acc = fmaf(o_bf2f(b_row[u]), s2, acc);
  return acc;
}

/* mlx gemv.h (bf16 weights, float accumulate) via src/ops/matmul.rs:334-437 */
static float bf_unit(const bf16* w_row, int u, const float* x, float acc) {
  float p[2] = {0.f, 0.f}; /* the unit's products: even and odd chains; their sum joins the lane's total */
  for (int i = 0; i < 8; ++i) p[i & 1] = fmaf(x[8 * u + i], o_bf2f(w_row[8 * u + i]), p[i & 1]);
  return acc + (p[0] + p[1]);
}

float orc_row_dot(const orc_lin* L, int e, int o, const float* x) {
  float lanes[32];
  for (int l = 0; l < 32; ++l) lanes[l] = 0.f;
  int64_t row = (int64_t)e * L->O + o;
  int K = L->K;
  switch (L->kind) {
    case ORC_Q4K: {
      int nb = K / 256;
      const uint8_t* q = (const uint8_t*)L->w + row * nb * 128;
      const uint8_t* s = (const uint8_t*)L->s + row * nb * 12;
      const uint16_t* dm = (const uint16_t*)L->b + row * nb * 2;
      for (int u = 0; u < K / 32; ++u) lanes[u & 31] = q4k_unit(q, s, dm, u, x, lanes[u & 31]);
    } break;
    case ORC_Q6K: {
      int nb = K / 256;
      const uint8_t* q = (const uint8_t*)L->w + row * nb * 192;
      const int8_t* s = (const int8_t*)L->s + row * nb * 16;
      const uint16_t* dm = (const uint16_t*)L->b + row * nb;
      for (int u = 0; u < K / 16; ++u) lanes[u & 31] = q6k_unit(q, s, dm, u, x, lanes[u & 31]);
    } break;
    case ORC_A8: {
      const uint8_t* q = (const uint8_t*)L->w + row * K;
      const bf16* s = (const bf16*)L->s + row * (K / 64);
      const bf16* b = (const bf16*)L->b + row * (K / 64);
      for (int u = 0; u < K / 16; ++u) lanes[u & 31] = a8_unit(q, s, b, u, x, lanes[u & 31]);
    } break;
    case ORC_A4: {
      const uint8_t* q = (const uint8_t*)L->w + row * (K / 2);
      const bf16* s = (const bf16*)L->s + row * (K / 32);
      const bf16* b = (const bf16*)L->b + row * (K / 32);
      for (int u = 0; u < K / 32; ++u) lanes[u & 31] = a4_unit(q, s, b, u, x, lanes[u & 31]);
    } break;
    default: {
      const bf16* w = (const bf16*)L->w + row * K;
      for (int u = 0; u < K / 8; ++u) lanes[u & 31] = bf_unit(w, u, x, lanes[u & 31]);
    } break;
  }
  return o_fold32(lanes);
}

static void widen(const bf16* x, int n, float* out) {
  for (int i = 0; i < n; ++i) out[i] = o_bf2f(x[i]);
}

/* src/ops/kquant.rs:539-595 (qmv), src/ops/quantized.rs:249-333, matmul.rs:
 * y[M,O] = x[M,K] W^T, each row with the single-row arithmetic
 * (src/ops/invariant.rs:78-116).  y_f32 and/or y_bf may be NULL. */
void orc_gemv(const orc_lin* L, const bf16* x, int M, float* y_f32, bf16* y_bf) {
  int K = L->K, O = L->O;
  float* xf = (float*)malloc(sizeof(float) * (size_t)M * K);
  widen(x, M * K, xf);
#pragma omp parallel for schedule(static)
  for (int o = 0; o < O; ++o)
    for (int m = 0; m < M; ++m) {
      float v = orc_row_dot(L, 0, o, xf + (size_t)m * K);
      if (y_f32) y_f32[(size_t)m * O + o] = v;
      if (y_bf) y_bf[(size_t)m * O + o] = o_f2bf(v);
    }
  free(xf);
}

/* src/ops/kquant.rs:741-770 (gather_qmv): row r = W[rhs[r]] . x[lhs[r]] */
void orc_gather_gemv(const orc_lin* L, const bf16* x, const uint32_t* lhs,
                     const uint32_t* rhs, int rows, bf16* y) {
  int K = L->K, O = L->O;
#pragma omp parallel
  {
    float* xf = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static) collapse(1)
    for (int r = 0; r < rows; ++r) {
      widen(x + (size_t)lhs[r] * K, K, xf);
      for (int o = 0; o < O; ++o)
        y[(size_t)r * O + o] = o_f2bf(orc_row_dot(L, (int)rhs[r], o, xf));
    }
    free(xf);
  }
}

/* src/ops/embedding.rs:18-47 + mlx quantized.h:2727-2787: affine-8 row gather,
 * value = bf( f32(scale)*q + f32(bias) ) as one fma then one rounding. */
void orc_embedding_a8(const orc_lin* L, const uint32_t* ids, int T, bf16* out) {
  int K = L->K;
  for (int t = 0; t < T; ++t) {
    const uint8_t* q = (const uint8_t*)L->w + (size_t)ids[t] * K;
    const bf16* s = (const bf16*)L->s + (size_t)ids[t] * (K / 64);
    const bf16* b = (const bf16*)L->b + (size_t)ids[t] * (K / 64);
    for (int i = 0; i < K; ++i)
      out[(size_t)t * K + i] = o_f2bf(fmaf(o_bf2f(s[i >> 6]), (float)q[i], o_bf2f(b[i >> 6])));
  }
}

/* ------------------------------------------------------------------------- */
/* norms                                                                      */
/* ------------------------------------------------------------------------- */
/* Sum of squares of n floats in the order of mlx rms_single_row
 * (kernels/ornith_norm.metal:30-112): thread t owns elements 4t..4t+3 and
 * chains fma(x,x,acc); 32 threads fold by butterfly; the warp sums (zero
 * padded to 32) fold by butterfly again. */
float orc_sumsq(const float* x, int n) {
  float warps[32];
  for (int i = 0; i < 32; ++i) warps[i] = 0.f;
  int threads = (n + 3) / 4;
  int nw = (threads + 31) / 32;
  for (int w = 0; w < nw; ++w) {
    float lanes[32];
    for (int l = 0; l < 32; ++l) {
      float acc = 0.f;
      int t = w * 32 + l;
      for (int i = 0; i < 4; ++i) {
        int idx = 4 * t + i;
        if (idx < n) acc = fmaf(x[idx], x[idx], acc);
      }
      lanes[l] = acc;
    }
    warps[w] = o_fold32(lanes);
  }
  return o_fold32(warps);
}

/* mlx rms_norm.metal:11-80: out = bf( w * bf(x * inv) ), w may be NULL (= 1) */
void orc_rms_norm(const bf16* x, const bf16* w, int rows, int n, float eps, bf16* out) {
  float* xf = (float*)malloc(sizeof(float) * (size_t)n);
  for (int r = 0; r < rows; ++r) {
    widen(x + (size_t)r * n, n, xf);
    float inv = o_rsqrtf(orc_sumsq(xf, n) / (float)n + eps);
    for (int i = 0; i < n; ++i) {
      float v = o_bfr(xf[i] * inv);
      if (w) v = o_bfr(o_bf2f(w[i]) * v);
      out[(size_t)r * n + i] = o_f2bf(v);
    }
  }
  free(xf);
}

/* kernels/ornith_norm.metal:28-112 (add_rms_single_row): h = bf(a+b) is stored
 * as the new residual, then normalised. */
void orc_add_rms_norm(const bf16* a, const bf16* b, const bf16* w, int rows, int n, float eps,
                      bf16* h, bf16* out) {
  for (int i = 0; i < rows * n; ++i) h[i] = o_f2bf(o_bf2f(a[i]) + o_bf2f(b[i]));
  orc_rms_norm(h, w, rows, n, eps, out);
}

/* kernels/ornith_norm.metal:119-185 (rms_gated_single_row) */
void orc_rms_norm_gated(const bf16* x, const bf16* w, const bf16* z, int rows, int n, float eps,
                        bf16* out) {
  float* xf = (float*)malloc(sizeof(float) * (size_t)n);
  for (int r = 0; r < rows; ++r) {
    widen(x + (size_t)r * n, n, xf);
    float inv = o_rsqrtf(orc_sumsq(xf, n) / (float)n + eps);
    for (int i = 0; i < n; ++i) {
      float normed = o_bfr(o_bf2f(w[i]) * o_bfr(xf[i] * inv));
      float g = o_bf2f(z[(size_t)r * n + i]);
      g = g * o_sigmoid_f32(g);
      out[(size_t)r * n + i] = o_f2bf(g * normed);
    }
  }
  free(xf);
}

/* kernels/ornith_elementwise.metal:120-134: out = bf( sigmoid_bf(gate) * x ) */
void orc_sigmoid_gate(const bf16* gate, const bf16* x, int n, int inner, bf16* out) {
  for (int i = 0; i < n; ++i)
    out[i] = o_f2bf(o_sigmoid_bf(o_bf2f(gate[i / inner])) * o_bf2f(x[i]));
}

void orc_swiglu(const bf16* g, const bf16* u, int n, bf16* out) {
  for (int i = 0; i < n; ++i) out[i] = o_f2bf(o_swiglu_bf(o_bf2f(g[i]), o_bf2f(u[i])));
}

/* ------------------------------------------------------------------------- */
/* router                                                                     */
/* ------------------------------------------------------------------------- */
/* mlx softmax.h:10-99 (precise: float accumulate).  max is exact; thread t
 * owns 4 consecutive gates and adds their exponentials in order; threads fold
 * by butterfly per 32, then across warps. */
void orc_softmax_precise(const bf16* x, int rows, int n, bf16* out) {
  float* e = (float*)malloc(sizeof(float) * (size_t)n);
  for (int r = 0; r < rows; ++r) {
    const bf16* xr = x + (size_t)r * n;
    float m = -INFINITY;
    for (int i = 0; i < n; ++i) m = fmaxf(m, o_bf2f(xr[i]));
    float warps[32];
    for (int i = 0; i < 32; ++i) warps[i] = 0.f;
    int threads = (n + 3) / 4, nw = (threads + 31) / 32;
    for (int w = 0; w < nw; ++w) {
      float lanes[32];
      for (int l = 0; l < 32; ++l) {
        float acc = 0.f;
        for (int i = 0; i < 4; ++i) {
          int idx = 4 * (w * 32 + l) + i;
          if (idx < n) {
            e[idx] = o_expf(o_bf2f(xr[idx]) - m);
            acc = acc + e[idx];
          }
        }
        lanes[l] = acc;
      }
      warps[w] = o_fold32(lanes);
    }
    float inv = 1.0f / o_fold32(warps);
    for (int i = 0; i < n; ++i) out[(size_t)r * n + i] = o_f2bf(e[i] * inv);
  }
  free(e);
}

/* kernels/moe.metal:568-614 (router_top_k): k rounds of "largest value, then
 * largest index"; round r goes to slot k-1-r. */
void orc_router_topk(const bf16* gates, int rows, int n, int k, uint32_t* inds, bf16* scores) {
  float* v = (float*)malloc(sizeof(float) * (size_t)n);
  for (int r = 0; r < rows; ++r) {
    for (int i = 0; i < n; ++i) v[i] = o_bf2f(gates[(size_t)r * n + i]);
    for (int rr = 0; rr < k; ++rr) {
      float best = -INFINITY;
      int bi = 0;
      for (int i = 0; i < n; ++i)
        if (v[i] > best || (v[i] == best && i > bi)) { best = v[i]; bi = i; }
      inds[(size_t)r * k + (k - 1 - rr)] = (uint32_t)bi;
      scores[(size_t)r * k + (k - 1 - rr)] = gates[(size_t)r * n + bi];
      v[bi] = -INFINITY;
    }
  }
  free(v);
}

/* kernels/moe.metal:207-244 (moe_combine): all arithmetic in bfloat16,
 * ascending j. y is [T,k,dim]; gate is [T]; shared is [T,dim]. */
void orc_moe_combine(const bf16* scores, const bf16* y, const bf16* gate, const bf16* shared,
                     int T, int k, int dim, int normalize, bf16* out) {
  for (int t = 0; t < T; ++t) {
    const bf16* s = scores + (size_t)t * k;
    float denom = 0.f;
    if (normalize)
      for (int j = 0; j < k; ++j) denom = o_bfr(o_bf2f(s[j]) + denom);
    float g = o_sigmoid_bf(o_bf2f(gate[t]));
    for (int c = 0; c < dim; ++c) {
      float acc = 0.f;
      for (int j = 0; j < k; ++j) {
        float w = normalize ? o_bfr(o_bf2f(s[j]) / denom) : o_bf2f(s[j]);
        float weighted = o_bfr(o_bf2f(y[((size_t)t * k + j) * dim + c]) * w);
        acc = o_bfr(weighted + acc);
      }
      float gated = o_bfr(g * o_bf2f(shared[(size_t)t * dim + c]));
      out[(size_t)t * dim + c] = o_f2bf(acc + gated);
    }
  }
}

/* ------------------------------------------------------------------------- */
/* gated delta net                                                            */
/* ------------------------------------------------------------------------- */
/* kernels/gdn_front.metal:65-190.  conv_state [S=K-1, D]; qkv [T, D]; cw [D,K];
 * a,b [T,Hv]; outputs q,k [T,Hk,Dh], v [T,Hv,Dh], beta [T,Hv] bf16, g [T,Hv]
 * f32, conv_next [S, D].  Batch is 1 on this path. */
void orc_gdn_front(const bf16* conv_state, const bf16* qkv, const bf16* cw, const bf16* a_in,
                   const bf16* b_in, const bf16* a_log, const bf16* dt_bias, int T, int Hk,
                   int Hv, int Dh, int Kc, float eps, bf16* conv_next, bf16* q_out, bf16* k_out,
                   bf16* v_out, bf16* beta_out, float* g_out) {
  int S = Kc - 1;
  int key_dim = Hk * Dh, D = 2 * key_dim + Hv * Dh;
  float q_scale, k_scale;
  {
    float inv_scale = 1.0f / sqrtf((float)Dh); /* powf(dk, -0.5): qwen3_5.rs:506 */
    q_scale = o_bfr(inv_scale * inv_scale);
    k_scale = o_bfr(inv_scale);
  }
  float* y = (float*)malloc(sizeof(float) * (size_t)D);
  for (int t = 0; t < T; ++t) {
    for (int c = 0; c < D; ++c) {
      float acc = 0.f;
      for (int i = 0; i < Kc; ++i) {
        int j = t + i;
        const bf16* src = (j < S) ? (conv_state + (size_t)j * D) : (qkv + (size_t)(j - S) * D);
        acc = fmaf(o_bf2f(src[c]), o_bf2f(cw[(size_t)c * Kc + i]), acc);
      }
      y[c] = o_silu_bf(o_bfr(acc));
    }
    for (int slot = 0; slot < 2 * Hk; ++slot) {
      const float* ys = y + (size_t)slot * Dh;
      float inv = o_rsqrtf(orc_sumsq(ys, Dh) / (float)Dh + eps);
      int is_q = slot < Hk;
      bf16* dst = is_q ? (q_out + ((size_t)t * Hk + slot) * Dh)
                       : (k_out + ((size_t)t * Hk + (slot - Hk)) * Dh);
      float sc = is_q ? q_scale : k_scale;
      for (int i = 0; i < Dh; ++i) dst[i] = o_f2bf(sc * o_bfr(ys[i] * inv));
    }
    for (int i = 0; i < Hv * Dh; ++i) v_out[(size_t)t * Hv * Dh + i] = o_f2bf(y[2 * key_dim + i]);
    for (int h = 0; h < Hv; ++h) {
      size_t i = (size_t)t * Hv + h;
      float sp = o_softplus_bf(o_bfr(o_bf2f(a_in[i]) + o_bf2f(dt_bias[h])));
      float decay = o_expf(o_bf2f(a_log[h]));
      g_out[i] = o_expf((-decay) * sp);
      beta_out[i] = o_f2bf(o_sigmoid_bf(o_bf2f(b_in[i])));
    }
  }
  /* rows T .. T+S-1 of the concatenation are the next cached window */
  for (int j = 0; j < S; ++j) {
    int row = T + j;
    const bf16* src = (row < S) ? (conv_state + (size_t)row * D) : (qkv + (size_t)(row - S) * D);
    memcpy(conv_next + (size_t)j * D, src, sizeof(bf16) * (size_t)D);
  }
  free(y);
}

/* kernels/gated_delta.metal:36-142 (gated_delta_step_packed_btree), Dk = 128.
 * Four lanes per value row, 32 state elements per lane as eight chains of four
 * fmas; chains fold pairwise, lanes fold xor 1 then xor 2.  state [Hv,Dv,Dk]
 * f32 is updated in place; if `snaps` is not NULL the state after token t is
 * also copied to snaps + t*Hv*Dv*Dk. */
static float gd_fold(const float* part /* [4][8] */) {
  float l[4];
  for (int j = 0; j < 4; ++j) {
    const float* p = part + 8 * j;
    l[j] = ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));
  }
  return (l[0] + l[1]) + (l[2] + l[3]);
}
void orc_gated_delta(const bf16* q, const bf16* k, const bf16* v, const float* g, const bf16* beta,
                     float* state, int T, int Hk, int Hv, bf16* y, float* snaps) {
  const int D = 128;
  size_t ssz = (size_t)Hv * D * D;
  for (int t = 0; t < T; ++t) {
#pragma omp parallel for schedule(static)
    for (int hv = 0; hv < Hv; ++hv) {
      int hk = hv / (Hv / Hk);
      float qf[128], kf[128];
      for (int i = 0; i < D; ++i) {
        qf[i] = o_bf2f(q[((size_t)t * Hk + hk) * D + i]);
        kf[i] = o_bf2f(k[((size_t)t * Hk + hk) * D + i]);
      }
      float gt = g[(size_t)t * Hv + hv];
      float bt = o_bf2f(beta[(size_t)t * Hv + hv]);
      for (int dv = 0; dv < D; ++dv) {
        float* S = state + ((size_t)hv * D + dv) * D;
        float part[32];
        for (int c = 0; c < 32; ++c) {
          float acc = 0.f;
          for (int i = 0; i < 4; ++i) {
            int e = 4 * c + i;
            S[e] = S[e] * gt;
            acc = fmaf(S[e], kf[e], acc);
          }
          part[c] = acc;
        }
        float kv = gd_fold(part);
        float delta = (o_bf2f(v[((size_t)t * Hv + hv) * D + dv]) - kv) * bt;
        for (int c = 0; c < 32; ++c) {
          float acc = 0.f;
          for (int i = 0; i < 4; ++i) {
            int e = 4 * c + i;
            S[e] = fmaf(kf[e], delta, S[e]);
            acc = fmaf(S[e], qf[e], acc);
          }
          part[c] = acc;
        }
        y[((size_t)t * Hv + hv) * D + dv] = o_f2bf(gd_fold(part));
      }
    }
    if (snaps) memcpy(snaps + (size_t)t * ssz, state, sizeof(float) * ssz);
  }
}

/* ------------------------------------------------------------------------- */
/* attention                                                                  */
/* ------------------------------------------------------------------------- */
/* mlx rope.metal:11-60 via src/ops/rope.rs:23-89: non-traditional (half-split)
 * rotary on the first `dims` of each head; x is [T, H, hd] rotated in place at
 * positions offset+t. */
void orc_rope(bf16* x, int T, int H, int hd, int dims, float theta_base_ln_over_half, int offset) {
  int half = dims / 2;
  for (int t = 0; t < T; ++t)
    for (int i = 0; i < half; ++i) {
      float inv_freq = o_expf(-(float)i * theta_base_ln_over_half);
      float ang = (float)(offset + t) * inv_freq;
      float sn, cs;
      o_sincosf(ang, &sn, &cs);
      for (int h = 0; h < H; ++h) {
        bf16* p = x + ((size_t)t * H + h) * hd;
        float x1 = o_bf2f(p[i]), x2 = o_bf2f(p[i + half]);
        float t1 = x2 * sn;
        float t2 = x2 * cs;
        p[i] = o_f2bf(fmaf(x1, cs, -t1));
        p[i + half] = o_f2bf(fmaf(x1, sn, t2));
      }
    }
}

/* mlx sdpa_vector.h:15-175 as used by src/ops/sdpa.rs:122-229.  q [T,Hq,hd];
 * kc,vc [Hkv, cap, hd] hold N = offset+T keys; row r sees keys 0..offset+r.
 * Key n belongs to group n mod 32; a group runs the online softmax over its
 * keys in ascending order; each q.k dot gives dims 8l..8l+7 to lane l (fma
 * chain) and folds lanes by butterfly; groups merge by butterfly. */
void orc_sdpa_decode(const bf16* q, const bf16* kc, const bf16* vc, int T, int Hq, int Hkv,
                     int hd, int cap, int offset, float scale, bf16* out) {
  int dpl = hd / 32;
#pragma omp parallel for schedule(static) collapse(2)
  for (int r = 0; r < T; ++r)
    for (int h = 0; h < Hq; ++h) {
      int kvh = h / (Hq / Hkv);
      int L = offset + r + 1;
      float qs[512];
      for (int d = 0; d < hd; ++d) qs[d] = o_bf2f(q[((size_t)r * Hq + h) * hd + d]) * scale;
      float gmax[32], gsum[32];
      float* go = (float*)malloc(sizeof(float) * 32 * (size_t)hd);
      for (int gi = 0; gi < 32; ++gi) {
        float mx = -INFINITY, sm = 0.f;
        float* o = go + (size_t)gi * hd;
        for (int d = 0; d < hd; ++d) o[d] = 0.f;
        for (int n = gi; n < L; n += 32) {
          const bf16* kr = kc + ((size_t)kvh * cap + n) * hd;
          const bf16* vr = vc + ((size_t)kvh * cap + n) * hd;
          float lanes[32];
          for (int l = 0; l < 32; ++l) {
            float acc = 0.f;
            for (int i = 0; i < dpl; ++i) acc = fmaf(qs[l * dpl + i], o_bf2f(kr[l * dpl + i]), acc);
            lanes[l] = acc;
          }
          float score = o_fold32(lanes);
          float nm = fmaxf(mx, score);
          float factor = o_expf(mx - nm);
          float e = o_expf(score - nm);
          mx = nm;
          sm = fmaf(sm, factor, e);
          for (int d = 0; d < hd; ++d) o[d] = fmaf(o[d], factor, e * o_bf2f(vr[d]));
        }
        gmax[gi] = mx;
        gsum[gi] = sm;
      }
      float M = -INFINITY;
      for (int gi = 0; gi < 32; ++gi) M = fmaxf(M, gmax[gi]);
      float f[32], ss[32];
      for (int gi = 0; gi < 32; ++gi) {
        f[gi] = o_expf(gmax[gi] - M);
        ss[gi] = gsum[gi] * f[gi];
      }
      float S = o_fold32(ss);
      for (int d = 0; d < hd; ++d) {
        float col[32];
        for (int gi = 0; gi < 32; ++gi) col[gi] = go[(size_t)gi * hd + d] * f[gi];
        out[((size_t)r * Hq + h) * hd + d] = o_f2bf(o_fold32(col) / S);
      }
      free(go);
    }
}

/* ------------------------------------------------------------------------- */
/* greedy sampling                                                            */
/* ------------------------------------------------------------------------- */
/* src/ops/sample.rs:134-147 with mlx logsumexp.h:3-74: lse = bf(max + log sum
 * exp(x - max)), lp = bf(x - lse), argmax with the lowest index on ties
 * (arg_reduce.metal:53-66).  The sum is organised in chunks of 1024 logits:
 * chunk maximum m_b; thread t of 256 adds exp(x - m_b) of its 4 consecutive
 * logits; 8 warps fold by butterfly, then across warps; chunks merge in
 * ascending order as S = fma(S_b, exp(m_b - M), S). */
void orc_lse_chunk(const bf16* x, int n /* <= 1024 */, float* m_out, float* s_out) {
  float m = -INFINITY;
  for (int i = 0; i < n; ++i) m = fmaxf(m, o_bf2f(x[i]));
  float warps[32];
  for (int i = 0; i < 32; ++i) warps[i] = 0.f;
  for (int w = 0; w < 8; ++w) {
    float lanes[32];
    for (int l = 0; l < 32; ++l) {
      float acc = 0.f;
      for (int i = 0; i < 4; ++i) {
        int idx = 4 * (w * 32 + l) + i;
        if (idx < n) acc = acc + o_expf(o_bf2f(x[idx]) - m);
      }
      lanes[l] = acc;
    }
    warps[w] = o_fold32(lanes);
  }
  *m_out = m;
  *s_out = o_fold32(warps);
}

bf16 orc_logsumexp(const bf16* x, int V) {
  int nc = (V + 1023) / 1024;
  float* ms = (float*)malloc(sizeof(float) * 2 * (size_t)nc);
  float M = -INFINITY;
#pragma omp parallel for schedule(static)
  for (int b = 0; b < nc; ++b) {
    int n = V - b * 1024 < 1024 ? V - b * 1024 : 1024;
    orc_lse_chunk(x + (size_t)b * 1024, n, &ms[2 * b], &ms[2 * b + 1]);
  }
  for (int b = 0; b < nc; ++b) M = fmaxf(M, ms[2 * b]);
  float S = 0.f;
  for (int b = 0; b < nc; ++b) S = fmaf(ms[2 * b + 1], o_expf(ms[2 * b] - M), S);
  free(ms);
  return o_f2bf(M + o_logf(S));
}

uint32_t orc_greedy_token(const bf16* logits, int V, int normalize) {
  float lse = normalize ? o_bf2f(orc_logsumexp(logits, V)) : 0.f;
  float best = -INFINITY;
  uint32_t bi = 0;
  for (int i = 0; i < V; ++i) {
    float lp = normalize ? o_bfr(o_bf2f(logits[i]) - lse) : o_bf2f(logits[i]);
    if (lp > best) { best = lp; bi = (uint32_t)i; }
  }
  return bi;
}

/* number of OpenMP threads of the row loops (a launcher may have set OMP_NUM_THREADS=1) */
#ifdef _OPENMP
#include <omp.h>
void orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int orc_get_threads(void) { return omp_get_max_threads(); }
#else
void orc_set_threads(int n) { (void)n; }
int orc_get_threads(void) { return 1; }
#endif
