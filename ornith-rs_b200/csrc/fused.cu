// Persistent fused kernels of the decode step.
//
// A decode step at batch 1 reads ~2.7 GB of weights through ~240 dependent
// stages of a few microseconds each, so the step is organised as six kernels
// per layer, each a grid of (SM count x k) CTAs that
//   1. rebuilds its small input redundantly per CTA in shared memory (residual
//      add, RMS norm, gated norm, router softmax + top-k, SwiGLU inputs ...),
//   2. streams its share of weight rows with 128-bit coalesced loads, dequantises
//      in registers against the staged activations and folds with warp shuffles,
//   3. applies the elementwise tail in the epilogue (bf16 store, SwiGLU, the MoE
//      combine).
// The arithmetic of every stage is the arithmetic of the stand-alone kernels in
// linear.cu / ops.cu / gdn.cu / attn.cu (same rounding points, same reduction
// orders), which is what the parity tests hold both paths to.
//
// Reference functions covered: Linear::matmul / gather_matmul
// (src/ops/linear.rs:23-144), add_rms_norm / rms_norm_gated (src/ops/norm.rs),
// sparse_moe_block (src/ops/moe.rs:662-741), gdn_front + gated_delta_kernel
// (src/ops/gdn.rs:191-413), Attention::forward (src/model/qwen3_5.rs:430-474).
#include <algorithm>
#include <cstdio>
#include <mutex>
#include <set>
#include <string>
#include <utility>

#include "orn_internal.h"
#include "orn_quant.cuh"
#include "fused.h"

namespace {

// Out-of-line copies of the elementary functions: these kernels run each piece of code once or
// twice per launch, so instruction-cache misses cost more than calls do.
__device__ __noinline__ float expf_call(float x) { return orn_expf(x); }
// n / d for small n (n * d < 2^32) as one multiply: the task loops of the expert kernels divide on
// every tile, on the warp's critical path, and a hardware-less integer division is a hundred cycles
struct SmallDiv {
  uint32_t mg;
  int d;
  ORN_D explicit SmallDiv(int dd) : mg(dd > 1 ? 0xFFFFFFFFu / (uint32_t)dd + 1u : 0u), d(dd) {}
  ORN_D int operator()(int n) const { return d > 1 ? (int)__umulhi((uint32_t)n, mg) : n; }
};
// four at once: the evaluations interleave in the pipelines instead of running one after another
__device__ __noinline__ void expf4_call(float* v) {
  const float a = orn_expf(v[0]), b = orn_expf(v[1]), c = orn_expf(v[2]), d = orn_expf(v[3]);
  v[0] = a; v[1] = b; v[2] = c; v[3] = d;
}
__device__ __noinline__ float silu_bf_call(float x) { return orn_silu_bf(x); }
__device__ __noinline__ float sigmoid_bf_call(float x) { return orn_sigmoid_bf(x); }
__device__ __noinline__ float sigmoid_f32_call(float x) { return orn_sigmoid_f32(x); }
__device__ __noinline__ float softplus_bf_call(float x) { return orn_softplus_bf(x); }
__device__ __noinline__ void sincosf_call(float a, float* sn, float* cs) { orn_sincosf(a, sn, cs); }

constexpr int kMoeThreads = 512;    // expert up kernel: 16 warps, at verify width each has at most one tile
constexpr int kFusedThreads = 256;  // one CTA per SM: 8 warps (up to 255 registers each), each with its own weight ring

// ---------------------------------------------------------------------------
// activation staging: a row of K floats re-ordered so that lane l's pieces of
// unit (l + 32 s) are 16-byte neighbours of lane l+1's: conflict-free LDS.128
// ---------------------------------------------------------------------------
template <int KIND> struct Lay;
template <> struct Lay<ORN_A8>   { static constexpr int P = 4, WPU = 16, NS = 1; };
template <> struct Lay<ORN_Q4K>  { static constexpr int P = 8, WPU = 32, NS = 2; };
template <> struct Lay<ORN_Q6K>  { static constexpr int P = 4, WPU = 16, NS = 0; };
template <> struct Lay<ORN_BF16> { static constexpr int P = 2, WPU = 8,  NS = 0; };

template <int KIND> ORN_D int src_index(int u, int p);
template <> ORN_D int src_index<ORN_A8>(int u, int p) { return 16 * u + 4 * p; }
template <> ORN_D int src_index<ORN_Q4K>(int u, int p) {
  int base = (u >> 3) * 256 + 64 * ((u & 7) >> 1) + 16 * (u & 1);
  return p < 4 ? base + 4 * p : base + 32 + 4 * (p - 4);
}
template <> ORN_D int src_index<ORN_Q6K>(int u, int p) {
  return (u >> 4) * 256 + 128 * ((u & 15) >> 3) + 4 * (u & 7) + 32 * p;
}
template <> ORN_D int src_index<ORN_BF16>(int u, int p) { return 8 * u + 4 * p; }

struct XStage {
  float* xs;    // [rows][S][P][32] float4
  float* sums;  // [rows][units][NS]
  int units, S, rows;
};

__host__ __device__ inline int kind_wpu(int kind) { return kind == ORN_Q4K ? 32 : kind == ORN_BF16 ? 8 : 16; }
__host__ __device__ inline int kind_p(int kind) { return kind == ORN_Q4K ? 8 : kind == ORN_BF16 ? 2 : 4; }
__host__ __device__ inline int kind_ns(int kind) { return kind == ORN_A8 ? 1 : kind == ORN_Q4K ? 2 : 0; }
__host__ __device__ inline size_t stage_floats(int kind, int rows, int K) {
  int units = K / kind_wpu(kind);
  int S = (units + 31) / 32;
  return (size_t)rows * S * kind_p(kind) * 32 * 4 + (size_t)rows * units * kind_ns(kind);
}

// carve a stage out of shared memory (returns the next free float)
ORN_D float* stage_carve(float* base, int kind, int rows, int K, XStage& X) {
  X.units = K / kind_wpu(kind);
  X.S = (X.units + 31) / 32;
  X.rows = rows;
  X.xs = base;
  X.sums = base + (size_t)rows * X.S * kind_p(kind) * 32 * 4;
  return X.sums + (size_t)rows * X.units * kind_ns(kind);
}

// The staged place of the four consecutive activations x[k .. k+3] (k a multiple of 4) of row m:
// the inverse of src_index.  Formats without per-unit sums can be staged piece by piece straight
// from the registers a thread loaded them into, with no linear copy of the row in between.
template <int KIND> ORN_D void unit_of(int k, int& u, int& p);
template <> ORN_D void unit_of<ORN_A8>(int k, int& u, int& p) { u = k >> 4; p = (k & 15) >> 2; }
template <> ORN_D void unit_of<ORN_BF16>(int k, int& u, int& p) { u = k >> 3; p = (k & 7) >> 2; }
template <> ORN_D void unit_of<ORN_Q6K>(int k, int& u, int& p) {
  const int r = k & 255, r2 = r & 127;
  u = (k >> 8) * 16 + (r >> 7) * 8 + ((r2 & 31) >> 2);
  p = r2 >> 5;
}
template <> ORN_D void unit_of<ORN_Q4K>(int k, int& u, int& p) {
  const int r = k & 255, r2 = r & 63, r3 = r2 & 31;
  u = (k >> 8) * 8 + (r >> 6) * 2 + (r3 >> 4);
  p = (r2 >> 5) * 4 + ((r3 & 15) >> 2);
}
template <int KIND>
ORN_D void stage_piece(const XStage& X, int m, int k, float4 v) {
  constexpr int P = Lay<KIND>::P;
  int u, p;
  unit_of<KIND>(k, u, p);
  reinterpret_cast<float4*>(X.xs)[((size_t)(m * X.S + (u >> 5)) * P + p) * 32 + (u & 31)] = v;
}
// zero the unit slots behind the last unit of every row (rows whose unit count is not a multiple of 32)
template <int KIND>
ORN_D void stage_zero_tail(const XStage& X) {
  constexpr int P = Lay<KIND>::P;
  const int tail = X.S * 32 - X.units;
  if (tail == 0) return;
  for (int idx = threadIdx.x; idx < X.rows * tail * P; idx += blockDim.x) {
    const int m = idx / (tail * P), rem = idx - m * tail * P;
    const int u = X.units + rem / P, p = rem % P;
    reinterpret_cast<float4*>(X.xs)[((size_t)(m * X.S + (u >> 5)) * P + p) * 32 + (u & 31)] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// lin: [rows][K] floats (row stride `stride`) -> stage, by the threads tid of nthreads (a subset of
// the CTA may stage while other warps do something else); no sync inside.  A thread owns whole
// units of any row (rows x unit slots are one flat index space, so short rows keep every thread
// busy): it moves the unit's P pieces to their permuted places and, for the formats that need it,
// adds the unit's elements in ascending order into the staged sum.
template <int KIND>
__device__ __noinline__ void stage_fill_part(const float* lin, int stride, const XStage& X, int tid, int nthreads) {
  constexpr int P = Lay<KIND>::P, NS = Lay<KIND>::NS;
  const int padded = X.S * 32;  // unit slots per row, including the empty tail
  const int total = X.rows * padded;
#pragma unroll 1
  for (int idx = tid; idx < total; idx += nthreads) {
    const int m = idx / padded, u = idx - m * padded;
    const float* src = lin + (size_t)m * stride;
    float4* dst = reinterpret_cast<float4*>(X.xs) + (size_t)m * padded * P;
    const int lane = u & 31, s = u >> 5;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int p = 0; p < P; ++p) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (u < X.units) v = *reinterpret_cast<const float4*>(src + src_index<KIND>(u, p));
      dst[(s * P + p) * 32 + lane] = v;
      if (NS == 1 || (NS == 2 && p < 4)) { s0 = s0 + v.x; s0 = s0 + v.y; s0 = s0 + v.z; s0 = s0 + v.w; }
      if (NS == 2 && p >= 4) { s1 = s1 + v.x; s1 = s1 + v.y; s1 = s1 + v.z; s1 = s1 + v.w; }
    }
    if (u < X.units) {
      if (NS == 1) X.sums[(size_t)m * X.units + u] = s0;
      if (NS == 2) { X.sums[((size_t)m * X.units + u) * 2] = s0; X.sums[((size_t)m * X.units + u) * 2 + 1] = s1; }
    }
  }
}

// the same by every thread of the CTA
template <int KIND>
__device__ __noinline__ void stage_fill(const float* lin, int stride, const XStage& X) {
  stage_fill_part<KIND>(lin, stride, X, threadIdx.x, blockDim.x);
}
ORN_D void stage_fill_kind(int kind, const float* lin, int stride, const XStage& X) {
  switch (kind) {
    case ORN_A8: stage_fill<ORN_A8>(lin, stride, X); break;
    case ORN_Q4K: stage_fill<ORN_Q4K>(lin, stride, X); break;
    case ORN_Q6K: stage_fill<ORN_Q6K>(lin, stride, X); break;
    default: stage_fill<ORN_BF16>(lin, stride, X); break;
  }
}

// ---------------------------------------------------------------------------
// weight units (the arithmetic of linear.cu's Fmt<>, activations from registers)
// ---------------------------------------------------------------------------
template <int KIND> struct WU;

template <> struct WU<ORN_A8> {
  struct W { uint4 q; uint32_t sb; };
  // unit u of a row record staged in shared memory: [codes K][{scale, bias} K/64]
  ORN_D static void lds(const uint8_t* rec, uint32_t off1, uint32_t, int u, W& w) {
    w.q = *reinterpret_cast<const uint4*>(rec + 16 * u);
    w.sb = *reinterpret_cast<const uint32_t*>(rec + off1 + 4 * (u >> 2));
  }
  ORN_D static float fold(const W& w, const float* x, const float* sm, int, float acc) {
    const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
    const uint64_t nm = pk2(-8388608.0f, -8388608.0f);
    uint64_t s2 = pk2(0.f, 0.f);  // (even chain, odd chain)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      s2 = ffma2(pk2(x[4 * k + 0], x[4 * k + 1]), byte2_f<0>(qw[k], nm), s2);
      s2 = ffma2(pk2(x[4 * k + 2], x[4 * k + 3]), byte2_f<2>(qw[k], nm), s2);
    }
    acc = fmaf(bf_lo(w.sb), pk2_sum(s2), acc);
    acc = fmaf(bf_hi(w.sb), sm[0], acc);
    return acc;
  }
};

template <> struct WU<ORN_Q4K> {
  struct W { uint4 q; uint4 meta; };
  // staged row record: [codes nb*128][headers nb*16]
  ORN_D static void lds(const uint8_t* rec, uint32_t off1, uint32_t, int u, W& w) {
    w.q = *reinterpret_cast<const uint4*>(rec + 16 * u);
    w.meta = *reinterpret_cast<const uint4*>(rec + off1 + (u >> 3) * 16);
  }
  ORN_D static float fold(const W& w, const float* x, const float* sm, int u, float acc) {
    const int g = (u & 7) >> 1;
    const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
    const uint64_t nm = pk2(-8388608.0f, -8388608.0f);
    uint64_t lo2 = pk2(0.f, 0.f), hi2 = pk2(0.f, 0.f);  // (even chain, odd chain) of the two sub-blocks
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t l4 = qw[k] & 0x0F0F0F0Fu, h4 = (qw[k] >> 4) & 0x0F0F0F0Fu;
      lo2 = ffma2(pk2(x[4 * k + 0], x[4 * k + 1]), byte2_f<0>(l4, nm), lo2);
      lo2 = ffma2(pk2(x[4 * k + 2], x[4 * k + 3]), byte2_f<2>(l4, nm), lo2);
      hi2 = ffma2(pk2(x[16 + 4 * k + 0], x[16 + 4 * k + 1]), byte2_f<0>(h4, nm), hi2);
      hi2 = ffma2(pk2(x[16 + 4 * k + 2], x[16 + 4 * k + 3]), byte2_f<2>(h4, nm), hi2);
    }
    const float lo = pk2_sum(lo2), hi = pk2_sum(hi2);
    const float d = h2f((uint16_t)(w.meta.x & 0xffff)), dmin = h2f((uint16_t)(w.meta.x >> 16));
    // get_scale_min_k4 (kernels/q4k.metal:43-56) for the sub-blocks 2g and 2g+1 at once: their
    // bytes are neighbours in each of the three scale words, so both come out of 16-bit pieces
    // (j < 4: sc = q[j] & 63, m = q[j+4] & 63; else sc = (q[j+4] & 15) | (q[j-4] >> 6 << 4),
    // m = (q[j+4] >> 4) | (q[j] >> 6 << 4))
    const int sh = (g & 1) * 16;
    const uint32_t qa = (w.meta.y >> sh) & 0xffffu, qb = (w.meta.z >> sh) & 0xffffu, qc = (w.meta.w >> sh) & 0xffffu;
    const bool low = g < 2;
    const uint32_t sc2 = low ? (qa & 0x3f3fu) : ((qc & 0x0f0fu) | ((qa >> 2) & 0x3030u));
    const uint32_t mn2 = low ? (qb & 0x3f3fu) : (((qc >> 4) & 0x0f0fu) | ((qb >> 2) & 0x3030u));
    float s1, s2, m1, m2;
    {
      const uint64_t sp = byte2_f<0>(sc2, nm), mp = byte2_f<0>(mn2, nm);
      asm("mov.b64 {%0, %1}, %2;" : "=f"(s1), "=f"(s2) : "l"(sp));
      asm("mov.b64 {%0, %1}, %2;" : "=f"(m1), "=f"(m2) : "l"(mp));
    }
    float t = s1 * lo;
    t = fmaf(s2, hi, t);
    float mt = m1 * sm[0];
    mt = fmaf(m2, sm[1], mt);
    acc = fmaf(d, t, acc);
    acc = fmaf(-dmin, mt, acc);
    return acc;
  }
};

template <> struct WU<ORN_Q6K> {
  struct W { uint32_t qa, qb, qh, sc4; float d; };
  // staged row record: [ql|qh nb*192][scales nb*16][d nb*2]
  ORN_D static void lds(const uint8_t* rec, uint32_t off1, uint32_t off2, int u, W& w) {
    const int blk = u >> 4, j = u & 15, half = j >> 3, l0 = 4 * (j & 7);
    const uint8_t* base = rec + blk * 192;
    w.qa = *reinterpret_cast<const uint32_t*>(base + 64 * half + l0);
    w.qb = *reinterpret_cast<const uint32_t*>(base + 64 * half + 32 + l0);
    w.qh = *reinterpret_cast<const uint32_t*>(base + 128 + 32 * half + l0);
    const uint2 s8 = *reinterpret_cast<const uint2*>(rec + off1 + blk * 16 + 8 * half);
    // scales sc[is + 0, 2, 4, 6] of this half: bytes is, is+2 of either word, one byte permute
    w.sc4 = __byte_perm(s8.x, s8.y, (l0 >> 4) ? 0x7531u : 0x6420u);
    w.d = h2f(*reinterpret_cast<const uint16_t*>(rec + off2 + 2 * blk));
  }
  ORN_D static float fold(const W& w, const float* x, const float*, int, float acc) {
    const uint32_t q1 = (w.qa & 0x0F0F0F0Fu) | ((w.qh & 0x03030303u) << 4);
    const uint32_t q2 = (w.qb & 0x0F0F0F0Fu) | ((w.qh & 0x0C0C0C0Cu) << 2);
    const uint32_t q3 = ((w.qa >> 4) & 0x0F0F0F0Fu) | (w.qh & 0x30303030u);
    const uint32_t q4 = ((w.qb >> 4) & 0x0F0F0F0Fu) | ((w.qh & 0xC0C0C0C0u) >> 2);
    const uint64_t nm = pk2(-8388640.0f, -8388640.0f);  // -(2^23 + 32)
    const uint64_t z = pk2(0.f, 0.f);
    uint64_t p0 = ffma2(pk2(x[0], x[1]), byte2_f<0>(q1, nm), z);
    p0 = ffma2(pk2(x[2], x[3]), byte2_f<2>(q1, nm), p0);
    uint64_t p1 = ffma2(pk2(x[4], x[5]), byte2_f<0>(q2, nm), z);
    p1 = ffma2(pk2(x[6], x[7]), byte2_f<2>(q2, nm), p1);
    uint64_t p2 = ffma2(pk2(x[8], x[9]), byte2_f<0>(q3, nm), z);
    p2 = ffma2(pk2(x[10], x[11]), byte2_f<2>(q3, nm), p2);
    uint64_t p3 = ffma2(pk2(x[12], x[13]), byte2_f<0>(q4, nm), z);
    p3 = ffma2(pk2(x[14], x[15]), byte2_f<2>(q4, nm), p3);
    const float s0 = pk2_sum(p0), s1 = pk2_sum(p1), s2 = pk2_sum(p2), s3 = pk2_sum(p3);
    // four int8 scales -> float: b ^ 0x80 is b + 128 as an unsigned byte, then the exact byte -> float form
    float c0, c1, c2, c3;
    {
      const uint32_t ub = w.sc4 ^ 0x80808080u;
      const uint64_t nb = pk2(-8388736.0f, -8388736.0f);  // -(2^23 + 128)
      const uint64_t c01 = byte2_f<0>(ub, nb), c23 = byte2_f<2>(ub, nb);
      asm("mov.b64 {%0, %1}, %2;" : "=f"(c0), "=f"(c1) : "l"(c01));
      asm("mov.b64 {%0, %1}, %2;" : "=f"(c2), "=f"(c3) : "l"(c23));
    }
    float t = c0 * s0;
    t = fmaf(c1, s1, t);
    t = fmaf(c2, s2, t);
    t = fmaf(c3, s3, t);
    return fmaf(w.d, t, acc);
  }
};

template <> struct WU<ORN_BF16> {
  struct W { uint4 q; };
  ORN_D static void lds(const uint8_t* rec, uint32_t, uint32_t, int u, W& w) {
    w.q = *reinterpret_cast<const uint4*>(rec + 16 * u);
  }
  ORN_D static float fold(const W& w, const float* x, const float*, int, float acc) {
    float f[8];
    widen8(w.q, f);
    uint64_t s2 = pk2(0.f, 0.f);  // the unit's (even chain, odd chain); their sum joins the lane's total
#pragma unroll
    for (int i = 0; i < 8; i += 2) s2 = ffma2(pk2(x[i], x[i + 1]), pk2(f[i], f[i + 1]), s2);
    return acc + pk2_sum(s2);
  }
};

// ---------------------------------------------------------------------------
// weight streaming: per-warp rings of shared-memory slots filled by bulk async
// copies (cp.async.bulk, the 1-D TMA form) that complete on an mbarrier.
// Weight rows are contiguous records in HBM (codes, then scales), so ONE bulk
// copy brings a tile of R consecutive rows; lane 0 of a warp issues the copies
// for the warp's next tiles, all 32 lanes wait on the slot's barrier and read
// their own 16-byte pieces (consecutive lanes, consecutive addresses: no bank
// conflicts).  A warp only ever waits for copies it issued itself, so there is
// no cross-warp dependency; the wait is bounded and reports through `err`.
// ---------------------------------------------------------------------------
ORN_D uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
ORN_D void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
ORN_D void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
ORN_D void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
constexpr uint32_t kWaitHintNs = 200000;  // a waiting warp may be suspended this long per try
ORN_D bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kWaitHintNs)
      : "memory");
  return ok != 0;
}
ORN_D void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
ORN_D void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

constexpr uint32_t kWaitLimit = 1u << 14;  // try_wait rounds before giving up (each round may sleep kWaitHintNs)

// Rows per tile by format and row length class (0: K <= 512, 1: K <= 2048, 2: longer), chosen so
// that a tile is at most 9216 bytes: 8 warps x 2 slots of that fit beside the staged activations.
constexpr int kSlotMax = 9216;
__host__ __device__ constexpr int k_class(int K) { return K <= 512 ? 0 : K <= 2048 ? 1 : 2; }
__host__ __device__ constexpr int tile_rows(int kind, int kc) {
  return kind == ORN_A8    ? (kc == 0 ? 8 : kc == 1 ? 4 : 2)
         : kind == ORN_Q4K ? (kc == 0 ? 8 : 2)
         : kind == ORN_Q6K ? (kc == 2 ? 2 : 4)
                           : (kc == 0 ? 8 : kc == 1 ? 2 : 1);
}
// rows per tile in the expert kernels
__host__ __device__ constexpr int moe_rows(int kind, int kc) {
  return kind == ORN_A8    ? (kc == 0 ? 8 : kc == 1 ? 4 : 2)
         : kind == ORN_Q4K ? (kc == 0 ? 8 : 4)
         : kind == ORN_Q6K ? (kc == 2 ? 2 : 4)
                           : (kc == 0 ? 8 : kc == 1 ? 2 : 1);
}
// rows of a tile in the expert up kernel: half of them gate rows, half their up rows
__host__ __device__ constexpr int up_rows(int kind, int kc) {
  return kind == ORN_A8    ? (kc <= 1 ? 4 : 2)
         : kind == ORN_Q4K ? (kc <= 1 ? 8 : 4)
         : kind == ORN_Q6K ? (kc <= 1 ? 4 : 2)
                           : 2;
}
__host__ __device__ constexpr int pad_m(int M) { return M == 3 ? 4 : M; }

struct Ring {
  uint32_t bar0;       // shared address of this warp's first barrier
  uint32_t buf0;       // shared address of this warp's first slot
  uint8_t* buf;        // generic address of the same
  uint32_t slot_bytes;
  int depth;
  int* err;
  uint32_t limit;      // try_wait rounds before a wait gives up
};

// lane 0: one bulk copy of `bytes` (a multiple of 16) into a slot
ORN_D void ring_fill(const Ring& R, int slot, const uint8_t* src, uint32_t bytes) {
  const uint32_t bar = R.bar0 + 8 * slot;
  mbar_expect_tx(bar, bytes);
  bulk_g2s(R.buf0 + slot * R.slot_bytes, src, bytes, bar);
}
// lane 0: two bulk copies into one slot (a gate tile at offset 0 and its up tile at `off1`)
ORN_D void ring_fill2(const Ring& R, int slot, const uint8_t* src0, const uint8_t* src1, uint32_t bytes, uint32_t off1) {
  const uint32_t bar = R.bar0 + 8 * slot;
  const uint32_t dst = R.buf0 + slot * R.slot_bytes;
  mbar_expect_tx(bar, 2 * bytes);
  bulk_g2s(dst, src0, bytes, bar);
  bulk_g2s(dst + off1, src1, bytes, bar);
}
// all lanes: wait for a slot; false after the bounded wait ran out
ORN_D bool ring_wait(const Ring& R, int slot, uint32_t parity) {
  const uint32_t bar = R.bar0 + 8 * slot;
  for (uint32_t it = 0; it < R.limit; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  if ((threadIdx.x & 31) == 0) atomicExch(R.err, 1);
  return false;
}

// carve the rings of all warps out of shared memory and initialise the barriers
ORN_D void ring_setup(Ring& R, uint8_t* base, uint32_t slot_bytes, int depth, int* err) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base);
  uint8_t* bufs = base + (((size_t)nwarps * depth * 8 + 127) & ~(size_t)127);
  R.bar0 = smem_u32(bars + (size_t)warp * depth);
  R.buf = bufs + (size_t)warp * depth * slot_bytes;
  R.buf0 = smem_u32(R.buf);
  R.slot_bytes = slot_bytes;
  R.depth = depth;
  R.err = err;
  R.limit = kWaitLimit;
  if (lane == 0)
    for (int i = 0; i < depth; ++i) mbar_init(R.bar0 + 8 * i, 1);
  fence_mbar_init();
  fence_proxy_async();
}
__host__ __device__ inline size_t ring_bytes(int nwarps, int depth, uint32_t slot_bytes) {
  return (((size_t)nwarps * depth * 8 + 127) & ~(size_t)127) + (size_t)nwarps * depth * slot_bytes;
}

// One warp, a tile of R staged row records (record r at buf + r*rec): adds every unit of the rows
// to the lane partials acc[r*MP + m] of activation rows m0 .. m0+M-1 (MP = M padded to a power of
// two).  A lane visits its units in ascending order, the staged activations of a lane-step are
// read once and folded into all R rows.
template <int KIND, int M, int R, bool TAIL>
ORN_D void tile_step(const uint8_t* buf, uint32_t rec, uint32_t off1, uint32_t off2, int ss, int units, const float4* xb,
                     int xrow, const float* sb, int srow, int lane, float* acc) {
  using U = WU<KIND>;
  constexpr int P = Lay<KIND>::P, NS = Lay<KIND>::NS, MP = pad_m(M);
  const int u = lane + 32 * ss;
  if (TAIL && u >= units) return;
  typename U::W w[R];
#pragma unroll
  for (int r = 0; r < R; ++r) U::lds(buf + r * rec, off1, off2, u, w[r]);
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float xv[P * 4];
    const float4* xp = xb + m * xrow + ss * (P * 32);
#pragma unroll
    for (int p = 0; p < P; ++p) {
      const float4 v = xp[p * 32];
      xv[4 * p] = v.x; xv[4 * p + 1] = v.y; xv[4 * p + 2] = v.z; xv[4 * p + 3] = v.w;
    }
    float sm[NS > 0 ? NS : 1];
#pragma unroll
    for (int i = 0; i < NS; ++i) sm[i] = sb[m * srow + ss * 32 * NS + i];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r * MP + m] = U::fold(w[r], xv, sm, u, acc[r * MP + m]);
  }
}

template <int KIND, int M, int R>
ORN_D void tile_dot(const uint8_t* buf, const LinDev& L, const XStage& X, int m0, int lane, float* acc) {
  constexpr int P = Lay<KIND>::P, NS = Lay<KIND>::NS;
  const RecGeom g = rec_geom(KIND, L.K);
  const float4* xb = reinterpret_cast<const float4*>(X.xs) + (size_t)m0 * X.S * (P * 32) + lane;
  const int xrow = X.S * P * 32;
  const float* sb = X.sums + ((size_t)m0 * X.units + lane) * NS;
  const int srow = X.units * NS;
  // the last lane-step may be partial; one checked copy of the loop body serves both (a second,
  // unchecked copy costs more in instruction-cache misses than the check costs in issue slots)
  for (int ss = 0; ss < X.S; ++ss)
    tile_step<KIND, M, R, true>(buf, g.rec, g.b0, g.b0 + g.b1, ss, X.units, xb, xrow, sb, srow, lane, acc);
}

// Butterfly over V values per lane (V a power of two <= 32) in reduce-scatter form: at the level
// with xor mask m a lane keeps half of its values and adds its partner's copies of them, so each
// value goes through exactly the additions of the plain xor-16..1 butterfly (a + b is commutative,
// both partners hold the same sum) with V-1 + (5 - log2 V) shuffles instead of 5 V.  Returns the
// lane's value; `which` is its index.  Lanes that differ only in the low 5 - log2 V bits hold copies.
template <int V>
ORN_D float rs_butterfly(float* v, int lane, int& which) {
  int idx = 0;
  int n = V;
#pragma unroll
  for (int mask = 16; mask >= 1; mask >>= 1) {
    if (n > 1) {
      const int h = n >> 1;
      const bool upper = (lane & mask) != 0;
#pragma unroll
      for (int i = 0; i < V / 2; ++i) {
        if (i < h) {
          const float send = upper ? v[i] : v[i + h];
          const float keep = upper ? v[i + h] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
        }
      }
      idx = idx * 2 + (upper ? 1 : 0);
      n = h;
    } else {
      v[0] = v[0] + __shfl_xor_sync(0xffffffffu, v[0], mask);
    }
  }
  which = idx;
  return v[0];
}
template <>
ORN_D float rs_butterfly<1>(float* v, int, int& which) {
  which = 0;
  return warp_sum(v[0]);
}

// ---------------------------------------------------------------------------
// block-wide RMS statistics in the order of the stand-alone rms kernels:
// virtual thread t owns elements 4t..4t+3, 32 virtual threads fold by
// butterfly, the warp sums (zero padded to 32) fold by butterfly again.
// lin holds `rows` rows of n raw values (stride `stride`); inv[m] receives
// 1/sqrt(sumsq/n + eps).  `red` is rows*32 floats of shared memory.
// ---------------------------------------------------------------------------
__device__ __noinline__ void block_rms_inv(const float* lin, int stride, int rows, int n, float eps, float* red, float* inv) {
  const int lane = threadIdx.x & 31;
#pragma unroll 1
  for (int i = threadIdx.x; i < rows * 32; i += blockDim.x) red[i] = 0.f;
  __syncthreads();
  const int nvt = (n + 3) / 4;
  const int nvt_pad = ((nvt + 31) / 32) * 32;
#pragma unroll 1
  for (int m = 0; m < rows; ++m) {
#pragma unroll 1
    for (int vt = threadIdx.x; vt < nvt_pad; vt += blockDim.x) {
      float acc = 0.f;
      if (4 * vt < n) {  // n is a multiple of 4 here
        const float4 v = *reinterpret_cast<const float4*>(lin + (size_t)m * stride + 4 * vt);
        acc = fmaf(v.x, v.x, acc);
        acc = fmaf(v.y, v.y, acc);
        acc = fmaf(v.z, v.z, acc);
        acc = fmaf(v.w, v.w, acc);
      }
      acc = warp_sum(acc);
      if (lane == 0) red[m * 32 + (vt >> 5)] = acc;
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5;
#pragma unroll 1
  for (int m = warp; m < rows; m += (blockDim.x >> 5)) {
    const float total = warp_sum(red[m * 32 + lane]);
    if (lane == 0) inv[m] = orn_rsqrtf(total / (float)n + eps);
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------
// prologues: build lin[M][K] (floats holding bfloat16 values) in shared memory
// ---------------------------------------------------------------------------
struct Prologue {
  int mode;            // PRO_*
  int K;               // length of the staged row
  const bf16_t* a;     // ADDNORM: [M][K] ; PLAIN: [M][K] ; GATED: y [M][K] ; MTPJOIN: trunk hidden [M][K/2]
  const bf16_t* b;     // ADDNORM: second addend or null ; GATED: z [M][K]
  const bf16_t* w;     // norm weight ([K], GATED: [128], MTPJOIN: pre_fc_norm_embedding [K/2])
  const bf16_t* w2;    // MTPJOIN: pre_fc_norm_hidden
  bf16_t* sum_out;     // ADDNORM: where CTA 0 stores bf(a+b) (may be null)
  bf16_t* norm_out;    // where CTA 0 stores the staged row as bfloat16 (may be null)
  LinDev emb;          // MTPJOIN: embedding table
  const uint32_t* ids; // MTPJOIN: token ids [M]
  float eps;
};

// The prologues off the hottest path (plain copy, gated norm over heads, MTP join), one
// out-of-line copy shared by every instantiation; M is a run-time count here.
__device__ __noinline__ void prologue_other(const Prologue& P, int M, float* lin, float* red) {
  const int K = P.K;
  float* inv = red + M * 32;
  if (P.mode == PRO_PLAIN) {
#pragma unroll 1
    for (int c = threadIdx.x * 4; c < M * K; c += blockDim.x * 4) {
      const uint2 av = __ldg(reinterpret_cast<const uint2*>(P.a + c));
      *reinterpret_cast<float4*>(lin + c) = make_float4(bf_lo(av.x), bf_hi(av.x), bf_lo(av.y), bf_hi(av.y));
    }
  } else if (P.mode == PRO_GATED) {
    // rms_norm_gated over 128-wide heads (kernels/ornith_norm.metal:119-185): a warp per (row, head)
    // pair, four pairs in flight per warp so that their loads overlap
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int pairs = M * (K >> 7);
    const uint2 wv = __ldg(reinterpret_cast<const uint2*>(P.w + 4 * lane));
    const float wf[4] = {bf_lo(wv.x), bf_hi(wv.x), bf_lo(wv.y), bf_hi(wv.y)};
    for (int p0 = warp; p0 < pairs; p0 += 4 * nw) {
      uint2 av[4], zv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int pair = p0 + j * nw;
        if (pair < pairs) {
          av[j] = __ldg(reinterpret_cast<const uint2*>(P.a + pair * 128 + 4 * lane));
          zv[j] = __ldg(reinterpret_cast<const uint2*>(P.b + pair * 128 + 4 * lane));
        }
      }
#pragma unroll 1
      for (int j = 0; j < 4; ++j) {
        const int pair = p0 + j * nw;
        if (pair >= pairs) break;
        const int base = pair * 128 + 4 * lane;
        const uint2 a2 = j == 0 ? av[0] : j == 1 ? av[1] : j == 2 ? av[2] : av[3];
        const uint2 z2 = j == 0 ? zv[0] : j == 1 ? zv[1] : j == 2 ? zv[2] : zv[3];
        const float xv[4] = {bf_lo(a2.x), bf_hi(a2.x), bf_lo(a2.y), bf_hi(a2.y)};
        const float gz[4] = {bf_lo(z2.x), bf_hi(z2.x), bf_lo(z2.y), bf_hi(z2.y)};
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc = fmaf(xv[i], xv[i], acc);
        acc = warp_sum(acc);
        const float iv = orn_rsqrtf(acc / 128.0f + P.eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float normed = bfr(wf[i] * bfr(xv[i] * iv));
          float g = gz[i];
          g = g * sigmoid_f32_call(g);
          lin[base + i] = bfr(g * normed);
        }
      }
    }
  } else {  // PRO_MTPJOIN: [norm(embed(id)) | norm(trunk hidden)] (src/model/mtp.rs:179-187)
    const int H = K >> 1;
    for (int m = 0; m < M; ++m) {
      int64_t row = P.ids[m];
      if (row >= P.emb.O) row = P.emb.O - 1;  // an id outside the table (argmax over NaN logits) must not fault
#pragma unroll 1
      for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const uint32_t sb = reinterpret_cast<const uint32_t*>(P.emb.s + row * P.emb.rec)[c >> 6];
        lin[(size_t)m * K + c] = bfr(fmaf(bf_lo(sb), (float)P.emb.w[row * P.emb.rec + c], bf_hi(sb)));
        lin[(size_t)m * K + H + c] = bf2f(P.a[(size_t)m * H + c]);
      }
    }
    __syncthreads();
    block_rms_inv(lin, K, M, H, P.eps, red, inv);
#pragma unroll 1
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      const float w = bf2f(P.w[c]);
      for (int m = 0; m < M; ++m) lin[(size_t)m * K + c] = bfr(w * bfr(lin[(size_t)m * K + c] * inv[m]));
    }
    __syncthreads();
    block_rms_inv(lin + H, K, M, H, P.eps, red, inv);
#pragma unroll 1
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      const float w = bf2f(P.w2[c]);
      for (int m = 0; m < M; ++m) lin[(size_t)m * K + H + c] = bfr(w * bfr(lin[(size_t)m * K + H + c] * inv[m]));
    }
  }
}

// The add + norm prologue's global operands, fetched into registers before the weight prefetch
// starts: a thread owns up to kAddNormGroups groups of 4 consecutive elements of every row
// (K <= 4 * kAddNormGroups * blockDim.x is checked at launch).
constexpr int kAddNormGroups = 2;
template <int M>
struct AddNormIn {
  uint2 w[kAddNormGroups], a[M][kAddNormGroups], b[M][kAddNormGroups];
  ORN_D void load(const Prologue& P) {
#pragma unroll
    for (int g = 0; g < kAddNormGroups; ++g) {
      const int c = 4 * (threadIdx.x + g * blockDim.x);
      if (c < P.K) {
        w[g] = __ldg(reinterpret_cast<const uint2*>(P.w + c));
#pragma unroll
        for (int m = 0; m < M; ++m) {
          a[m][g] = __ldg(reinterpret_cast<const uint2*>(P.a + (size_t)m * P.K + c));
          if (P.b != nullptr) b[m][g] = __ldg(reinterpret_cast<const uint2*>(P.b + (size_t)m * P.K + c));
        }
      }
    }
  }
};

// scratch: red[M*32 + M] floats.  Every loop walks (row m, 4-element group) so
// that no index needs a division and global traffic is at least 64-bit.
// PRO_ADDNORM leaves the normalised rows in the stages X (pieces go from the registers to their
// staged places, unit sums by a 4-lane chain); the other modes leave them in `lin` for stage_fill.
template <int M, int MASK>
ORN_D void run_prologue(const Prologue& P, const AddNormIn<M>& in, float* lin, float* red, const XStage* X) {
  const int K = P.K;
  float* inv = red + M * 32;
  if (P.mode == PRO_ADDNORM) {
    // A thread's 4-element groups are exactly the virtual threads of the RMS statistic (group g of
    // thread t = virtual thread t + g * blockDim), so the sums of squares come straight from the
    // registers: warp butterflies here, one barrier, the second-level butterfly, one barrier.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float hv[M][kAddNormGroups][4];
#pragma unroll
    for (int g = 0; g < kAddNormGroups; ++g) {
      const int c0 = 4 * (threadIdx.x + g * blockDim.x);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float* v = hv[m][g];
        v[0] = v[1] = v[2] = v[3] = 0.f;
        if (c0 < K) {
          const uint2 av = in.a[m][g];
          v[0] = bf_lo(av.x); v[1] = bf_hi(av.x); v[2] = bf_lo(av.y); v[3] = bf_hi(av.y);
          if (P.b != nullptr) {
            const uint2 bv = in.b[m][g];
            v[0] = bfr(v[0] + bf_lo(bv.x)); v[1] = bfr(v[1] + bf_hi(bv.x));
            v[2] = bfr(v[2] + bf_lo(bv.y)); v[3] = bfr(v[3] + bf_hi(bv.y));
          }
          if (P.sum_out != nullptr && blockIdx.x == 0) {
            uint2 o;
            o.x = (uint32_t)f2bf(v[0]) | ((uint32_t)f2bf(v[1]) << 16);
            o.y = (uint32_t)f2bf(v[2]) | ((uint32_t)f2bf(v[3]) << 16);
            *reinterpret_cast<uint2*>(P.sum_out + (size_t)m * K + c0) = o;
          }
        }
        float acc = 0.f;  // a virtual thread past the row contributes an exact zero
        acc = fmaf(v[0], v[0], acc);
        acc = fmaf(v[1], v[1], acc);
        acc = fmaf(v[2], v[2], acc);
        acc = fmaf(v[3], v[3], acc);
        acc = warp_sum(acc);
        if (lane == 0) red[m * 32 + warp + g * nw] = acc;  // virtual warp (t + g * blockDim) / 32
      }
    }
    // virtual warps nobody owns (the CTA has kAddNormGroups * nw <= 32 of them) are zero
    if (warp == 0 && lane >= kAddNormGroups * nw)
#pragma unroll
      for (int m = 0; m < M; ++m) red[m * 32 + lane] = 0.f;
    __syncthreads();
    if (warp < M) {
      const float total = warp_sum(red[warp * 32 + lane]);
      if (lane == 0) inv[warp] = orn_rsqrtf(total / (float)K + P.eps);
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < kAddNormGroups; ++g) {
      const int c0 = 4 * (threadIdx.x + g * blockDim.x);
      if (c0 < K) {
        const uint2 ww = in.w[g];
        const float wv[4] = {bf_lo(ww.x), bf_hi(ww.x), bf_lo(ww.y), bf_hi(ww.y)};
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float* v = hv[m][g];
          const float iv = inv[m];
          const float4 f = make_float4(bfr(wv[0] * bfr(v[0] * iv)), bfr(wv[1] * bfr(v[1] * iv)),
                                       bfr(wv[2] * bfr(v[2] * iv)), bfr(wv[3] * bfr(v[3] * iv)));
          if (MASK & (1 << ORN_Q4K)) stage_piece<ORN_Q4K>(X[ORN_Q4K], m, c0, f);
          if (MASK & (1 << ORN_Q6K)) stage_piece<ORN_Q6K>(X[ORN_Q6K], m, c0, f);
          if (MASK & (1 << ORN_A8)) stage_piece<ORN_A8>(X[ORN_A8], m, c0, f);
          if (MASK & (1 << ORN_BF16)) stage_piece<ORN_BF16>(X[ORN_BF16], m, c0, f);
          if (P.norm_out != nullptr && blockIdx.x == 0) {
            uint2 o;
            o.x = (uint32_t)f2bf(f.x) | ((uint32_t)f2bf(f.y) << 16);
            o.y = (uint32_t)f2bf(f.z) | ((uint32_t)f2bf(f.w) << 16);
            *reinterpret_cast<uint2*>(P.norm_out + (size_t)m * K + c0) = o;
          }
          if (MASK & ((1 << ORN_A8) | (1 << ORN_Q4K))) {
            // The 16 activations of an aligned run (four lanes' pieces) are one unit of the 8-bit
            // format and half a unit of Q4_K: their sum, added in ascending order from zero, passes
            // from lane to lane (c0 < K holds for whole warps: K is a multiple of 256).
            float run = 0.f;
#pragma unroll
            for (int step = 0; step < 4; ++step) {
              if ((lane & 3) == step) { run = run + f.x; run = run + f.y; run = run + f.z; run = run + f.w; }
              const float up = __shfl_up_sync(0xffffffffu, run, 1);
              if ((lane & 3) == step + 1) run = up;
            }
            if ((lane & 3) == 3) {
              if (MASK & (1 << ORN_A8)) X[ORN_A8].sums[(size_t)m * X[ORN_A8].units + (c0 >> 4)] = run;
              if (MASK & (1 << ORN_Q4K)) {
                int u, pp;
                unit_of<ORN_Q4K>(c0, u, pp);
                X[ORN_Q4K].sums[((size_t)m * X[ORN_Q4K].units + u) * 2 + (pp >> 2)] = run;
              }
            }
          }
        }
      }
    }
    if (MASK & (1 << ORN_Q4K)) stage_zero_tail<ORN_Q4K>(X[ORN_Q4K]);
    if (MASK & (1 << ORN_Q6K)) stage_zero_tail<ORN_Q6K>(X[ORN_Q6K]);
    if (MASK & (1 << ORN_A8)) stage_zero_tail<ORN_A8>(X[ORN_A8]);
    if (MASK & (1 << ORN_BF16)) stage_zero_tail<ORN_BF16>(X[ORN_BF16]);
  } else if (P.mode == PRO_PLAIN) {
    // rows as they are: pieces go from the loads (a batch of four per thread in flight) to their
    // staged places, unit sums as above.  M * K / 4 pieces over whole warps: rounds are warp-uniform.
    constexpr int kBatch = 4;
    const int lane = threadIdx.x & 31;
    const int step = blockDim.x * 4;
#pragma unroll 1
    for (int base = threadIdx.x * 4; base < M * K; base += kBatch * step) {
      uint2 av[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j)
        if (base + j * step < M * K) av[j] = __ldg(reinterpret_cast<const uint2*>(P.a + base + j * step));
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int c = base + j * step;
        if (c < M * K) {
          const float4 f = make_float4(bf_lo(av[j].x), bf_hi(av[j].x), bf_lo(av[j].y), bf_hi(av[j].y));
          const int m = c / K, k = c - m * K;
          if (MASK & (1 << ORN_Q4K)) stage_piece<ORN_Q4K>(X[ORN_Q4K], m, k, f);
          if (MASK & (1 << ORN_Q6K)) stage_piece<ORN_Q6K>(X[ORN_Q6K], m, k, f);
          if (MASK & (1 << ORN_A8)) stage_piece<ORN_A8>(X[ORN_A8], m, k, f);
          if (MASK & (1 << ORN_BF16)) stage_piece<ORN_BF16>(X[ORN_BF16], m, k, f);
          if (P.norm_out != nullptr && blockIdx.x == 0) *reinterpret_cast<uint2*>(P.norm_out + c) = av[j];
          if (MASK & ((1 << ORN_A8) | (1 << ORN_Q4K))) {
            float run = 0.f;
#pragma unroll
            for (int st = 0; st < 4; ++st) {
              if ((lane & 3) == st) { run = run + f.x; run = run + f.y; run = run + f.z; run = run + f.w; }
              const float up = __shfl_up_sync(0xffffffffu, run, 1);
              if ((lane & 3) == st + 1) run = up;
            }
            if ((lane & 3) == 3) {
              if (MASK & (1 << ORN_A8)) X[ORN_A8].sums[(size_t)m * X[ORN_A8].units + (k >> 4)] = run;
              if (MASK & (1 << ORN_Q4K)) {
                int u, pp;
                unit_of<ORN_Q4K>(k, u, pp);
                X[ORN_Q4K].sums[((size_t)m * X[ORN_Q4K].units + u) * 2 + (pp >> 2)] = run;
              }
            }
          }
        }
      }
    }
    if (MASK & (1 << ORN_Q4K)) stage_zero_tail<ORN_Q4K>(X[ORN_Q4K]);
    if (MASK & (1 << ORN_Q6K)) stage_zero_tail<ORN_Q6K>(X[ORN_Q6K]);
    if (MASK & (1 << ORN_A8)) stage_zero_tail<ORN_A8>(X[ORN_A8]);
    if (MASK & (1 << ORN_BF16)) stage_zero_tail<ORN_BF16>(X[ORN_BF16]);
  } else {
    prologue_other(P, M, lin, red);
    __syncthreads();
    if (P.norm_out != nullptr && blockIdx.x == 0) {
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll 1
        for (int c = threadIdx.x; c < K; c += blockDim.x) P.norm_out[(size_t)m * K + c] = f2bf(lin[(size_t)m * K + c]);
    }
  }
}

// ---------------------------------------------------------------------------
// kernel 1: prologue + up to four row jobs over the same staged input
// ---------------------------------------------------------------------------
struct RowJob {
  LinDev lin;    // weight matrix (E == 1)
  LinDev lin2;   // EPI_SWIGLU: the "up" matrix paired with lin ("gate")
  bf16_t* out;   // [M][O]
  int epi;       // EPI_STORE | EPI_SWIGLU
  int tiles;     // row tiles of the job
};
struct RowJobs {
  RowJob job[4];
  int njobs;
  int total;       // tiles of all jobs
  int kinds_mask;  // bit k set when some job has weights of kind k
};

// rows per tile of a format inside a launch whose rows have K weights (class KC)
template <int KC>
ORN_D int rows_of(int kind) {
  return kind == ORN_A8 ? tile_rows(ORN_A8, KC) : kind == ORN_Q4K ? tile_rows(ORN_Q4K, KC)
         : kind == ORN_Q6K ? tile_rows(ORN_Q6K, KC) : tile_rows(ORN_BF16, KC);
}

// dot of one staged tile for the format of L (only formats in MASK are compiled in)
template <int M, int MASK, int KC>
ORN_D void tile_dot_masked(const uint8_t* buf, const LinDev& L, const XStage* X, int lane, float* acc) {
  if ((MASK & (1 << ORN_A8)) && L.kind == ORN_A8)
    tile_dot<ORN_A8, M, tile_rows(ORN_A8, KC)>(buf, L, X[ORN_A8], 0, lane, acc);
  else if ((MASK & (1 << ORN_Q4K)) && L.kind == ORN_Q4K)
    tile_dot<ORN_Q4K, M, tile_rows(ORN_Q4K, KC)>(buf, L, X[ORN_Q4K], 0, lane, acc);
  else if ((MASK & (1 << ORN_Q6K)) && L.kind == ORN_Q6K)
    tile_dot<ORN_Q6K, M, tile_rows(ORN_Q6K, KC)>(buf, L, X[ORN_Q6K], 0, lane, acc);
  else if ((MASK & (1 << ORN_BF16)) && L.kind == ORN_BF16)
    tile_dot<ORN_BF16, M, tile_rows(ORN_BF16, KC)>(buf, L, X[ORN_BF16], 0, lane, acc);
}

__device__ __noinline__ float swiglu_bf_call(float g, float u) { return orn_swiglu_bf(g, u); }

// butterfly + store of a finished tile of R x M sums.  A SwiGLU tile holds R/2 gate rows followed
// by their R/2 up rows: after the butterfly the up sums sit 16 lanes above the gate sums.
template <int M, int R>
ORN_D void tile_store(float* acc, bool swiglu, int lane, bf16_t* out, int O, int row0, int nvalid) {
  constexpr int MP = pad_m(M), V = R * MP;
  int which;
  float v = rs_butterfly<V>(acc, lane, which);
  bool writer = (lane & (32 / V - 1)) == 0;
  if (swiglu) {
    const float u = __shfl_down_sync(0xffffffffu, v, 16);
    v = swiglu_bf_call(bfr(v), bfr(u));
    writer = writer && lane < 16;
  }
  const int r = which / MP, m = which % MP;
  if (writer && r < nvalid && m < M) out[(size_t)m * O + row0 + r] = f2bf(v);
}
template <int M, int MASK, int KC>
ORN_D void tile_store_masked(int kind, float* acc, bool swiglu, int lane, bf16_t* out, int O, int row0, int nvalid) {
  if ((MASK & (1 << ORN_A8)) && kind == ORN_A8)
    tile_store<M, tile_rows(ORN_A8, KC)>(acc, swiglu, lane, out, O, row0, nvalid);
  else if ((MASK & (1 << ORN_Q4K)) && kind == ORN_Q4K)
    tile_store<M, tile_rows(ORN_Q4K, KC)>(acc, swiglu, lane, out, O, row0, nvalid);
  else if ((MASK & (1 << ORN_Q6K)) && kind == ORN_Q6K)
    tile_store<M, tile_rows(ORN_Q6K, KC)>(acc, swiglu, lane, out, O, row0, nvalid);
  else if ((MASK & (1 << ORN_BF16)) && kind == ORN_BF16)
    tile_store<M, tile_rows(ORN_BF16, KC)>(acc, swiglu, lane, out, O, row0, nvalid);
}

// position of a warp in its tile sequence: tile g of the concatenated jobs (stepping by GW),
// resolved to (job j, tile t).  A SwiGLU job's tile is rows/2 gate rows and their up rows.
struct Cursor {
  int g, j, t;
  ORN_D void locate(const RowJobs& J) {
    j = 0;
    t = g;
    while (j < J.njobs && t >= J.job[j].tiles) { t -= J.job[j].tiles; ++j; }
  }
  ORN_D bool valid(const RowJobs& J) const { return g < J.total; }
  ORN_D void advance(const RowJobs& J, int GW) {
    g += GW;
    if (g < J.total) locate(J);
  }
};

constexpr int kMaxAcc = 32;  // R * pad(M) never exceeds this

template <int M, int MASK, int KC>
__global__ void __launch_bounds__(kFusedThreads, 1) k_norm_gemv(Prologue P, RowJobs J, uint32_t slot_bytes, int depth,
                                                                uint32_t ring_off, int late, int* err) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float* smem = reinterpret_cast<float*>(smem_raw);
  const int lane = threadIdx.x & 31;
  // a launch with fewer tiles than warps gives warp w of CTA b the tiles w * CTAs + b, so that it
  // still spreads over every SM; otherwise a CTA's warps take neighbouring tiles
  const int gw = J.total >= (int)(gridDim.x * (blockDim.x >> 5)) ? blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)
                                                                  : (threadIdx.x >> 5) * gridDim.x + blockIdx.x;
  const int GW = gridDim.x * (blockDim.x >> 5);
  // The weights do not depend on the activations, so the kernel is launched as a programmatic
  // dependent: barriers and the first `depth` tiles of every warp are requested while the
  // previous kernel is still draining; only then does it wait for that kernel's results and
  // rebuild its input while HBM is busy.
  // (`late`: wide windows whose staged rows leave too little room run the rings over the
  // prologue's scratch instead, so their first tiles can only be requested after the staging.)
  pdl_trigger();
  Ring R;
  if (!late) {
    ring_setup(R, smem_raw + ring_off, slot_bytes, depth, err);
    __syncwarp();
  }
  Cursor pc{gw, 0, 0}, cc{gw, 0, 0};
  if (pc.valid(J)) { pc.locate(J); cc = pc; }
  int pslot = 0;
  auto issue = [&]() {  // all lanes keep the cursor; lane 0 issues
    const RowJob& job = J.job[pc.j];
    if (lane == 0) {
      const LinDev& L = job.lin;
      const int rows = rows_of<KC>(L.kind);
      if (job.epi == EPI_SWIGLU) {
        const int half = rows >> 1;
        const int row = pc.t * half;
        const int n = min(half, L.O - row);
        ring_fill2(R, pslot, L.w + (size_t)row * L.rec, job.lin2.w + (size_t)row * L.rec, n * L.rec, half * L.rec);
      } else {
        const int row = pc.t * rows;
        const int n = min(rows, L.O - row);
        ring_fill(R, pslot, L.w + (size_t)row * L.rec, n * L.rec);
      }
    }
    pc.advance(J, GW);
    if (++pslot == depth) pslot = 0;
  };
  int primed = 0;
  if (!late)
    for (; primed < 1 && pc.valid(J); ++primed) issue();  // one tile per warp ahead of the wait ...
  pdl_wait();  // everything below reads what earlier kernels wrote
  AddNormIn<M> pin;
  if (P.mode == PRO_ADDNORM) pin.load(P);
  if (!late)
    for (; primed < depth && pc.valid(J); ++primed) issue();  // ... the rest behind the prologue's own loads

  // stages, then the prologue's scratch
  float* next = smem;
  XStage X[4];
  constexpr int mask = MASK;
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (mask & (1 << k)) next = stage_carve(next, k, M, P.K, X[k]);
  // the add + norm and the plain prologue stage from registers: they need the reduction scratch
  // only, no linear copy of the rows (the launch sizes shared memory accordingly)
  float* lin = smem + (((next - smem) + 31) & ~31);
  float* red = (P.mode == PRO_ADDNORM || P.mode == PRO_PLAIN) ? lin : lin + (size_t)M * P.K;
  run_prologue<M, MASK>(P, pin, lin, red, X);
  if (P.mode != PRO_ADDNORM && P.mode != PRO_PLAIN) {
    if (mask & (1 << ORN_Q4K)) stage_fill<ORN_Q4K>(lin, P.K, X[ORN_Q4K]);
    if (mask & (1 << ORN_Q6K)) stage_fill<ORN_Q6K>(lin, P.K, X[ORN_Q6K]);
    if (mask & (1 << ORN_A8)) stage_fill<ORN_A8>(lin, P.K, X[ORN_A8]);
    if (mask & (1 << ORN_BF16)) stage_fill<ORN_BF16>(lin, P.K, X[ORN_BF16]);
  }
  __syncthreads();
  if (late) {
    ring_setup(R, smem_raw + ring_off, slot_bytes, depth, err);
    __syncwarp();
    for (int i = 0; i < depth && pc.valid(J); ++i) issue();
  }

  float acc[kMaxAcc];
  int slot = 0;
  uint32_t parity = 0;
  while (cc.valid(J)) {
    if (!ring_wait(R, slot, parity)) return;
    const RowJob& job = J.job[cc.j];
    const uint8_t* buf = R.buf + (size_t)slot * slot_bytes;
#pragma unroll
    for (int i = 0; i < kMaxAcc; ++i) acc[i] = 0.f;
    tile_dot_masked<M, MASK, KC>(buf, job.lin, X, lane, acc);
    __syncwarp();
    const bool swiglu = job.epi == EPI_SWIGLU;
    const int kind = job.lin.kind, O = job.lin.O, t = cc.t;
    bf16_t* out = job.out;
    if (pc.valid(J)) {
      if (lane == 0) fence_proxy_async();
      issue();  // refills the slot just consumed
    }
    const int rows = swiglu ? rows_of<KC>(kind) >> 1 : rows_of<KC>(kind);
    const int row0 = t * rows;
    tile_store_masked<M, MASK, KC>(kind, acc, swiglu, lane, out, O, row0, min(rows, O - row0));
    cc.advance(J, GW);
    if (++slot == depth) { slot = 0; parity ^= 1; }
  }
}

// ---------------------------------------------------------------------------
// kernel 2: router top-k in the prologue, routed expert gate/up + SwiGLU
// ---------------------------------------------------------------------------
struct MoeUpParams {
  const bf16_t* logits;  // [M][E] router logits
  const bf16_t* x;       // [M][H] normed input
  LinDev gate, up;       // [E, I, H]
  uint32_t* inds;        // [M][k] out (CTA 0)
  bf16_t* scores;        // [M][k] out (CTA 0)
  bf16_t* act;           // [M*k][I] out
  int M, E, k, H, I;
};

// softmax (mlx softmax.h:10-99, float accumulate) then router_top_k
// (kernels/moe.metal:568-614) for one token by one warp; results to shared
// kMaxVW virtual warps of 128 logits (so n <= 128 * kMaxVW); the 256-expert instantiation carries
// half the code of the 512-expert one, and this code runs once per CTA from cold instruction caches
template <int kMaxVW>
__device__ __noinline__ void warp_softmax_topk_n(const bf16_t* logits, int n, int k, float* probs /*[n] smem*/,
                             float* red /*[32] smem*/, uint32_t* inds, float* scores, int lane) {
  // the lane's logits (4 consecutive per virtual warp) come in with one round of loads; the
  // maximum and the exponentials then work from registers
  const int nvt = (n + 3) / 4;
  const int nvw = (nvt + 31) / 32;
  float xv[kMaxVW][4];
  const bool vec = (n & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 7) == 0;
#pragma unroll
  for (int vw = 0; vw < kMaxVW; ++vw) {
    const int base = 4 * (vw * 32 + lane);
#pragma unroll
    for (int i = 0; i < 4; ++i) xv[vw][i] = -INFINITY;
    if (vw < nvw) {
      if (vec && base < n) {
        const uint2 r = __ldg(reinterpret_cast<const uint2*>(logits + base));
        xv[vw][0] = bf_lo(r.x); xv[vw][1] = bf_hi(r.x); xv[vw][2] = bf_lo(r.y); xv[vw][3] = bf_hi(r.y);
      } else if (!vec) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (base + i < n) xv[vw][i] = bf2f(logits[base + i]);
      }
    }
  }
  float mx = -INFINITY;
#pragma unroll
  for (int vw = 0; vw < kMaxVW; ++vw)
#pragma unroll
    for (int i = 0; i < 4; ++i) mx = fmaxf(mx, xv[vw][i]);
  mx = warp_max(mx);
  red[lane] = 0.f;
  __syncwarp();
#pragma unroll
  for (int vw = 0; vw < kMaxVW; ++vw) {
    if (vw < nvw) {
      const int vt = vw * 32 + lane;
      float ev[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) ev[i] = xv[vw][i] - mx;  // absent entries are -inf - mx: their exp is not used
      expf4_call(ev);
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = 4 * vt + i;
        if (idx < n) {
          probs[idx] = ev[i];
          acc = acc + ev[i];
        }
      }
      acc = warp_sum(acc);
      if (lane == 0) red[vw] = acc;
    }
  }
  __syncwarp();
  const float inv = 1.0f / warp_sum(red[lane]);
  __syncwarp();
  for (int i = lane; i < n; i += 32) probs[i] = bfr(probs[i] * inv);
  __syncwarp();
  // k rounds of argmax: largest value, ties to the larger index.  The probabilities are
  // non-negative bfloat16 values, so their float bits order like the values and have 16 free low
  // bits: (bits | index) + 1 is a key whose unsigned maximum is exactly that rule, and one
  // hardware warp reduction per round finds it (0 marks entries that are absent, taken, or NaN;
  // with nothing left the round yields index 0, as the comparison form does).
  constexpr int kMaxPerLane = 4 * kMaxVW;
  uint32_t key[kMaxPerLane];
#pragma unroll
  for (int s = 0; s < kMaxPerLane; ++s) {
    const int i = lane + 32 * s;
    key[s] = 0;
    if (i < n) {
      const float p = probs[i];
      const uint32_t bits = __float_as_uint(p);
      if (p == p && (int)bits >= 0) key[s] = (bits | (uint32_t)i) + 1u;
    }
  }
  for (int r = 0; r < k; ++r) {
    uint32_t best = 0;
#pragma unroll
    for (int s = 0; s < kMaxPerLane; ++s) best = key[s] > best ? key[s] : best;
    const uint32_t m = __reduce_max_sync(0xffffffffu, best);
    const uint32_t mi = m ? ((m - 1u) & 0xffffu) : 0u;
#pragma unroll
    for (int s = 0; s < kMaxPerLane; ++s)
      if (m != 0 && key[s] == m) key[s] = 0;
    if (lane == 0) {
      inds[k - 1 - r] = mi;
      scores[k - 1 - r] = probs[mi];
    }
  }
  __syncwarp();
}
ORN_D void warp_softmax_topk(const bf16_t* logits, int n, int k, float* probs, float* red, uint32_t* inds,
                             float* scores, int lane) {
  if (n <= 256) warp_softmax_topk_n<2>(logits, n, k, probs, red, inds, scores, lane);
  else warp_softmax_topk_n<4>(logits, n, k, probs, red, inds, scores, lane);
}

template <int KIND, int KC>
__global__ void __launch_bounds__(kMoeThreads, 1) k_moe_up(MoeUpParams P, uint32_t slot_bytes, int depth,
                                                             uint32_t ring_off, int* err) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float* smem = reinterpret_cast<float*>(smem_raw);
  constexpr int RT = up_rows(KIND, KC);
  const int M = P.M;
  XStage X;
  float* next = stage_carve(smem, KIND, M, P.H, X);
  uint32_t* inds = reinterpret_cast<uint32_t*>(next);  // [M][k], lives through the kernel
  next += M * P.k;
  float* lin = smem + (((next - smem) + 31) & ~31);    // [M][H]
  float* probs = lin + (size_t)M * P.H;                // [M][E]
  float* red = probs + (size_t)M * P.E;                // [M][32]
  float* scores = red + M * 32;                        // [M][k]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_trigger();
  Ring R;
  ring_setup(R, smem_raw + ring_off, slot_bytes, depth, err);
  pdl_wait();  // the routing (and so the first weight tile) depends on the previous kernel's logits
  // the first M warps route their token while the other warps stage x: one barrier for both
  if (warp < M)
    warp_softmax_topk(P.logits + (size_t)warp * P.E, P.E, P.k, probs + (size_t)warp * P.E, red + warp * 32,
                      inds + warp * P.k, scores + warp * P.k, lane);
  else {
    // pieces of four activations go from the load straight to their staged places; the sum of an
    // aligned run of 16 (a unit of the 8-bit format, half a unit of Q4_K) passes along four lanes
    // in ascending order.  M * H / 4 pieces over whole warps: every round is warp-uniform.
    const int tid = threadIdx.x - 32 * M, nt = blockDim.x - 32 * M;
    for (int i = tid * 4; i < M * P.H; i += nt * 4) {
      const uint2 v = __ldg(reinterpret_cast<const uint2*>(P.x + i));
      const float4 f = make_float4(bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y));
      const int m = i / P.H, k = i - m * P.H;
      stage_piece<KIND>(X, m, k, f);
      if (Lay<KIND>::NS > 0) {
        float run = 0.f;
#pragma unroll
        for (int step = 0; step < 4; ++step) {
          if ((lane & 3) == step) { run = run + f.x; run = run + f.y; run = run + f.z; run = run + f.w; }
          const float up = __shfl_up_sync(0xffffffffu, run, 1);
          if ((lane & 3) == step + 1) run = up;
        }
        if ((lane & 3) == 3) {
          int u, pp;
          unit_of<KIND>(k, u, pp);
          if (Lay<KIND>::NS == 1) X.sums[(size_t)m * X.units + u] = run;
          else X.sums[((size_t)m * X.units + u) * 2 + (pp >> 2)] = run;
        }
      }
    }
    const int tail = X.S * 32 - X.units;  // empty unit slots behind a row's last unit
    for (int idx = tid; idx < M * tail * Lay<KIND>::P; idx += nt) {
      const int m = idx / (tail * Lay<KIND>::P), rem = idx - m * tail * Lay<KIND>::P;
      const int u = X.units + rem / Lay<KIND>::P, pc = rem % Lay<KIND>::P;
      reinterpret_cast<float4*>(X.xs)[((size_t)(m * X.S + (u >> 5)) * Lay<KIND>::P + pc) * 32 + (u & 31)] =
          make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  __syncthreads();
  // task g = (routed row mj, tile t): RT/2 consecutive output rows of the expert's gate matrix and the
  // same rows of its up matrix in one slot, one dot over the RT staged rows, one butterfly
  constexpr int HALF = RT / 2;
  const int gw = warp * gridDim.x + blockIdx.x, GW = gridDim.x * (blockDim.x >> 5);  // few tiles still reach every SM
  const int ntile = (P.I + HALF - 1) / HALF;
  const int total = M * P.k * ntile;
  const SmallDiv by_ntile(ntile), by_k(P.k);
  const RecGeom geo = rec_geom(KIND, P.H);
  int pg = gw, pslot = 0;
  auto issue = [&]() {
    if (lane == 0) {
      const int mj = by_ntile(pg), t = pg - mj * ntile;
      const int o = t * HALF;
      const int n = min(HALF, P.I - o);
      const size_t row = (size_t)inds[mj] * P.I + o;
      ring_fill2(R, pslot, P.gate.w + row * geo.rec, P.up.w + row * geo.rec, n * geo.rec, HALF * geo.rec);
    }
    pg += GW;
    if (++pslot == depth) pslot = 0;
  };
  for (int i = 0; i < depth && pg < total; ++i) issue();
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i < M * P.k; i += blockDim.x) {
      P.inds[i] = inds[i];
      P.scores[i] = f2bf(scores[i]);
    }
  float gu[RT];
  int slot = 0;
  uint32_t parity = 0;
  for (int cg = gw; cg < total; cg += GW) {
    const int mj = by_ntile(cg), t = cg - mj * ntile;
    const int m = by_k(mj);
#pragma unroll
    for (int r = 0; r < RT; ++r) gu[r] = 0.f;
    if (!ring_wait(R, slot, parity)) return;
    tile_dot<KIND, 1, RT>(R.buf + (size_t)slot * slot_bytes, P.gate, X, m, lane, gu);
    __syncwarp();
    if (pg < total) {
      if (lane == 0) fence_proxy_async();
      issue();
    }
    if (++slot == depth) { slot = 0; parity ^= 1; }
    int which;
    const float gs = rs_butterfly<RT>(gu, lane, which);  // gate sums in lanes 0..15, up sums 16 lanes above
    const float us = __shfl_down_sync(0xffffffffu, gs, 16);
    const int o = t * HALF + which;
    if (lane < 16 && (lane & (32 / RT - 1)) == 0 && o < P.I)
      P.act[(size_t)mj * P.I + o] = f2bf(swiglu_bf_call(bfr(gs), bfr(us)));
  }
}

// ---------------------------------------------------------------------------
// kernel 3: routed down projections + shared down + combine
// (kernels/moe.metal:207-244 arithmetic in the epilogue)
// ---------------------------------------------------------------------------
struct MoeDownParams {
  const bf16_t* act;     // [M*k][I]
  const bf16_t* sact;    // [M][SI]
  const uint32_t* inds;  // [M][k]
  const bf16_t* scores;  // [M][k]
  const bf16_t* gs;      // [M] shared-expert gate logits
  LinDev down;           // [E, H, I]
  LinDev sh_down;        // [1, H, SI]
  bf16_t* out;           // [M][H]
  int M, k, H, I, SI, normalize;
};

// Task = (token m, group of RT consecutive output columns).  Consecutive columns are consecutive
// weight rows of one expert, so one bulk copy brings a group's rows of one routed expert.  A task
// belongs to a PAIR of warps: the even warp takes the first half of the routed experts, the odd
// warp the second half and the shared expert, so the serial chain of tiles per warp is half as
// long and 16 warps hide each other's latencies.  After the butterfly each lane holds one column's
// sum; the even warp runs its part of the bf16 combine (ascending j) and hands the running value
// to the odd warp through shared memory, which adds its own terms in order and stores.
constexpr int kDownThreads = 512;

template <int KIND, int KC>
__global__ void __launch_bounds__(kDownThreads, 1) k_moe_down(MoeDownParams P, uint32_t slot_bytes, int depth,
                                                                uint32_t ring_off, int* err) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float* smem = reinterpret_cast<float*>(smem_raw);
  constexpr int RT = moe_rows(KIND, KC);
  const int M = P.M;
  const int rows = M * P.k;
  XStage X, XS;
  float* next = stage_carve(smem, KIND, rows, P.I, X);
  next = stage_carve(next, KIND, M, P.SI, XS);
  constexpr bool kDirect = Lay<KIND>::NS == 0;       // staged straight from registers (no per-unit sums)
  float* wts = next;                                   // [M][k] normalised scores
  float* raw = wts + rows;                             // [M][k] the router's scores
  float* gsig = raw + rows;                            // [M]
  float* xch = gsig + M;                               // [2][pairs][32] running combine values
  uint32_t* inds = reinterpret_cast<uint32_t*>(xch + 2 * (kDownThreads / 64) * 32);
  next = reinterpret_cast<float*>(inds + rows);
  float* lin = smem + (((next - smem) + 31) & ~31);    // [rows][I] then [M][SI], only when !kDirect
  float* lin2 = lin + (size_t)rows * P.I;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_trigger();
  Ring R;
  ring_setup(R, smem_raw + ring_off, slot_bytes, depth, err);
  pdl_wait();
  // the first batch of routed activations and the shared expert's into registers, so that their
  // latency overlaps the routing table's and the first weight requests
  constexpr int kPre = 4;
  uint2 pre[kPre], spre = make_uint2(0u, 0u);
#pragma unroll
  for (int j = 0; j < kPre; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < rows * P.I) pre[j] = __ldg(reinterpret_cast<const uint2*>(P.act + i));
  }
  if (threadIdx.x * 4 < M * P.SI) spre = __ldg(reinterpret_cast<const uint2*>(P.sact + threadIdx.x * 4));
  float sc_mine = 0.f, gs_mine = 0.f;
  if (threadIdx.x < rows) {
    inds[threadIdx.x] = P.inds[threadIdx.x];
    sc_mine = bf2f(P.scores[threadIdx.x]);
    if (threadIdx.x < M) gs_mine = bf2f(P.gs[threadIdx.x]);
    raw[threadIdx.x] = sc_mine;  // the denominators below read all k of a token
  }
  __syncthreads();
  // warp pair `gp` walks the tasks; this warp's tiles of a task are q = 0 .. nt-1
  const int h = warp & 1, pair = warp >> 1, npairs = blockDim.x >> 6;
  const int gp = pair * gridDim.x + blockIdx.x, GP = gridDim.x * npairs;  // few tasks still reach every SM
  const int ngroups = (P.H + RT - 1) / RT;
  const int total = M * ngroups;
  const SmallDiv by_ngroups(ngroups);
  const int k0 = P.k >> 1;
  const int nt = h ? P.k - k0 + 1 : k0;  // the odd warp's last tile is the shared expert's
  const RecGeom geo = rec_geom(KIND, P.I), sgeo = rec_geom(KIND, P.SI);
  int pg = gp, pq = 0, pslot = 0;  // producer: task, tile within the task
  auto fill = [&](int task, int q, int slot) {  // one lane: request tile q of `task` into `slot`
    const int m = by_ngroups(task), grp = task - m * ngroups;
    const int c0 = grp * RT;
    const int n = min(RT, P.H - c0);
    const int j = (h ? k0 : 0) + q;
    if (j < P.k) ring_fill(R, slot, P.down.w + ((size_t)inds[m * P.k + j] * P.H + c0) * geo.rec, n * geo.rec);
    else ring_fill(R, slot, P.sh_down.w + (size_t)c0 * sgeo.rec, n * sgeo.rec);
  };
  // the first `depth` tiles of the warp are requested by as many lanes at once (a request costs
  // one lane some hundred cycles of address arithmetic and copy-engine hand-over)
  if (nt > 0 && pg < total) {
    const int ahead = min(depth, nt * ((total - pg + GP - 1) / GP));
    if (lane < ahead) fill(pg + (lane / nt) * GP, lane % nt, lane);
    pg += (ahead / nt) * GP;
    pq = ahead % nt;
    pslot = ahead == depth ? 0 : ahead;
  }
  auto issue = [&]() {  // steady state: lane 0 refills the slot just consumed
    if (lane == 0) fill(pg, pq, pslot);
    if (++pq == nt) { pq = 0; pg += GP; }
    if (++pslot == depth) pslot = 0;
  };
  if (threadIdx.x < rows) {  // thread (m, j): the normalised score of routed expert j of token m
    if (P.normalize) {
      const int m = threadIdx.x / P.k;
      float denom = 0.f;
      for (int jj = 0; jj < P.k; ++jj) denom = bfr(raw[m * P.k + jj] + denom);
      sc_mine = bfr(sc_mine / denom);
    }
    wts[threadIdx.x] = sc_mine;
    if (threadIdx.x < M) gsig[threadIdx.x] = sigmoid_bf_call(gs_mine);
  }
  // widen a loaded piece and put it where the dot will read it (or into the linear copy)
  auto place = [&](bool shared_row, int i, uint2 v) {
    const float4 f = make_float4(bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y));
    if (kDirect) {
      const int K = shared_row ? P.SI : P.I;
      const int m = i / K;
      stage_piece<KIND>(shared_row ? XS : X, m, i - m * K, f);
    } else {
      *reinterpret_cast<float4*>((shared_row ? lin2 : lin) + i) = f;
    }
  };
#pragma unroll
  for (int j = 0; j < kPre; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < rows * P.I) place(false, i, pre[j]);
  }
  for (int i = (threadIdx.x + kPre * blockDim.x) * 4; i < rows * P.I; i += blockDim.x * 4)
    place(false, i, __ldg(reinterpret_cast<const uint2*>(P.act + i)));
  if (threadIdx.x * 4 < M * P.SI) place(true, threadIdx.x * 4, spre);
  for (int i = (threadIdx.x + blockDim.x) * 4; i < M * P.SI; i += blockDim.x * 4)
    place(true, i, __ldg(reinterpret_cast<const uint2*>(P.sact + i)));
  if (kDirect) {
    stage_zero_tail<KIND>(X);
    stage_zero_tail<KIND>(XS);
  } else {
    __syncthreads();
    stage_fill<KIND>(lin, P.I, X);
    stage_fill<KIND>(lin2, P.SI, XS);
  }
  __syncthreads();
  int slot = 0, round = 0;
  uint32_t parity = 0;
  bool ok = true;  // a wait that ran out: no more waits or stores, but the pair's barriers are kept
  for (int cg = gp; cg < total; cg += GP, ++round) {
    const int m = by_ngroups(cg), grp = cg - m * ngroups;
    const int c0 = grp * RT;
    float acc = 0.f;                               // even warp: the running combine value
    float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;  // odd warp: its routed terms, newest in t3
    float sh = 0.f;
    int which = 0;
    for (int q = 0; q < nt; ++q) {
      ok = ok && ring_wait(R, slot, parity);
      const uint8_t* buf = R.buf + (size_t)slot * slot_bytes;
      float d[RT];
#pragma unroll
      for (int r = 0; r < RT; ++r) d[r] = 0.f;
      const int j = (h ? k0 : 0) + q;
      const bool routed = j < P.k;  // one copy of the dot serves the routed and the shared tile
      if (ok) tile_dot<KIND, 1, RT>(buf, routed ? P.down : P.sh_down, routed ? X : XS, routed ? m * P.k + j : m, lane, d);
      __syncwarp();
      if (pg < total && ok) {
        if (lane == 0) fence_proxy_async();
        issue();
      }
      const float v = rs_butterfly<RT>(d, lane, which);
      if (!routed) sh = bfr(gsig[m] * bfr(v));
      else if (h == 0) acc = bfr(bfr(bfr(v) * wts[m * P.k + j]) + acc);
      else { t0 = t1; t1 = t2; t2 = t3; t3 = bfr(bfr(v) * wts[m * P.k + j]); }
      if (++slot == depth) { slot = 0; parity ^= 1; }
    }
    float* cell = xch + ((size_t)(round & 1) * npairs + pair) * 32 + lane;
    if (h == 0) *cell = acc;
    asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");  // the two warps of the pair
    if (h == 1) {
      acc = *cell;
      const int mine = nt - 1;  // routed terms of this warp, oldest first
      if (mine >= 4) acc = bfr(t0 + acc);
      if (mine >= 3) acc = bfr(t1 + acc);
      if (mine >= 2) acc = bfr(t2 + acc);
      if (mine >= 1) acc = bfr(t3 + acc);
      const int c = c0 + which;
      if (ok && (lane & (32 / RT - 1)) == 0 && c < P.H) P.out[(size_t)m * P.H + c] = f2bf(acc + sh);
    }
  }
}

// ---------------------------------------------------------------------------
// kernel 4: gated-delta front end + recurrence in one launch
// ---------------------------------------------------------------------------
struct GdnParams {
  const bf16_t* conv;   // [S + T][D]: cached window rows then this call's qkv rows
  const bf16_t* cw;     // [D][Kc]
  const bf16_t* a_in;   // [T][Hv]
  const bf16_t* b_in;   // [T][Hv]
  const bf16_t* a_log;  // [Hv]
  const bf16_t* dt_bias;
  float* ring;          // [nring][Hv][128][128]
  const int* cur;
  bf16_t* y;            // [T][Hv][128]
  int T, S, Kc, D, Hk, Hv, nring, final_only;
  float q_scale, k_scale, eps;
  // optional epilogue: rms_norm_gated of the outputs (kernels/ornith_norm.metal:119-185) by the
  // last CTA of each head to finish; null `gated_out` leaves y as the only output
  const bf16_t* z;          // [T][Hv*128] gate rows
  const bf16_t* norm_w;     // [128]
  bf16_t* gated_out;        // [T][Hv*128]
  unsigned int* arrivals;   // [Hv], zero between launches
  float norm_eps;
};

constexpr int kGdnRows = 16;
constexpr int kGdnMaxT = 4;

// CTA = (head hv, block of kGdnRows state rows).  Threads 0 .. 4*kGdnRows-1 own the state (a row's
// 128 floats over 4 lanes) and run the recurrence; the front end is spread over one warp per
// (q or k, window token), one warp for the block's value rows and one for the gates, so that its
// out-of-line calls run side by side: 2 T + 2 warps in all.
constexpr int kGdnStateThreads = kGdnRows * 4;
__host__ __device__ constexpr int gdn_threads(int T) { return 32 * (2 * T + 2); }

template <bool TAPS4>  // TAPS4: the convolution has 4 taps (every Qwen3.5 artifact); else any width
__global__ void __launch_bounds__(gdn_threads(kGdnMaxT)) k_gdn(GdnParams p) {
  __shared__ float s_q[kGdnMaxT][128], s_k[kGdnMaxT][128], s_v[kGdnMaxT][kGdnRows];
  __shared__ float s_g[kGdnMaxT], s_beta[kGdnMaxT];
  pdl_trigger();
  const int hv = blockIdx.y;
  const int hk = hv / (p.Hv / p.Hk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int key_dim = p.Hk * 128;
  const bool owner = threadIdx.x < kGdnStateThreads;
  // the state rows do not depend on the front end: request them first so that the 2 MB of HBM
  // reads per layer overlap the convolution and the norms
  const int row = blockIdx.x * kGdnRows + ((threadIdx.x >> 2) & (kGdnRows - 1));
  const int lir = threadIdx.x & 3;
  const size_t ssz = (size_t)p.Hv * 128 * 128;
  const size_t off = ((size_t)hv * 128 + row) * 128 + lir * 32;
  const int cur = *p.cur;
  const float* sin = p.ring + (size_t)(cur % p.nring) * ssz + off;
  float S[32];
  if (owner) {  // a thread's 32 state floats are one 128-byte line: four requests of a whole sector each
#pragma unroll
    for (int i = 0; i < 4; ++i)
      asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                   : "=f"(S[8 * i]), "=f"(S[8 * i + 1]), "=f"(S[8 * i + 2]), "=f"(S[8 * i + 3]), "=f"(S[8 * i + 4]),
                     "=f"(S[8 * i + 5]), "=f"(S[8 * i + 6]), "=f"(S[8 * i + 7])
                   : "l"(sin + 8 * i));
  }
  // The state and the ring position were written by an earlier step (a graph launch, a copy or a
  // host read lies in between), not by the kernel this one may overlap: only what follows reads
  // the previous kernel's output.
  pdl_wait();
  // ---- front end (kernels/gdn_front.metal:65-190)
  if constexpr (TAPS4) {
    if (warp < 2 * p.T) {
      // q (even warps) or k (odd warps) head of window token t: the four window rows and the taps
      // of the lane's four channels are requested together
      const int t = warp >> 1;
      const bool isk = (warp & 1) != 0;
      const int c0 = (isk ? key_dim + hk * 128 : hk * 128) + 4 * lane;
      uint2 xr[4], wr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xr[i] = *reinterpret_cast<const uint2*>(p.conv + (size_t)(t + i) * p.D + c0);
#pragma unroll
      for (int r = 0; r < 4; ++r) wr[r] = *reinterpret_cast<const uint2*>(p.cw + (size_t)(c0 + r) * 4);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float xs[4] = {bf_lo(xr[i].x), bf_hi(xr[i].x), bf_lo(xr[i].y), bf_hi(xr[i].y)};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float tap = i == 0 ? bf_lo(wr[r].x) : i == 1 ? bf_hi(wr[r].x) : i == 2 ? bf_lo(wr[r].y) : bf_hi(wr[r].y);
          acc[r] = fmaf(xs[r], tap, acc[r]);
        }
      }
      float yv[4];
      float sum = 0.f;
#pragma unroll
      for (int r = 0; r < 4; ++r) { yv[r] = silu_bf_call(bfr(acc[r])); sum = fmaf(yv[r], yv[r], sum); }
      sum = warp_sum(sum);
      const float inv = orn_rsqrtf(sum / 128.0f + p.eps);
      const float sc = isk ? p.k_scale : p.q_scale;
      float* dst = isk ? s_k[t] : s_q[t];
#pragma unroll
      for (int r = 0; r < 4; ++r) dst[4 * lane + r] = bfr(sc * bfr(yv[r] * inv));
    } else if (warp == 2 * p.T) {
      // the block's value channels: item = (state row r, window token t)
#pragma unroll 1
      for (int idx = lane; idx < kGdnRows * p.T; idx += 32) {
        const int r = idx & (kGdnRows - 1), t = idx / kGdnRows;
        const int cv = 2 * key_dim + hv * 128 + blockIdx.x * kGdnRows + r;
        bf16_t vr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) vr[i] = p.conv[(size_t)(t + i) * p.D + cv];
        const uint2 vw = *reinterpret_cast<const uint2*>(p.cw + (size_t)cv * 4);
        const float vtap[4] = {bf_lo(vw.x), bf_hi(vw.x), bf_lo(vw.y), bf_hi(vw.y)};
        float av = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) av = fmaf(bf2f(vr[i]), vtap[i], av);
        s_v[t][r] = silu_bf_call(bfr(av));
      }
    } else if (lane < p.T) {
      // the head's gates of window token `lane`
      const size_t i = (size_t)lane * p.Hv + hv;
      const float ga = bf2f(p.a_in[i]), gb = bf2f(p.b_in[i]), gdt = bf2f(p.dt_bias[hv]), gal = bf2f(p.a_log[hv]);
      const float sp = softplus_bf_call(bfr(ga + gdt));
      const float decay = expf_call(gal);
      s_g[lane] = expf_call((-decay) * sp);
      s_beta[lane] = sigmoid_bf_call(gb);
    }
  } else if (warp < 2) {  // any number of taps: warp 0 -> q, warp 1 -> k, then value rows and gates
  for (int t = 0; t < p.T; ++t) {
    const int c0 = (warp == 0 ? hk * 128 : key_dim + hk * 128) + 4 * lane;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < p.Kc; ++i) {
      const uint2 xv = *reinterpret_cast<const uint2*>(p.conv + (size_t)(t + i) * p.D + c0);
      const float xs[4] = {bf_lo(xv.x), bf_hi(xv.x), bf_lo(xv.y), bf_hi(xv.y)};
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[r] = fmaf(xs[r], bf2f(p.cw[(size_t)(c0 + r) * p.Kc + i]), acc[r]);
    }
    float yv[4];
    float sum = 0.f;
#pragma unroll
    for (int r = 0; r < 4; ++r) { yv[r] = silu_bf_call(bfr(acc[r])); sum = fmaf(yv[r], yv[r], sum); }
    sum = warp_sum(sum);
    const float inv = orn_rsqrtf(sum / 128.0f + p.eps);
    const float sc = warp == 0 ? p.q_scale : p.k_scale;
    float* dst = warp == 0 ? s_q[t] : s_k[t];
#pragma unroll
    for (int r = 0; r < 4; ++r) dst[4 * lane + r] = bfr(sc * bfr(yv[r] * inv));
  }
  // value rows of this CTA and the per-head gates
  if (lir == 0) {
    const int c = 2 * key_dim + hv * 128 + row;
    for (int t = 0; t < p.T; ++t) {
      float acc = 0.f;
      for (int i = 0; i < p.Kc; ++i)
        acc = fmaf(bf2f(p.conv[(size_t)(t + i) * p.D + c]), bf2f(p.cw[(size_t)c * p.Kc + i]), acc);
      s_v[t][threadIdx.x >> 2] = silu_bf_call(bfr(acc));
    }
  }
  if (threadIdx.x < p.T) {
    const int t = threadIdx.x;
    const size_t i = (size_t)t * p.Hv + hv;
    const float sp = softplus_bf_call(bfr(bf2f(p.a_in[i]) + bf2f(p.dt_bias[hv])));
    const float decay = expf_call(bf2f(p.a_log[hv]));
    s_g[t] = expf_call((-decay) * sp);
    s_beta[t] = sigmoid_bf_call(bf2f(p.b_in[i]));
  }
    }
  __syncthreads();
  // ---- recurrence (kernels/gated_delta.metal:36-142), by the threads that own the state
  if (owner)
  for (int t = 0; t < p.T; ++t) {
    const float* kf = s_k[t] + lir * 32;
    const float* qf = s_q[t] + lir * 32;
    const float gt = s_g[t], bt = s_beta[t], vt = s_v[t][threadIdx.x >> 2];
    float part[8];
#pragma unroll
    for (int pb = 0; pb < 8; ++pb) {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = pb * 4 + i;
        S[e] = S[e] * gt;
        acc = fmaf(S[e], kf[e], acc);
      }
      part[pb] = acc;
    }
    float kv = ((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]));
    kv = kv + __shfl_xor_sync(0xffffffffu, kv, 1);
    kv = kv + __shfl_xor_sync(0xffffffffu, kv, 2);
    const float delta = (vt - kv) * bt;
#pragma unroll
    for (int pb = 0; pb < 8; ++pb) {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = pb * 4 + i;
        S[e] = fmaf(kf[e], delta, S[e]);
        acc = fmaf(S[e], qf[e], acc);
      }
      part[pb] = acc;
    }
    float o = ((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]));
    o = o + __shfl_xor_sync(0xffffffffu, o, 1);
    o = o + __shfl_xor_sync(0xffffffffu, o, 2);
    if (lir == 0) p.y[((size_t)t * p.Hv + hv) * 128 + row] = f2bf(o);
    float* sout = nullptr;
    if (!p.final_only) sout = p.ring + (size_t)((cur + 1 + t) % p.nring) * ssz + off;
    else if (t + 1 == p.T) sout = p.ring + (size_t)((cur + 1) % p.nring) * ssz + off;
    if (sout != nullptr) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(sout + 8 * i), "f"(S[8 * i]),
                     "f"(S[8 * i + 1]), "f"(S[8 * i + 2]), "f"(S[8 * i + 3]), "f"(S[8 * i + 4]), "f"(S[8 * i + 5]),
                     "f"(S[8 * i + 6]), "f"(S[8 * i + 7])
                     : "memory");
    }
  }
  if (p.gated_out == nullptr) return;
  // The 128 / kGdnRows CTAs of a head each wrote their rows of y.  The last of them to get here
  // normalises the head (one warp per window row, the arithmetic of the stand-alone
  // rms_norm_gated) and resets the head's counter for the next launch.
  __shared__ unsigned int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(p.arrivals + hv, 1u);
    s_last = (prev == gridDim.x - 1) ? 1u : 0u;
    if (s_last) atomicExch(p.arrivals + hv, 0u);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const uint2 wv = __ldg(reinterpret_cast<const uint2*>(p.norm_w + 4 * lane));
  const float wf[4] = {bf_lo(wv.x), bf_hi(wv.x), bf_lo(wv.y), bf_hi(wv.y)};
  for (int t = warp; t < p.T; t += (blockDim.x >> 5)) {
    const size_t base = ((size_t)t * p.Hv + hv) * 128 + 4 * lane;
    const uint2 a2 = __ldcg(reinterpret_cast<const uint2*>(p.y + base));  // written by other CTAs: read through L2
    const uint2 z2 = __ldg(reinterpret_cast<const uint2*>(p.z + base));
    const float xv[4] = {bf_lo(a2.x), bf_hi(a2.x), bf_lo(a2.y), bf_hi(a2.y)};
    const float gz[4] = {bf_lo(z2.x), bf_hi(z2.x), bf_lo(z2.y), bf_hi(z2.y)};
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc = fmaf(xv[i], xv[i], acc);
    acc = warp_sum(acc);
    const float iv = orn_rsqrtf(acc / 128.0f + p.norm_eps);
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float normed = bfr(wf[i] * bfr(xv[i] * iv));
      float g = gz[i];
      g = g * sigmoid_f32_call(g);
      o[i] = f2bf(g * normed);
    }
    uint2 ov;
    ov.x = o[0] | (o[1] << 16);
    ov.y = o[2] | (o[3] << 16);
    *reinterpret_cast<uint2*>(p.gated_out + base) = ov;
  }
}

// ---------------------------------------------------------------------------
// kernel 5: q/k norm + rotary + KV append + attention + output gate
// ---------------------------------------------------------------------------
struct AttnParams {
  const bf16_t* qg;      // [T][Hq][2*256]: query | gate
  const bf16_t* k;       // [T][Hkv][256]
  const bf16_t* v;       // [T][Hkv][256]
  const bf16_t* q_norm;  // [256]
  const bf16_t* k_norm;  // [256]
  bf16_t* kc;            // [Hkv][cap][256]
  bf16_t* vc;
  const int* pos;
  bf16_t* out;           // [T][Hq*256] gated attention output
  int T, Hq, Hkv, cap, rope_dims;
  float lnb, scale, eps;
};

// norm + rope of one 256-wide head row by one warp (8 dims per lane); the
// result (bfloat16 values as floats) goes to dst[256]
ORN_D void warp_norm_rope(const bf16_t* src, const bf16_t* w, float eps, int rope_dims, float lnb, int position,
                          float* dst, float* red /*[2]*/, int lane) {
  // rms over 256 = 64 virtual threads of 4 -> two virtual warps
  float xv[8];
  widen8(ldg128(src + 8 * lane), xv);
  // lane holds elements 8l..8l+7 = virtual threads 2l, 2l+1; virtual warp = (2l+j)/32
  float a0 = 0.f, a1 = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) { a0 = fmaf(xv[i], xv[i], a0); a1 = fmaf(xv[4 + i], xv[4 + i], a1); }
  // virtual warp 0 = lanes 0..15 (both halves), virtual warp 1 = lanes 16..31.  Its butterfly over
  // virtual lanes (xor 16,8,4,2,1 of the virtual index 2l+j) is: xor 8,4,2,1 across lanes, then j.
  // virtual index v = 2*(lane&15) + j; xor 16 <-> lane xor 8; xor 8 <-> lane xor 4; xor 4 <-> lane xor 2;
  // xor 2 <-> lane xor 1; xor 1 <-> j.
  float b0 = a0 + __shfl_xor_sync(0xffffffffu, a0, 8);
  float b1 = a1 + __shfl_xor_sync(0xffffffffu, a1, 8);
  b0 = b0 + __shfl_xor_sync(0xffffffffu, b0, 4); b1 = b1 + __shfl_xor_sync(0xffffffffu, b1, 4);
  b0 = b0 + __shfl_xor_sync(0xffffffffu, b0, 2); b1 = b1 + __shfl_xor_sync(0xffffffffu, b1, 2);
  b0 = b0 + __shfl_xor_sync(0xffffffffu, b0, 1); b1 = b1 + __shfl_xor_sync(0xffffffffu, b1, 1);
  const float vw = b0 + b1;  // sum of this lane's virtual warp
  const float other = __shfl_xor_sync(0xffffffffu, vw, 16);
  const float w0 = lane < 16 ? vw : other, w1 = lane < 16 ? other : vw;
  // second level: butterfly of [w0, w1, 0, ...] = w0 + w1 after exact additions of zero
  const float total = (w0 + 0.f) + (w1 + 0.f);
  (void)red;
  const float inv = orn_rsqrtf(total / 256.0f + eps);
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[8 * lane + i] = bfr(bf2f(w[8 * lane + i]) * bfr(xv[i] * inv));
  __syncwarp();
  const int half = rope_dims / 2;
  for (int i = lane; i < half; i += 32) {
    const float inv_freq = expf_call(-(float)i * lnb);
    const float ang = (float)position * inv_freq;
    float sn, cs;
    sincosf_call(ang, &sn, &cs);
    const float x1 = dst[i], x2 = dst[i + half];
    const float t1 = x2 * sn, t2 = x2 * cs;
    dst[i] = bfr(fmaf(x1, cs, -t1));
    dst[i + half] = bfr(fmaf(x1, sn, t2));
  }
  __syncwarp();
}

// One key group's walk over the cache (keys grp, grp + 32, ... < L in ascending order): the online
// softmax of kernels/sdpa.metal per key, unchanged.  Keys are taken KB at a time: their cache rows are
// requested together, their dot products and butterflies run side by side, and only the (max, sum,
// out) update of each key waits for the one before it, so a memory round trip and the shuffle latency
// are paid once per KB keys.  The arithmetic of a key and the order of the keys are those of KB = 1.
template <int KB>
ORN_D void attn_walk(const AttnParams& p, const float (*s_knew)[256], const float* qs, int grp, int L, int pos, int kvh, int lane,
                     float* o, float& mx, float& sm) {
  constexpr int HD = 256;
  uint4 kr[KB], vr[KB];
  auto fetch_k = [&](int n, uint4& kq) {
    if (n < pos) kq = *reinterpret_cast<const uint4*>(p.kc + ((size_t)kvh * p.cap + n) * HD + 8 * lane);
  };
  auto fetch_v = [&](int n, uint4& vq) {
    if (n >= pos) vq = ldg128(p.v + ((size_t)(n - pos) * p.Hkv + kvh) * HD + 8 * lane);
    else vq = *reinterpret_cast<const uint4*>(p.vc + ((size_t)kvh * p.cap + n) * HD + 8 * lane);
  };
  auto dot = [&](int n, const uint4& kq) {
    float kf[8];
    if (n >= pos) {
#pragma unroll
      for (int i = 0; i < 8; ++i) kf[i] = s_knew[n - pos][8 * lane + i];
    } else {
      widen8(kq, kf);
    }
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(qs[i], kf[i], acc);
    return acc;
  };
  // one key folded in; expf inline: a call would make the warp wait for every cache row it has in flight
  auto fold = [&](float score, const uint4& vq) {
    float vf[8];
    widen8(vq, vf);
    const float nm = fmaxf(mx, score);
    const float factor = orn_expf(mx - nm);
    const float e = orn_expf(score - nm);
    mx = nm;
    sm = fmaf(sm, factor, e);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = fmaf(o[i], factor, e * vf[i]);
  };
#pragma unroll
  for (int j = 0; j < KB; ++j) {
    kr[j] = make_uint4(0u, 0u, 0u, 0u);
    vr[j] = kr[j];
    if (grp + 32 * j < L) { fetch_k(grp + 32 * j, kr[j]); fetch_v(grp + 32 * j, vr[j]); }
  }
  int n0 = grp;
  // whole blocks: straight-line code, so the KB butterflies and the 2 KB exponentials overlap
  for (; n0 + 32 * (KB - 1) < L; n0 += 32 * KB) {
    float score[KB];
    uint4 vcur[KB];
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      score[j] = dot(n0 + 32 * j, kr[j]);
      vcur[j] = vr[j];
    }
#pragma unroll
    for (int j = 0; j < KB; ++j) {  // the next block's rows while this block is folded in
      const int n = n0 + 32 * (KB + j);
      if (n < L) { fetch_k(n, kr[j]); fetch_v(n, vr[j]); }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
      for (int j = 0; j < KB; ++j) score[j] = score[j] + __shfl_xor_sync(0xffffffffu, score[j], off);
#pragma unroll
    for (int j = 0; j < KB; ++j) fold(score[j], vcur[j]);
  }
  // the keys of the last, partial block one by one (their rows are already here)
#pragma unroll
  for (int j = 0; j < KB - 1; ++j) {
    const int n = n0 + 32 * j;
    if (n < L) fold(warp_sum(dot(n, kr[j])), vr[j]);
  }
}

__global__ void __launch_bounds__(1024) k_attn(AttnParams p) {
  constexpr int HD = 256;
  __shared__ float s_o[32][HD];
  __shared__ float s_q[HD];
  __shared__ float s_knew[kGdnMaxT][HD];
  __shared__ float s_max[32], s_sum[32], s_f[32];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, r = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = p.Hq / p.Hkv;
  const int kvh = h / group;
  const int pos = *p.pos;
  if (warp == 0)
    warp_norm_rope(p.qg + ((size_t)r * p.Hq + h) * 2 * HD, p.q_norm, p.eps, p.rope_dims, p.lnb, pos + r, s_q, nullptr, lane);
  else if (warp <= p.T)
    warp_norm_rope(p.k + ((size_t)(warp - 1) * p.Hkv + kvh) * HD, p.k_norm, p.eps, p.rope_dims, p.lnb, pos + warp - 1,
                   s_knew[warp - 1], nullptr, lane);
  __syncthreads();
  // one CTA per kv head appends the window's keys and values to the cache
  if (r == 0 && (h % group) == 0) {
    for (int i = threadIdx.x; i < p.T * HD; i += blockDim.x) {
      const int t = i / HD, d = i - t * HD;
      if (pos + t < p.cap) {
        p.kc[((size_t)kvh * p.cap + pos + t) * HD + d] = f2bf(s_knew[t][d]);
        p.vc[((size_t)kvh * p.cap + pos + t) * HD + d] = p.v[((size_t)t * p.Hkv + kvh) * HD + d];
      }
    }
  }
  int L = pos + r + 1;
  if (L > p.cap) L = p.cap;
  float qs[8], o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { qs[i] = s_q[8 * lane + i] * p.scale; o[i] = 0.f; }
  float mx = -INFINITY, sm = 0.f;
  attn_walk<2>(p, s_knew, qs, warp, L, pos, kvh, lane, o, mx, sm);
  if (lane == 0) { s_max[warp] = mx; s_sum[warp] = sm; }
#pragma unroll
  for (int i = 0; i < 8; ++i) s_o[warp][8 * lane + i] = o[i];
  __syncthreads();
  if (warp == 0) {
    const float M = warp_max(s_max[lane]);
    const float f = expf_call(s_max[lane] - M);
    s_f[lane] = f;
    const float S = warp_sum(s_sum[lane] * f);
    if (lane == 0) s_sum[0] = S;
  }
  __syncthreads();
  if (threadIdx.x < HD) {
    const int d = threadIdx.x;
    float a[32];
#pragma unroll
    for (int g = 0; g < 32; ++g) a[g] = s_o[g][d] * s_f[g];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
      for (int i = 0; i < off; ++i) a[i] = a[i] + a[i + off];
    const float att = bfr(a[0] / s_sum[0]);
    const float gate = bf2f(p.qg[((size_t)r * p.Hq + h) * 2 * HD + HD + d]);
    p.out[((size_t)r * p.Hq + h) * HD + d] = f2bf(sigmoid_bf_call(gate) * att);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
constexpr size_t kSmemBudget = 220 * 1024;

// launch label for the per-kernel time report (ORN_KTIME=1): kernel, rows, first job's shape
std::mutex g_grant_mu;  // guards the label pool below and the table of shared-memory grants
const char* launch_label(orn_ctx* ctx, const char* kern, int M, int kind, int O, int K) {
  if (!ctx->kt) return kern;
  static std::set<std::string> pool;
  std::lock_guard<std::mutex> lock(g_grant_mu);
  char buf[96];
  snprintf(buf, sizeof buf, "%s M=%d kind=%d %dx%d", kern, M, kind, O, K);
  return pool.insert(buf).first->c_str();
}

// raise a kernel's dynamic shared-memory limit once per (device, kernel): the attribute belongs to
// the kernel's image on one device, and contexts of several devices (or host threads) share this table
std::set<std::pair<int, const void*>> g_granted;  // (device, kernel address); instantiations share a type
template <typename Kern>
int grant_smem(orn_ctx* ctx, Kern kern, size_t bytes) {
  const std::pair<int, const void*> key(ctx->device, reinterpret_cast<const void*>(kern));
  std::lock_guard<std::mutex> lock(g_grant_mu);
  if (g_granted.count(key)) return ORN_OK;
  ORN_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  g_granted.insert(key);
  return ORN_OK;
}
template <typename Kern>
int set_smem(orn_ctx* ctx, Kern kern, size_t bytes) {
  if (bytes > 227 * 1024) ORN_FAIL(ctx, ORN_ERR_ARG, "fused kernel: staged activations exceed shared memory");
  if (bytes > 48 * 1024) return grant_smem(ctx, kern, 227 * 1024);
  return ORN_OK;
}

// rings beside `fixed` bytes of stages and scratch: offset of the rings, their depth, the launch's
// dynamic shared memory
int plan_smem(orn_ctx* ctx, size_t fixed, uint32_t slot_bytes, int nwarps, int* depth, uint32_t* ring_off, size_t* total) {
  fixed = (fixed + 127) & ~(size_t)127;
  int d = 8;
  while (d > 1 && fixed + ring_bytes(nwarps, d, slot_bytes) > kSmemBudget) --d;
  *depth = d;
  *ring_off = (uint32_t)fixed;
  *total = fixed + ring_bytes(nwarps, d, slot_bytes) + 128;
  if (*total > 227 * 1024) ORN_FAIL(ctx, ORN_ERR_ARG, "fused kernel: rows too long for the shared-memory rings");
  return ORN_OK;
}

template <int M, int MASK, int KC>
int launch_norm_gemv_mask(orn_ctx* ctx, cudaStream_t s, const Prologue& P, const RowJobs& J, uint32_t slot) {
  size_t fixed = 0;
  for (int k = 0; k < 4; ++k)
    if (MASK & (1 << k)) fixed += stage_floats(k, M, P.K) * sizeof(float);
  fixed = (fixed + 127) & ~(size_t)127;
  const size_t stages = fixed;
  const bool direct = P.mode == PRO_ADDNORM || P.mode == PRO_PLAIN;  // staged from registers: no linear copy of the rows
  const size_t scratch = ((direct ? 0 : (size_t)M * P.K) + M * 33 + 64) * sizeof(float);
  fixed += scratch;
  int depth, late = 0;
  uint32_t ring_off;
  size_t bytes;
  int rc = plan_smem(ctx, fixed, slot, kFusedThreads / 32, &depth, &ring_off, &bytes);
  if (rc != ORN_OK || depth < 2) {
    // too little room for two slots per warp beside the scratch: run the rings over it
    rc = plan_smem(ctx, stages, slot, kFusedThreads / 32, &depth, &ring_off, &bytes);
    if (bytes < stages + scratch + 256) bytes = stages + scratch + 256;
    late = 1;
  }
  if (rc != ORN_OK) return rc;
  rc = set_smem(ctx, k_norm_gemv<M, MASK, KC>, bytes);
  if (rc != ORN_OK) return rc;
  ORN_CHECK_CUDA(ctx, orn_launch_dependent(ctx, s, 0, k_norm_gemv<M, MASK, KC>, dim3(ctx->sm_count), dim3(kFusedThreads),
                                           bytes, P, J, slot, depth, ring_off, late, ctx->dev_err));
  return orn_launch_check(ctx, launch_label(ctx, "k_norm_gemv", M, J.job[0].lin.kind, J.job[0].lin.O, P.K));
}

template <int M, int KC>
int launch_norm_gemv_kc(orn_ctx* ctx, cudaStream_t s, const Prologue& P, const RowJobs& J, uint32_t slot) {
  // one instantiation per set of formats present, so that a kernel carries only the code it runs
  switch (J.kinds_mask) {
    case 1: return launch_norm_gemv_mask<M, 1, KC>(ctx, s, P, J, slot);
    case 2: return launch_norm_gemv_mask<M, 2, KC>(ctx, s, P, J, slot);
    case 4: return launch_norm_gemv_mask<M, 4, KC>(ctx, s, P, J, slot);
    case 8: return launch_norm_gemv_mask<M, 8, KC>(ctx, s, P, J, slot);
    case 5: return launch_norm_gemv_mask<M, 5, KC>(ctx, s, P, J, slot);    // Q4_K + affine-8
    case 12: return launch_norm_gemv_mask<M, 12, KC>(ctx, s, P, J, slot);  // affine-8 + bf16
    case 9: return launch_norm_gemv_mask<M, 9, KC>(ctx, s, P, J, slot);    // Q4_K + bf16
    case 6: return launch_norm_gemv_mask<M, 6, KC>(ctx, s, P, J, slot);    // Q6_K + affine-8
    default: return launch_norm_gemv_mask<M, 15, KC>(ctx, s, P, J, slot);
  }
}

template <int M>
int launch_norm_gemv(orn_ctx* ctx, cudaStream_t s, const Prologue& P, RowJobs& J) {
  J.kinds_mask = 0;
  J.total = 0;
  uint32_t slot = 0;
  if (P.mode == PRO_ADDNORM && P.K > 4 * kAddNormGroups * kFusedThreads)
    ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: hidden size above 2048 is not supported by the norm prologue");
  if (P.K % 256) ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: K must be a multiple of 256");
  const int kc = P.K > 2048 ? 2 : 1;  // rows of 512 weights or fewer run with the class-1 tile heights
  for (int j = 0; j < J.njobs; ++j) {
    RowJob& job = J.job[j];
    J.kinds_mask |= 1 << job.lin.kind;
    if (job.lin.K != P.K) ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: weight K differs from the staged row");
    if (job.epi == EPI_SWIGLU &&
        (job.lin2.kind != job.lin.kind || job.lin2.K != job.lin.K || job.lin2.O != job.lin.O))
      ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: gate and up projections must share format and shape");
    const int rows = tile_rows(job.lin.kind, kc);
    if (job.epi == EPI_SWIGLU && rows < 2)
      ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: rows too long for a gate/up tile pair");
    const int per_tile = job.epi == EPI_SWIGLU ? rows / 2 : rows;
    job.tiles = (job.lin.O + per_tile - 1) / per_tile;
    J.total += job.tiles;
    const uint32_t bytes = (uint32_t)rows * job.lin.rec;
    slot = bytes > slot ? bytes : slot;
  }
  if (kc == 2) return launch_norm_gemv_kc<M, 2>(ctx, s, P, J, slot);
  return launch_norm_gemv_kc<M, 1>(ctx, s, P, J, slot);
}

template <int KIND, int KC>
int launch_moe_up_k(orn_ctx* ctx, cudaStream_t s, const MoeUpParams& P) {
  const int M = P.M;
  size_t fixed = stage_floats(KIND, M, P.H) * sizeof(float) + (size_t)M * P.k * 4;
  fixed = (fixed + 127) & ~(size_t)127;
  fixed += ((size_t)M * P.H + (size_t)M * P.E + M * 32 + M * P.k + 8) * sizeof(float);
  const uint32_t slot = up_rows(KIND, KC) * P.gate.rec;
  int depth;
  uint32_t ring_off;
  size_t bytes;
  int rc = plan_smem(ctx, fixed, slot, kMoeThreads / 32, &depth, &ring_off, &bytes);
  if (rc != ORN_OK) return rc;
  rc = set_smem(ctx, k_moe_up<KIND, KC>, bytes);
  if (rc != ORN_OK) return rc;
  ORN_CHECK_CUDA(ctx, orn_launch_dependent(ctx, s, 1, k_moe_up<KIND, KC>, dim3(ctx->sm_count), dim3(kMoeThreads), bytes,
                                           P, slot, depth, ring_off, ctx->dev_err));
  return orn_launch_check(ctx, launch_label(ctx, "k_moe_up", M, KIND, P.I, P.H));
}

template <int KIND, int KC>
int launch_moe_down_k(orn_ctx* ctx, cudaStream_t s, const MoeDownParams& P) {
  const int M = P.M;
  const int rows = M * P.k;
  size_t fixed = (stage_floats(KIND, rows, P.I) + stage_floats(KIND, M, P.SI) + 3 * rows + M + 2 * (kDownThreads / 64) * 32) * sizeof(float);
  fixed = (fixed + 127) & ~(size_t)127;
  if (kind_ns(KIND) != 0)  // formats with per-unit sums stage through a linear copy of the rows
    fixed += ((size_t)rows * P.I + (size_t)M * P.SI + 8) * sizeof(float);
  const uint32_t r0 = moe_rows(KIND, KC) * P.down.rec, r1 = moe_rows(KIND, KC) * P.sh_down.rec;
  const uint32_t slot = r0 > r1 ? r0 : r1;
  int depth;
  uint32_t ring_off;
  size_t bytes;
  int rc = plan_smem(ctx, fixed, slot, kDownThreads / 32, &depth, &ring_off, &bytes);
  if (rc != ORN_OK) return rc;
  rc = set_smem(ctx, k_moe_down<KIND, KC>, bytes);
  if (rc != ORN_OK) return rc;
  ORN_CHECK_CUDA(ctx, orn_launch_dependent(ctx, s, 2, k_moe_down<KIND, KC>, dim3(ctx->sm_count), dim3(kDownThreads), bytes,
                                           P, slot, depth, ring_off, ctx->dev_err));
  return orn_launch_check(ctx, launch_label(ctx, "k_moe_down", M, KIND, P.H, P.I));
}


// Probe of the give-up path: one warp sets up a ring like every streaming kernel, requests no copy
// at all and waits on the empty slot with a short limit.  Nothing is in flight when the wait runs
// out, so the kernel simply records the failure (as the streaming kernels do) and returns.
__global__ void k_wait_probe(uint32_t rounds, int* err, int* waited_out) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Ring R;
  ring_setup(R, smem_raw, 128, 1, err);
  R.limit = rounds;
  __syncwarp();
  const bool ok = ring_wait(R, 0, 0);
  if ((threadIdx.x & 31) == 0) *waited_out = ok ? 1 : 0;
}
}  // namespace

int f_norm_gemv(orn_ctx* ctx, cudaStream_t s, int M, const FusedPrologue& fp, const FusedJob* jobs, int njobs) {
  if (njobs < 1 || njobs > 4) ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: 1..4 jobs");
  Prologue P;
  P.mode = fp.mode; P.K = fp.K; P.a = fp.a; P.b = fp.b; P.w = fp.w; P.w2 = fp.w2; P.sum_out = fp.sum_out;
  P.norm_out = fp.norm_out; P.ids = fp.ids; P.eps = fp.eps;
  P.emb = fp.emb ? lin_dev(fp.emb) : LinDev{0, 0, 0, 0, nullptr, nullptr, nullptr, 0};
  RowJobs J;
  J.njobs = njobs;
  for (int j = 0; j < njobs; ++j) {
    J.job[j].lin = lin_dev(jobs[j].lin);
    J.job[j].lin2 = jobs[j].lin2 ? lin_dev(jobs[j].lin2) : J.job[j].lin;
    J.job[j].out = jobs[j].out;
    J.job[j].epi = jobs[j].epi;
  }
  switch (M) {
    case 1: return launch_norm_gemv<1>(ctx, s, P, J);
    case 2: return launch_norm_gemv<2>(ctx, s, P, J);
    case 3: return launch_norm_gemv<3>(ctx, s, P, J);
    case 4: return launch_norm_gemv<4>(ctx, s, P, J);
  }
  ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: 1..4 rows");
}

int f_moe_up(orn_ctx* ctx, cudaStream_t s, int M, const bf16_t* logits, const bf16_t* x, const orn_linear* gate,
             const orn_linear* up, int k, uint32_t* inds, bf16_t* scores, bf16_t* act) {
  if (gate->kind != up->kind || gate->K != up->K || gate->O != up->O)
    ORN_FAIL(ctx, ORN_ERR_ARG, "moe: gate and up experts must share format and shape");
  if (M < 1 || M > 4) ORN_FAIL(ctx, ORN_ERR_ARG, "moe_up: 1..4 rows");
  MoeUpParams P;
  P.logits = logits; P.x = x; P.gate = lin_dev(gate); P.up = lin_dev(up); P.inds = inds; P.scores = scores;
  P.act = act; P.M = M; P.E = gate->E; P.k = k; P.H = gate->K; P.I = gate->O;
  if (P.E > 512) ORN_FAIL(ctx, ORN_ERR_ARG, "moe: more than 512 experts");
  if (P.H % 256) ORN_FAIL(ctx, ORN_ERR_ARG, "moe_up: hidden must be a multiple of 256");
  if (P.H > 4096) ORN_FAIL(ctx, ORN_ERR_ARG, "moe_up: hidden above 4096");
#define ORN_UP(KIND) \
  return P.H > 2048 ? launch_moe_up_k<KIND, 2>(ctx, s, P) : launch_moe_up_k<KIND, 1>(ctx, s, P)
  switch (gate->kind) {
    case ORN_Q4K: ORN_UP(ORN_Q4K);
    case ORN_Q6K: ORN_UP(ORN_Q6K);
    case ORN_A8: ORN_UP(ORN_A8);
    default: ORN_UP(ORN_BF16);
  }
#undef ORN_UP
}

int f_moe_down(orn_ctx* ctx, cudaStream_t s, int M, const bf16_t* act, const bf16_t* sact, const uint32_t* inds,
               const bf16_t* scores, const bf16_t* gs, const orn_linear* down, const orn_linear* sh_down, int k,
               int normalize, bf16_t* out) {
  if (down->kind != sh_down->kind) ORN_FAIL(ctx, ORN_ERR_ARG, "moe: routed and shared down projections must share a format");
  if (M < 1 || M > 4) ORN_FAIL(ctx, ORN_ERR_ARG, "moe_down: 1..4 rows");
  MoeDownParams P;
  P.act = act; P.sact = sact; P.inds = inds; P.scores = scores; P.gs = gs; P.down = lin_dev(down);
  P.sh_down = lin_dev(sh_down); P.out = out; P.M = M; P.k = k; P.H = down->O; P.I = down->K; P.SI = sh_down->K;
  P.normalize = normalize;
  if (k > 8) ORN_FAIL(ctx, ORN_ERR_ARG, "moe: top_k above 8");
  if (P.I % 256 || P.SI % 256) ORN_FAIL(ctx, ORN_ERR_ARG, "moe_down: intermediate sizes must be multiples of 256");
  const int big = P.I > P.SI ? P.I : P.SI;
  if (big > 2048) ORN_FAIL(ctx, ORN_ERR_ARG, "moe_down: intermediate size above 2048");
#define ORN_DN(KIND) \
  return big > 512 ? launch_moe_down_k<KIND, 1>(ctx, s, P) : launch_moe_down_k<KIND, 0>(ctx, s, P)
  switch (down->kind) {
    case ORN_Q4K: ORN_DN(ORN_Q4K);
    case ORN_Q6K: ORN_DN(ORN_Q6K);
    case ORN_A8: ORN_DN(ORN_A8);
    default: ORN_DN(ORN_BF16);
  }
#undef ORN_DN
}

int f_gdn(orn_ctx* ctx, cudaStream_t s, const bf16_t* conv, const bf16_t* cw, const bf16_t* a, const bf16_t* b,
          const bf16_t* a_log, const bf16_t* dt_bias, float* ring, int nring, const int* cur, int final_only, int T,
          int Hk, int Hv, int Kc, float eps, bf16_t* y, const bf16_t* z, const bf16_t* norm_w, float norm_eps,
          bf16_t* gated_out) {
  if (T > kGdnMaxT) ORN_FAIL(ctx, ORN_ERR_ARG, "fused gdn: at most 4 rows");
  if (!final_only && T + 1 > nring) ORN_FAIL(ctx, ORN_ERR_ARG, "fused gdn: window wider than the state ring");
  GdnParams p;
  p.conv = conv; p.cw = cw; p.a_in = a; p.b_in = b; p.a_log = a_log; p.dt_bias = dt_bias; p.ring = ring;
  p.cur = cur; p.y = y; p.T = T; p.S = Kc - 1; p.Kc = Kc; p.D = 2 * Hk * 128 + Hv * 128; p.Hk = Hk; p.Hv = Hv;
  p.nring = nring; p.final_only = final_only;
  const float inv_scale = 1.0f / sqrtf(128.0f);
  p.q_scale = bfr(inv_scale * inv_scale);
  p.k_scale = bfr(inv_scale);
  p.eps = eps;
  p.z = z; p.norm_w = norm_w; p.gated_out = gated_out; p.norm_eps = norm_eps;
  p.arrivals = reinterpret_cast<unsigned int*>(ctx->dev_err) + 64;
  if (gated_out != nullptr && Hv > 512) ORN_FAIL(ctx, ORN_ERR_ARG, "fused gdn: more than 512 value heads");
  dim3 grid(128 / kGdnRows, Hv);
  const dim3 block(gdn_threads(T));
  // Unused dynamic shared memory caps the kernel at two CTAs per SM.  As a programmatic dependent
  // its CTAs become resident while the previous kernel drains, and without the cap the first SMs
  // to come free would take sixteen CTAs each instead of the grid spreading over the whole part.
  const size_t pad = 100 * 1024;
  // the kernel also has static shared memory: ask for the pad, not for the maximum
  {
    int rc = Kc == 4 ? grant_smem(ctx, k_gdn<true>, pad) : grant_smem(ctx, k_gdn<false>, pad);
    if (rc != ORN_OK) return rc;
  }
  if (Kc == 4) ORN_CHECK_CUDA(ctx, orn_launch_dependent(ctx, s, 3, k_gdn<true>, grid, block, pad, p));
  else ORN_CHECK_CUDA(ctx, orn_launch_dependent(ctx, s, 3, k_gdn<false>, grid, block, pad, p));
  return orn_launch_check(ctx, "k_gdn");
}

// The same attention with the 32 key groups of a (head, row) spread over kAttnSplit CTAs of 8 warps:
// at long contexts one CTA of 32 warps is bound by its own issue slots (every group walks L / 32 keys)
// while most SMs idle.  A group's arithmetic is unchanged (group = key index mod 32, keys in ascending
// order), the partials (max, sum, out[256]) of all 32 groups go through global memory, and the CTA that
// stores the last of them runs the same merge: the result has the bits of the one-CTA kernel.
constexpr int kAttnSplit = 4;
constexpr int kAttnMaxHeads = 128;
constexpr int kAttnPart = 260;  // floats per group partial: out[256], max, sum, pad
__global__ void __launch_bounds__(256) k_attn_split(AttnParams p, float* part, int* arrivals) {
  constexpr int HD = 256;
  __shared__ float s_o[32][HD];
  __shared__ float s_q[HD];
  __shared__ float s_knew[kGdnMaxT][HD];
  __shared__ float s_max[32], s_sum[32], s_f[32];
  __shared__ int s_last;
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, r = blockIdx.y, z = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = 8 * z + warp;  // this warp's key group
  const int group = p.Hq / p.Hkv;
  const int kvh = h / group;
  const int pos = *p.pos;
  if (warp == 0)
    warp_norm_rope(p.qg + ((size_t)r * p.Hq + h) * 2 * HD, p.q_norm, p.eps, p.rope_dims, p.lnb, pos + r, s_q, nullptr, lane);
  else if (warp <= p.T)
    warp_norm_rope(p.k + ((size_t)(warp - 1) * p.Hkv + kvh) * HD, p.k_norm, p.eps, p.rope_dims, p.lnb, pos + warp - 1,
                   s_knew[warp - 1], nullptr, lane);
  __syncthreads();
  if (r == 0 && (h % group) == 0 && z == 0) {
    for (int i = threadIdx.x; i < p.T * HD; i += blockDim.x) {
      const int t = i / HD, d = i - t * HD;
      if (pos + t < p.cap) {
        p.kc[((size_t)kvh * p.cap + pos + t) * HD + d] = f2bf(s_knew[t][d]);
        p.vc[((size_t)kvh * p.cap + pos + t) * HD + d] = p.v[((size_t)t * p.Hkv + kvh) * HD + d];
      }
    }
  }
  int L = pos + r + 1;
  if (L > p.cap) L = p.cap;
  float qs[8], o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { qs[i] = s_q[8 * lane + i] * p.scale; o[i] = 0.f; }
  float mx = -INFINITY, sm = 0.f;
  attn_walk<8>(p, s_knew, qs, grp, L, pos, kvh, lane, o, mx, sm);
  // this group's partial to global memory
  float* mine = part + (((size_t)h * kGdnMaxT + r) * 32 + grp) * kAttnPart;
  *reinterpret_cast<float4*>(mine + 8 * lane) = make_float4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<float4*>(mine + 8 * lane + 4) = make_float4(o[4], o[5], o[6], o[7]);
  if (lane == 0) { mine[HD] = mx; mine[HD + 1] = sm; }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&arrivals[h * kGdnMaxT + r], 1) == kAttnSplit - 1 ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* all = part + ((size_t)h * kGdnMaxT + r) * 32 * kAttnPart;
  for (int i = threadIdx.x; i < 32 * HD; i += blockDim.x) s_o[i / HD][i % HD] = __ldcg(all + (size_t)(i / HD) * kAttnPart + (i % HD));
  if (threadIdx.x < 32) {
    s_max[threadIdx.x] = __ldcg(all + (size_t)threadIdx.x * kAttnPart + HD);
    s_sum[threadIdx.x] = __ldcg(all + (size_t)threadIdx.x * kAttnPart + HD + 1);
  }
  if (threadIdx.x == 0) arrivals[h * kGdnMaxT + r] = 0;  // ready for the next launch
  __syncthreads();
  if (warp == 0) {
    const float M = warp_max(s_max[lane]);
    const float f = expf_call(s_max[lane] - M);
    s_f[lane] = f;
    const float S = warp_sum(s_sum[lane] * f);
    if (lane == 0) s_sum[0] = S;
  }
  __syncthreads();
  {
    const int d = threadIdx.x;
    float a[32];
#pragma unroll
    for (int g = 0; g < 32; ++g) a[g] = s_o[g][d] * s_f[g];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
      for (int i = 0; i < off; ++i) a[i] = a[i] + a[i + off];
    const float att = bfr(a[0] / s_sum[0]);
    const float gate = bf2f(p.qg[((size_t)r * p.Hq + h) * 2 * HD + HD + d]);
    p.out[((size_t)r * p.Hq + h) * HD + d] = f2bf(sigmoid_bf_call(gate) * att);
  }
}

int f_attn(orn_ctx* ctx, cudaStream_t s, const bf16_t* qg, const bf16_t* k, const bf16_t* v, const bf16_t* q_norm,
           const bf16_t* k_norm, bf16_t* kc, bf16_t* vc, const int* pos, int T, int Hq, int Hkv, int hd, int cap,
           int rope_dims, float lnb, float eps, bf16_t* out, int long_context) {
  if (hd != 256) ORN_FAIL(ctx, ORN_ERR_ARG, "fused attention: head_dim must be 256");
  if (T > kGdnMaxT) ORN_FAIL(ctx, ORN_ERR_ARG, "fused attention: at most 4 rows");
  AttnParams p;
  p.qg = qg; p.k = k; p.v = v; p.q_norm = q_norm; p.k_norm = k_norm; p.kc = kc; p.vc = vc; p.pos = pos; p.out = out;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.cap = cap; p.rope_dims = rope_dims; p.lnb = lnb;
  p.scale = 1.0f / sqrtf((float)hd);
  p.eps = eps;
  if (long_context) {
    if (ctx->attn_partial == nullptr) {  // first use: never inside a capture (a shape runs eagerly once before it is captured)
      ORN_CHECK_CUDA(ctx, cudaMalloc((void**)&ctx->attn_partial, sizeof(float) * (size_t)kAttnMaxHeads * kGdnMaxT * 32 * kAttnPart));
      ORN_CHECK_CUDA(ctx, cudaMalloc((void**)&ctx->attn_arrivals, sizeof(int) * kAttnMaxHeads * kGdnMaxT));
      ORN_CHECK_CUDA(ctx, cudaMemset(ctx->attn_arrivals, 0, sizeof(int) * kAttnMaxHeads * kGdnMaxT));
    }
    if (Hq > kAttnMaxHeads) ORN_FAIL(ctx, ORN_ERR_ARG, "fused attention: more than 128 query heads");
    dim3 sgrid(Hq, T, kAttnSplit);
    ORN_CHECK_CUDA(ctx, orn_launch_dependent(ctx, s, 4, k_attn_split, sgrid, dim3(256), 0, p, ctx->attn_partial, ctx->attn_arrivals));
    return orn_launch_check(ctx, "k_attn_split");
  }
  dim3 grid(Hq, T);
  ORN_CHECK_CUDA(ctx, orn_launch_dependent(ctx, s, 4, k_attn, grid, dim3(1024), 0, p));
  return orn_launch_check(ctx, "k_attn");
}

int f_wait_probe(orn_ctx* ctx, cudaStream_t s, uint32_t rounds, int* dev_waited) {
  k_wait_probe<<<1, 32, ring_bytes(1, 1, 128) + 128, s>>>(rounds, ctx->dev_err, dev_waited);
  return orn_launch_check(ctx, "k_wait_probe");
}
