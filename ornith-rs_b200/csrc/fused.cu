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
#include <set>
#include <string>

#include "orn_internal.h"
#include "orn_quant.cuh"
#include "fused.h"

#ifdef ORN_DEBUG_CLOCKS
__device__ long long g_dbg[32];
#define DBG(i) do { if (blockIdx.x == 3 && threadIdx.x == 0 && J.job[0].lin.O == 8192) g_dbg[i] = clock64(); } while (0)
extern "C" int orn_debug_clocks(long long* out) { return (int)cudaMemcpyFromSymbol(out, g_dbg, sizeof(long long) * 32); }
#else
#define DBG(i)
#endif

namespace {

constexpr int kFusedThreads = 512;  // one CTA per SM: 16 warps, each with its own weight ring

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

// lin: [rows][K] floats (row stride `stride`) -> stage; block-wide, no sync
// inside.  A thread owns whole units: it moves the unit's P pieces to their
// permuted places and, for the formats that need it, adds the unit's elements
// in ascending order into the staged sum.
template <int KIND>
ORN_D void stage_fill(const float* lin, int stride, const XStage& X) {
  constexpr int P = Lay<KIND>::P, NS = Lay<KIND>::NS;
  const int padded = X.S * 32;  // unit slots per row, including the empty tail
  for (int m = 0; m < X.rows; ++m) {
    const float* src = lin + (size_t)m * stride;
    float4* dst = reinterpret_cast<float4*>(X.xs) + (size_t)m * padded * P;
    for (int u = threadIdx.x; u < padded; u += blockDim.x) {
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
  ORN_D static void load(const LinDev& L, int64_t row, int u, W& w) {
    w.q = ldg128_stream(L.w + row * L.K + 16 * u);
    w.sb = __ldg(reinterpret_cast<const uint32_t*>(L.s) + row * (L.K >> 6) + (u >> 2));
  }
  // the same unit out of a row staged in shared memory: [codes K][sb K/16]
  ORN_D static void lds(const uint8_t* b0, const uint8_t* b1, const LinDev&, int64_t, int u, W& w) {
    w.q = *reinterpret_cast<const uint4*>(b0 + 16 * u);
    w.sb = *reinterpret_cast<const uint32_t*>(b1 + 4 * (u >> 2));
  }
  ORN_D static float fold(const W& w, const float* x, const float* sm, int, float acc) {
    const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
    float s1 = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      s1 = fmaf(x[4 * k + 0], byte_f<0>(qw[k]), s1);
      s1 = fmaf(x[4 * k + 1], byte_f<1>(qw[k]), s1);
      s1 = fmaf(x[4 * k + 2], byte_f<2>(qw[k]), s1);
      s1 = fmaf(x[4 * k + 3], byte_f<3>(qw[k]), s1);
    }
    acc = fmaf(bf_lo(w.sb), s1, acc);
    acc = fmaf(bf_hi(w.sb), sm[0], acc);
    return acc;
  }
};

template <> struct WU<ORN_Q4K> {
  struct W { uint4 q; uint4 meta; };
  ORN_D static void load(const LinDev& L, int64_t row, int u, W& w) {
    const int nb = L.K >> 8;
    w.q = ldg128_stream(L.w + (row * nb + (u >> 3)) * 128 + 16 * (u & 7));
    w.meta = ldg128(L.s + (row * nb + (u >> 3)) * 16);
  }
  // staged row: [codes nb*128][headers nb*16]
  ORN_D static void lds(const uint8_t* b0, const uint8_t* b1, const LinDev&, int64_t, int u, W& w) {
    w.q = *reinterpret_cast<const uint4*>(b0 + 16 * u);
    w.meta = *reinterpret_cast<const uint4*>(b1 + (u >> 3) * 16);
  }
  ORN_D static float fold(const W& w, const float* x, const float* sm, int u, float acc) {
    const int g = (u & 7) >> 1;
    const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
    float lo = 0.f, hi = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t l4 = qw[k] & 0x0F0F0F0Fu, h4 = (qw[k] >> 4) & 0x0F0F0F0Fu;
      lo = fmaf(x[4 * k + 0], byte_f<0>(l4), lo);
      lo = fmaf(x[4 * k + 1], byte_f<1>(l4), lo);
      lo = fmaf(x[4 * k + 2], byte_f<2>(l4), lo);
      lo = fmaf(x[4 * k + 3], byte_f<3>(l4), lo);
      hi = fmaf(x[16 + 4 * k + 0], byte_f<0>(h4), hi);
      hi = fmaf(x[16 + 4 * k + 1], byte_f<1>(h4), hi);
      hi = fmaf(x[16 + 4 * k + 2], byte_f<2>(h4), hi);
      hi = fmaf(x[16 + 4 * k + 3], byte_f<3>(h4), hi);
    }
    const float d = h2f((uint16_t)(w.meta.x & 0xffff)), dmin = h2f((uint16_t)(w.meta.x >> 16));
    float s1, m1, s2, m2;
    q4k_scale_min(2 * g, w.meta.y, w.meta.z, w.meta.w, &s1, &m1);
    q4k_scale_min(2 * g + 1, w.meta.y, w.meta.z, w.meta.w, &s2, &m2);
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
  ORN_D static void load(const LinDev& L, int64_t row, int u, W& w) {
    const int nb = L.K >> 8;
    const int blk = u >> 4, j = u & 15, half = j >> 3, l0 = 4 * (j & 7);
    const uint8_t* base = L.w + (row * nb + blk) * 192;
    w.qa = ldg32_stream(base + 64 * half + l0);
    w.qb = ldg32_stream(base + 64 * half + 32 + l0);
    w.qh = ldg32_stream(base + 128 + 32 * half + l0);
    const uint2 s8 = __ldg(reinterpret_cast<const uint2*>(L.s + (row * nb + blk) * 16 + 8 * half));
    const int is = l0 >> 4;
    const uint32_t lo = s8.x >> (8 * is), hi = s8.y >> (8 * is);
    w.sc4 = (lo & 0xff) | (((lo >> 16) & 0xff) << 8) | ((hi & 0xff) << 16) | (((hi >> 16) & 0xff) << 24);
    w.d = h2f(__ldg(reinterpret_cast<const uint16_t*>(L.b) + row * nb + blk));
  }
  // staged row: [ql|qh nb*192][scales nb*16]; the 2-byte super-scale comes from global memory
  ORN_D static void lds(const uint8_t* b0, const uint8_t* b1, const LinDev& L, int64_t row, int u, W& w) {
    const int nb = L.K >> 8;
    const int blk = u >> 4, j = u & 15, half = j >> 3, l0 = 4 * (j & 7);
    const uint8_t* base = b0 + blk * 192;
    w.qa = *reinterpret_cast<const uint32_t*>(base + 64 * half + l0);
    w.qb = *reinterpret_cast<const uint32_t*>(base + 64 * half + 32 + l0);
    w.qh = *reinterpret_cast<const uint32_t*>(base + 128 + 32 * half + l0);
    const uint2 s8 = *reinterpret_cast<const uint2*>(b1 + blk * 16 + 8 * half);
    const int is = l0 >> 4;
    const uint32_t lo = s8.x >> (8 * is), hi = s8.y >> (8 * is);
    w.sc4 = (lo & 0xff) | (((lo >> 16) & 0xff) << 8) | ((hi & 0xff) << 16) | (((hi >> 16) & 0xff) << 24);
    w.d = h2f(__ldg(reinterpret_cast<const uint16_t*>(L.b) + row * nb + blk));
  }
  ORN_D static float fold(const W& w, const float* x, const float*, int, float acc) {
    const uint32_t q1 = (w.qa & 0x0F0F0F0Fu) | ((w.qh & 0x03030303u) << 4);
    const uint32_t q2 = (w.qb & 0x0F0F0F0Fu) | ((w.qh & 0x0C0C0C0Cu) << 2);
    const uint32_t q3 = ((w.qa >> 4) & 0x0F0F0F0Fu) | (w.qh & 0x30303030u);
    const uint32_t q4 = ((w.qb >> 4) & 0x0F0F0F0Fu) | ((w.qh & 0xC0C0C0C0u) >> 2);
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    s0 = fmaf(x[0], byte_m32_f<0>(q1), s0); s0 = fmaf(x[1], byte_m32_f<1>(q1), s0);
    s0 = fmaf(x[2], byte_m32_f<2>(q1), s0); s0 = fmaf(x[3], byte_m32_f<3>(q1), s0);
    s1 = fmaf(x[4], byte_m32_f<0>(q2), s1); s1 = fmaf(x[5], byte_m32_f<1>(q2), s1);
    s1 = fmaf(x[6], byte_m32_f<2>(q2), s1); s1 = fmaf(x[7], byte_m32_f<3>(q2), s1);
    s2 = fmaf(x[8], byte_m32_f<0>(q3), s2); s2 = fmaf(x[9], byte_m32_f<1>(q3), s2);
    s2 = fmaf(x[10], byte_m32_f<2>(q3), s2); s2 = fmaf(x[11], byte_m32_f<3>(q3), s2);
    s3 = fmaf(x[12], byte_m32_f<0>(q4), s3); s3 = fmaf(x[13], byte_m32_f<1>(q4), s3);
    s3 = fmaf(x[14], byte_m32_f<2>(q4), s3); s3 = fmaf(x[15], byte_m32_f<3>(q4), s3);
    const float c0 = (float)(int8_t)(w.sc4 & 0xff), c1 = (float)(int8_t)((w.sc4 >> 8) & 0xff);
    const float c2 = (float)(int8_t)((w.sc4 >> 16) & 0xff), c3 = (float)(int8_t)(w.sc4 >> 24);
    float t = c0 * s0;
    t = fmaf(c1, s1, t);
    t = fmaf(c2, s2, t);
    t = fmaf(c3, s3, t);
    return fmaf(w.d, t, acc);
  }
};

template <> struct WU<ORN_BF16> {
  struct W { uint4 q; };
  ORN_D static void load(const LinDev& L, int64_t row, int u, W& w) {
    w.q = ldg128_stream(L.w + (row * L.K + 8 * u) * 2);
  }
  ORN_D static void lds(const uint8_t* b0, const uint8_t*, const LinDev&, int64_t, int u, W& w) {
    w.q = *reinterpret_cast<const uint4*>(b0 + 16 * u);
  }
  ORN_D static float fold(const W& w, const float* x, const float*, int, float acc) {
    float f[8];
    widen8(w.q, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(x[i], f[i], acc);
    return acc;
  }
};

// ---------------------------------------------------------------------------
// weight streaming: per-warp rings of shared-memory slots filled by bulk async
// copies (cp.async.bulk, the 1-D TMA form) that complete on an mbarrier.
// Rows of every format are contiguous in HBM, so one or two bulk copies bring a
// whole row (codes, then scales/headers); lane 0 of a warp issues the copies for
// the warp's next tasks, all 32 lanes wait on the slot's barrier and read their
// own 16-byte pieces (consecutive lanes, consecutive addresses: no bank
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

constexpr int kDownCols = 2;  // consecutive output columns a warp takes per bulk copy in the down projection
constexpr uint32_t kWaitLimit = 1u << 14;  // try_wait rounds before giving up (each round may sleep kWaitHintNs)

// A row is streamed in chunks of kChunkSteps lane-steps (32 units each).  Bytes
// of the two streams per step; a chunk of `units` units (a multiple of 8) is
// [stream 0][stream 1], both multiples of 16 bytes.
constexpr int kChunkSteps = 4;
__host__ __device__ inline uint32_t step_bytes0(int kind) { return kind == ORN_Q6K ? 384 : 512; }
__host__ __device__ inline uint32_t step_bytes1(int kind) {
  return kind == ORN_A8 ? 32 : kind == ORN_Q4K ? 64 : kind == ORN_Q6K ? 32 : 0;
}
__host__ __device__ inline uint32_t units_bytes0(int kind, int units) { return kind == ORN_Q6K ? units * 12 : units * 16; }
__host__ __device__ inline uint32_t units_bytes1(int kind, int units) {
  return kind == ORN_A8 ? units : kind == ORN_Q4K ? units * 2 : kind == ORN_Q6K ? units : 0;
}
__host__ __device__ inline int kind_units(int kind, int K) { return K / kind_wpu(kind); }
// largest chunk of a row, in bytes
__host__ __device__ inline uint32_t chunk_bytes_max(int kind, int K) {
  int units = kind_units(kind, K);
  if (units > 32 * kChunkSteps) units = 32 * kChunkSteps;
  return units_bytes0(kind, units) + units_bytes1(kind, units);
}
__host__ __device__ inline int row_chunks(int kind, int K) {
  return (kind_units(kind, K) + 32 * kChunkSteps - 1) / (32 * kChunkSteps);
}

struct Ring {
  uint32_t bar0;       // shared address of this warp's first barrier
  uint32_t buf0;       // shared address of this warp's first slot
  uint8_t* buf;        // generic address of the same
  uint32_t slot_bytes;
  int depth;
  int* err;
};

// lane 0: request chunk c of a row of L into a slot at byte offset `off`;
// returns the bytes requested (0 when the row has no such chunk)
ORN_D uint32_t chunk_units(const LinDev& L, int c) {
  const int units = kind_units(L.kind, L.K) - 32 * kChunkSteps * c;
  return units <= 0 ? 0 : (units > 32 * kChunkSteps ? 32 * kChunkSteps : units);
}
ORN_D uint32_t chunk_bytes(const LinDev& L, int c) {
  const int u = chunk_units(L, c);
  return units_bytes0(L.kind, u) + units_bytes1(L.kind, u);
}
ORN_D void ring_copy_chunk(const Ring& R, int slot, uint32_t off, const LinDev& L, int64_t row, int c) {
  const int u = chunk_units(L, c);
  if (u == 0) return;
  const uint32_t b0 = units_bytes0(L.kind, u), b1 = units_bytes1(L.kind, u);
  const int tot = kind_units(L.kind, L.K);
  const uint32_t bar = R.bar0 + 8 * slot;
  const uint32_t dst = R.buf0 + slot * R.slot_bytes + off;
  bulk_g2s(dst, L.w + row * (int64_t)units_bytes0(L.kind, tot) + (int64_t)c * kChunkSteps * step_bytes0(L.kind), b0, bar);
  if (b1)
    bulk_g2s(dst + b0, L.s + row * (int64_t)units_bytes1(L.kind, tot) + (int64_t)c * kChunkSteps * step_bytes1(L.kind),
             b1, bar);
}
// all lanes: wait for a slot; false after the bounded wait ran out
ORN_D bool ring_wait(const Ring& R, int slot, uint32_t parity) {
  const uint32_t bar = R.bar0 + 8 * slot;
  for (uint32_t it = 0; it < kWaitLimit; ++it)
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
  if (lane == 0)
    for (int i = 0; i < depth; ++i) mbar_init(R.bar0 + 8 * i, 1);
  fence_mbar_init();
  fence_proxy_async();
}
__host__ __device__ inline size_t ring_bytes(int nwarps, int depth, uint32_t slot_bytes) {
  return (((size_t)nwarps * depth * 8 + 127) & ~(size_t)127) + (size_t)nwarps * depth * slot_bytes;
}

// One warp, chunk c of one staged weight row (streams at p0 / p1): adds the chunk's units
// to the lane partials acc[m] of activation rows m0 .. m0+M-1.  Units are
// visited in ascending order within a lane across chunks; the caller zeroes
// acc before chunk 0 and folds the lanes (warp_sum) after the last chunk.
template <int KIND, int M>
ORN_D void warp_chunk_dot(const uint8_t* p0, const uint8_t* p1, const LinDev& L, int64_t row, int c, const XStage& X,
                          int m0, int lane, float (&acc)[M]) {
  using U = WU<KIND>;
  constexpr int P = Lay<KIND>::P, NS = Lay<KIND>::NS;
  // virtual stream bases so that absolute unit numbers index the chunk
  const uint8_t* b0 = p0 - (size_t)c * kChunkSteps * step_bytes0(KIND);
  const uint8_t* b1 = p1 - (size_t)c * kChunkSteps * step_bytes1(KIND);
  const int s_end = min(X.S, (c + 1) * kChunkSteps);
  for (int s = c * kChunkSteps; s < s_end; ++s) {
    const int u = lane + 32 * s;
    if (u < X.units) {
      typename U::W w;
      U::lds(b0, b1, L, row, u, w);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float xv[P * 4];
        const float4* xp = reinterpret_cast<const float4*>(X.xs) + ((size_t)((m0 + m) * X.S + s) * P) * 32 + lane;
#pragma unroll
        for (int p = 0; p < P; ++p) {
          const float4 v = xp[p * 32];
          xv[4 * p] = v.x; xv[4 * p + 1] = v.y; xv[4 * p + 2] = v.z; xv[4 * p + 3] = v.w;
        }
        float sm[NS > 0 ? NS : 1];
#pragma unroll
        for (int i = 0; i < NS; ++i) sm[i] = X.sums[((size_t)(m0 + m) * X.units + u) * NS + i];
        acc[m] = U::fold(w, xv, sm, u, acc[m]);
      }
    }
  }
}

// The same for R weight rows at once (row r's streams at p0 + r*st0, p1 + r*st1):
// the staged activations of a step are read once and folded into R rows.  The
// four steps of a chunk are unrolled so that every shared-memory access is a
// hoisted base plus an immediate.
template <int KIND, int M, int R>
ORN_D void warp_chunk_dot_rows(const uint8_t* p0, uint32_t st0, const uint8_t* p1, uint32_t st1, const LinDev& L,
                               int64_t row, int nvalid, int c, const XStage& X, int m0, int lane, float (&acc)[R][M]) {
  using U = WU<KIND>;
  constexpr int P = Lay<KIND>::P, NS = Lay<KIND>::NS;
  const int s_base = c * kChunkSteps;
  const uint8_t* b0 = p0 - (size_t)c * kChunkSteps * step_bytes0(KIND);
  const uint8_t* b1 = p1 - (size_t)c * kChunkSteps * step_bytes1(KIND);
  const float4* xbase = reinterpret_cast<const float4*>(X.xs) + (size_t)(m0 * X.S + s_base) * (P * 32) + lane;
  const int xrow = X.S * P * 32;  // float4 per activation row
  const float* sbase = X.sums + ((size_t)m0 * X.units + 32 * s_base + lane) * NS;
  const int srow = X.units * NS;
#pragma unroll
  for (int ss = 0; ss < kChunkSteps; ++ss) {
    const int u = lane + 32 * (s_base + ss);
    if (u < X.units) {
      typename U::W w[R];
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (r < nvalid) U::lds(b0 + r * st0, b1 + r * st1, L, row + r, u, w[r]);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float xv[P * 4];
        const float4* xp = xbase + m * xrow + ss * (P * 32);
#pragma unroll
        for (int p = 0; p < P; ++p) {
          const float4 v = xp[p * 32];
          xv[4 * p] = v.x; xv[4 * p + 1] = v.y; xv[4 * p + 2] = v.z; xv[4 * p + 3] = v.w;
        }
        float sm[NS > 0 ? NS : 1];
#pragma unroll
        for (int i = 0; i < NS; ++i) sm[i] = sbase[m * srow + ss * 32 * NS + i];
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (r < nvalid) acc[r][m] = U::fold(w[r], xv, sm, u, acc[r][m]);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// block-wide RMS statistics in the order of the stand-alone rms kernels:
// virtual thread t owns elements 4t..4t+3, 32 virtual threads fold by
// butterfly, the warp sums (zero padded to 32) fold by butterfly again.
// lin holds `rows` rows of n raw values (stride `stride`); inv[m] receives
// 1/sqrt(sumsq/n + eps).  `red` is rows*32 floats of shared memory.
// ---------------------------------------------------------------------------
ORN_D void block_rms_inv(const float* lin, int stride, int rows, int n, float eps, float* red, float* inv) {
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < rows * 32; i += blockDim.x) red[i] = 0.f;
  __syncthreads();
  const int nvt = (n + 3) / 4;
  const int nvt_pad = ((nvt + 31) / 32) * 32;
  for (int m = 0; m < rows; ++m) {
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

// scratch: red[M*32 + M] floats.  Every loop walks (row m, 8-element group) so
// that no index needs a division and global traffic is 128-bit.
template <int M>
ORN_D void run_prologue(const Prologue& P, float* lin, float* red) {
  const int K = P.K;
  float* inv = red + M * 32;
  if (P.mode == PRO_ADDNORM) {
    // the norm weight does not depend on the statistics: fetch it before the reduction
    float wv[4] = {0.f, 0.f, 0.f, 0.f};
    const int c0 = threadIdx.x * 4;  // K <= 4 * blockDim.x is checked at launch
    if (c0 < K) {
      const uint2 ww = __ldg(reinterpret_cast<const uint2*>(P.w + c0));
      wv[0] = bf_lo(ww.x); wv[1] = bf_hi(ww.x); wv[2] = bf_lo(ww.y); wv[3] = bf_hi(ww.y);
    }
#pragma unroll
    for (int m = 0; m < M; ++m)
      if (c0 < K) {
        const uint2 av = __ldg(reinterpret_cast<const uint2*>(P.a + (size_t)m * K + c0));
        float v[4] = {bf_lo(av.x), bf_hi(av.x), bf_lo(av.y), bf_hi(av.y)};
        if (P.b != nullptr) {
          const uint2 bv = __ldg(reinterpret_cast<const uint2*>(P.b + (size_t)m * K + c0));
          v[0] = bfr(v[0] + bf_lo(bv.x)); v[1] = bfr(v[1] + bf_hi(bv.x));
          v[2] = bfr(v[2] + bf_lo(bv.y)); v[3] = bfr(v[3] + bf_hi(bv.y));
        }
        *reinterpret_cast<float4*>(lin + (size_t)m * K + c0) = make_float4(v[0], v[1], v[2], v[3]);
        if (P.sum_out != nullptr && blockIdx.x == 0) {
          uint2 o;
          o.x = (uint32_t)f2bf(v[0]) | ((uint32_t)f2bf(v[1]) << 16);
          o.y = (uint32_t)f2bf(v[2]) | ((uint32_t)f2bf(v[3]) << 16);
          *reinterpret_cast<uint2*>(P.sum_out + (size_t)m * K + c0) = o;
        }
      }
    __syncthreads();
    block_rms_inv(lin, K, M, K, P.eps, red, inv);
#pragma unroll
    for (int m = 0; m < M; ++m)
      if (c0 < K) {
        float4 v = *reinterpret_cast<const float4*>(lin + (size_t)m * K + c0);
        const float iv = inv[m];
        v.x = bfr(wv[0] * bfr(v.x * iv)); v.y = bfr(wv[1] * bfr(v.y * iv));
        v.z = bfr(wv[2] * bfr(v.z * iv)); v.w = bfr(wv[3] * bfr(v.w * iv));
        *reinterpret_cast<float4*>(lin + (size_t)m * K + c0) = v;
      }
  } else if (P.mode == PRO_PLAIN) {
#pragma unroll
    for (int m = 0; m < M; ++m)
      for (int c = threadIdx.x * 4; c < K; c += blockDim.x * 4) {
        const uint2 av = __ldg(reinterpret_cast<const uint2*>(P.a + (size_t)m * K + c));
        *reinterpret_cast<float4*>(lin + (size_t)m * K + c) = make_float4(bf_lo(av.x), bf_hi(av.x), bf_lo(av.y), bf_hi(av.y));
      }
  } else if (P.mode == PRO_GATED) {
    // rms_norm_gated over 128-wide heads (kernels/ornith_norm.metal:119-185)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pairs = M * (K >> 7);
    for (int pair = warp; pair < pairs; pair += (blockDim.x >> 5)) {
      const int base = pair * 128 + 4 * lane;
      float xv[4];
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) { xv[i] = bf2f(P.a[base + i]); acc = fmaf(xv[i], xv[i], acc); }
      acc = warp_sum(acc);
      const float iv = orn_rsqrtf(acc / 128.0f + P.eps);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float normed = bfr(bf2f(P.w[4 * lane + i]) * bfr(xv[i] * iv));
        float g = bf2f(P.b[base + i]);
        g = g * orn_sigmoid_f32(g);
        lin[base + i] = bfr(g * normed);
      }
    }
  } else {  // PRO_MTPJOIN: [norm(embed(id)) | norm(trunk hidden)] (src/model/mtp.rs:179-187)
    const int H = K >> 1;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const int64_t row = P.ids[m];
      for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const uint32_t sb = reinterpret_cast<const uint32_t*>(P.emb.s)[row * (H >> 6) + (c >> 6)];
        lin[(size_t)m * K + c] = bfr(fmaf(bf_lo(sb), (float)P.emb.w[row * H + c], bf_hi(sb)));
        lin[(size_t)m * K + H + c] = bf2f(P.a[(size_t)m * H + c]);
      }
    }
    __syncthreads();
    block_rms_inv(lin, K, M, H, P.eps, red, inv);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      const float w = bf2f(P.w[c]);
#pragma unroll
      for (int m = 0; m < M; ++m) lin[(size_t)m * K + c] = bfr(w * bfr(lin[(size_t)m * K + c] * inv[m]));
    }
    __syncthreads();
    block_rms_inv(lin + H, K, M, H, P.eps, red, inv);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      const float w = bf2f(P.w2[c]);
#pragma unroll
      for (int m = 0; m < M; ++m) lin[(size_t)m * K + H + c] = bfr(w * bfr(lin[(size_t)m * K + H + c] * inv[m]));
    }
  }
  __syncthreads();
  if (P.norm_out != nullptr && blockIdx.x == 0) {
#pragma unroll
    for (int m = 0; m < M; ++m)
      for (int c = threadIdx.x; c < K; c += blockDim.x) P.norm_out[(size_t)m * K + c] = f2bf(lin[(size_t)m * K + c]);
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
  int tasks;     // row pairs of the job
  int units;     // lane units per row
  int nchunk;    // streamed chunks per row
  uint32_t rb0, rb1;  // bytes per row of the two streams
};
struct RowJobs {
  RowJob job[4];
  int njobs;
  int kinds_mask;  // bit k set when some job has weights of kind k
};

constexpr int kRowsPerTask = 2;  // consecutive weight rows a warp takes per task

// a warp's position in its task sequence: row pairs gw, gw+GW, ... of the
// concatenated jobs, each in `nchunk` chunks; no divisions
struct Cursor {
  int j, t, c;  // job, task (row pair) within the job, chunk
  ORN_D bool valid(const RowJobs& J) const { return j < J.njobs; }
  ORN_D void settle(const RowJobs& J) {
    while (j < J.njobs && t >= J.job[j].tasks) { t -= J.job[j].tasks; ++j; }
  }
  ORN_D void advance(const RowJobs& J, int GW) {
    if (++c == J.job[j].nchunk) {
      c = 0;
      t += GW;
      settle(J);
    }
  }
};

ORN_D int job_chunk_units(const RowJob& job, int c) {
  const int u = job.units - 32 * kChunkSteps * c;
  return u > 32 * kChunkSteps ? 32 * kChunkSteps : u;
}

// lane 0: request chunk c of rows [row, row+n) of matrix L into a slot at byte
// offset `off`, laid out [n x stream 0][n x stream 1].  Whole rows (nchunk == 1)
// are contiguous in HBM and travel as one copy per stream.
ORN_D void job_copy_tile(const Ring& R, int slot, uint32_t off, const RowJob& job, const LinDev& L, int row, int n,
                         int c, uint32_t b0, uint32_t b1) {
  const uint32_t bar = R.bar0 + 8 * slot;
  const uint32_t dst = R.buf0 + slot * R.slot_bytes + off;
  if (job.nchunk == 1) {
    bulk_g2s(dst, L.w + (int64_t)row * job.rb0, n * b0, bar);
    if (b1) bulk_g2s(dst + kRowsPerTask * b0, L.s + (int64_t)row * job.rb1, n * b1, bar);
  } else {
    for (int r = 0; r < n; ++r) {
      bulk_g2s(dst + r * b0, L.w + (int64_t)(row + r) * job.rb0 + (int64_t)c * kChunkSteps * step_bytes0(L.kind), b0, bar);
      if (b1)
        bulk_g2s(dst + kRowsPerTask * b0 + r * b1,
                 L.s + (int64_t)(row + r) * job.rb1 + (int64_t)c * kChunkSteps * step_bytes1(L.kind), b1, bar);
    }
  }
}

// tile dot for the formats present in MASK only (keeps the kernel small)
template <int M, int MASK>
ORN_D void tile_dot_masked(const uint8_t* buf, uint32_t b0, uint32_t b1, const LinDev& L, int64_t row, int nvalid, int c,
                           const XStage* X, int lane, float (&acc)[kRowsPerTask][M]) {
  const uint8_t* p1 = buf + kRowsPerTask * b0;
  if ((MASK & (1 << ORN_A8)) && L.kind == ORN_A8)
    warp_chunk_dot_rows<ORN_A8, M, kRowsPerTask>(buf, b0, p1, b1, L, row, nvalid, c, X[ORN_A8], 0, lane, acc);
  else if ((MASK & (1 << ORN_Q4K)) && L.kind == ORN_Q4K)
    warp_chunk_dot_rows<ORN_Q4K, M, kRowsPerTask>(buf, b0, p1, b1, L, row, nvalid, c, X[ORN_Q4K], 0, lane, acc);
  else if ((MASK & (1 << ORN_Q6K)) && L.kind == ORN_Q6K)
    warp_chunk_dot_rows<ORN_Q6K, M, kRowsPerTask>(buf, b0, p1, b1, L, row, nvalid, c, X[ORN_Q6K], 0, lane, acc);
  else if ((MASK & (1 << ORN_BF16)) && L.kind == ORN_BF16)
    warp_chunk_dot_rows<ORN_BF16, M, kRowsPerTask>(buf, b0, p1, b1, L, row, nvalid, c, X[ORN_BF16], 0, lane, acc);
}

template <int M, int MASK>
__global__ void __launch_bounds__(kFusedThreads, 1) k_norm_gemv(Prologue P, RowJobs J, uint32_t slot_bytes, int depth,
                                                                uint32_t ring_off, int* err) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float* smem = reinterpret_cast<float*>(smem_raw);
  const int lane = threadIdx.x & 31;
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int GW = gridDim.x * (blockDim.x >> 5);
  // The weights do not depend on the activations: the rings are set up and the
  // first `depth` tiles of every warp requested before the prologue runs, so
  // that HBM is busy while the CTA rebuilds its input.
  DBG(0);
  Ring R;
  ring_setup(R, smem_raw + ring_off, slot_bytes, depth, err);
  __syncthreads();
  DBG(1);
  Cursor pc{0, gw, 0}, cc{0, gw, 0};
  pc.settle(J);
  cc.settle(J);
  int pslot = 0;
  auto issue = [&]() {  // all lanes keep the cursor; lane 0 issues
    const RowJob& job = J.job[pc.j];
    if (lane == 0) {
      const int u = job_chunk_units(job, pc.c);
      const uint32_t b0 = units_bytes0(job.lin.kind, u), b1 = units_bytes1(job.lin.kind, u);
      const int row = pc.t * kRowsPerTask;
      const int n = min(kRowsPerTask, job.lin.O - row);
      mbar_expect_tx(R.bar0 + 8 * pslot, (job.epi == EPI_SWIGLU ? 2 : 1) * n * (b0 + b1));
      job_copy_tile(R, pslot, 0, job, job.lin, row, n, pc.c, b0, b1);
      if (job.epi == EPI_SWIGLU) job_copy_tile(R, pslot, kRowsPerTask * (b0 + b1), job, job.lin2, row, n, pc.c, b0, b1);
    }
    pc.advance(J, GW);
    if (++pslot == depth) pslot = 0;
  };
  for (int i = 0; i < depth && pc.valid(J); ++i) issue();
  DBG(2);

  // stages, then the prologue's scratch
  float* next = smem;
  XStage X[4];
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (MASK & (1 << k)) next = stage_carve(next, k, M, P.K, X[k]);
  float* lin = smem + (((next - smem) + 31) & ~31);
  float* red = lin + (size_t)M * P.K;
  run_prologue<M>(P, lin, red);
  DBG(3);
  if (MASK & (1 << ORN_Q4K)) stage_fill<ORN_Q4K>(lin, P.K, X[ORN_Q4K]);
  if (MASK & (1 << ORN_Q6K)) stage_fill<ORN_Q6K>(lin, P.K, X[ORN_Q6K]);
  if (MASK & (1 << ORN_A8)) stage_fill<ORN_A8>(lin, P.K, X[ORN_A8]);
  if (MASK & (1 << ORN_BF16)) stage_fill<ORN_BF16>(lin, P.K, X[ORN_BF16]);
  __syncthreads();
  DBG(4);

  float acc[kRowsPerTask][M], up[kRowsPerTask][M];
  int slot = 0;
  uint32_t parity = 0;
  int dbg_n = 0;
  while (cc.valid(J)) {
    if (!ring_wait(R, slot, parity)) return;
    if (dbg_n < 8) { DBG(5 + 2 * dbg_n); }
    const RowJob& job = J.job[cc.j];
    const uint8_t* buf = R.buf + (size_t)slot * slot_bytes;
    const int cu = job_chunk_units(job, cc.c);
    const uint32_t b0 = units_bytes0(job.lin.kind, cu), b1 = units_bytes1(job.lin.kind, cu);
    const int row = cc.t * kRowsPerTask;
    const int nvalid = min(kRowsPerTask, job.lin.O - row);
    if (cc.c == 0) {
#pragma unroll
      for (int r = 0; r < kRowsPerTask; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) { acc[r][m] = 0.f; up[r][m] = 0.f; }
    }
    if (dbg_n == 0) { DBG(20); }
    tile_dot_masked<M, MASK>(buf, b0, b1, job.lin, row, nvalid, cc.c, X, lane, acc);
    if (dbg_n == 0) { DBG(21); }
    if (job.epi == EPI_SWIGLU)
      tile_dot_masked<M, MASK>(buf + kRowsPerTask * (b0 + b1), b0, b1, job.lin2, row, nvalid, cc.c, X, lane, up);
    if (dbg_n == 0) { DBG(22); }
    if (cc.c == job.nchunk - 1) {
#pragma unroll
      for (int r = 0; r < kRowsPerTask; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) {
          float v = warp_sum(acc[r][m]);
          if (job.epi == EPI_SWIGLU) v = orn_swiglu_bf(bfr(v), bfr(warp_sum(up[r][m])));
          if (lane == 0 && r < nvalid) job.out[(size_t)m * job.lin.O + row + r] = f2bf(v);
        }
    }
    if (dbg_n == 0) { DBG(23); }
    __syncwarp();
    if (pc.valid(J)) {
      if (lane == 0) fence_proxy_async();
      issue();  // refills the slot just consumed
    }
    if (dbg_n == 0) { DBG(24); }
    cc.advance(J, GW);
    if (++slot == depth) { slot = 0; parity ^= 1; }
    if (dbg_n < 8) { DBG(6 + 2 * dbg_n); }
    ++dbg_n;
  }
  DBG(30);
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
  int E, k, H, I;
};

// softmax (mlx softmax.h:10-99, float accumulate) then router_top_k
// (kernels/moe.metal:568-614) for one token by one warp; results to shared
ORN_D void warp_softmax_topk(const bf16_t* logits, int n, int k, float* probs /*[n] smem*/,
                             float* red /*[32] smem*/, uint32_t* inds, float* scores, int lane) {
  float mx = -INFINITY;
  for (int i = lane; i < n; i += 32) mx = fmaxf(mx, bf2f(logits[i]));
  mx = warp_max(mx);
  const int nvt = (n + 3) / 4;
  const int nvw = (nvt + 31) / 32;
  red[lane] = 0.f;
  __syncwarp();
  for (int vw = 0; vw < nvw; ++vw) {
    const int vt = vw * 32 + lane;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = 4 * vt + i;
      if (idx < n) {
        const float e = orn_expf(bf2f(logits[idx]) - mx);
        probs[idx] = e;
        acc = acc + e;
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) red[vw] = acc;
  }
  __syncwarp();
  const float inv = 1.0f / warp_sum(red[lane]);
  __syncwarp();
  for (int i = lane; i < n; i += 32) probs[i] = bfr(probs[i] * inv);
  __syncwarp();
  constexpr int kMaxPerLane = 16;
  float v[kMaxPerLane];
  int held = 0;
#pragma unroll
  for (int s = 0; s < kMaxPerLane; ++s) {
    const int i = lane + 32 * s;
    v[s] = -INFINITY;
    if (i < n) { v[s] = probs[i]; held = s + 1; }
  }
  for (int r = 0; r < k; ++r) {
    float best = -INFINITY;
    uint32_t besti = 0;
#pragma unroll
    for (int s = 0; s < kMaxPerLane; ++s) {
      const uint32_t i = lane + 32 * s;
      if (s < held && (v[s] > best || (v[s] == best && i > besti))) { best = v[s]; besti = i; }
    }
    const float m = warp_max(best);
    const uint32_t mi = warp_max_u32(best == m ? besti + 1 : 0u) - 1;
#pragma unroll
    for (int s = 0; s < kMaxPerLane; ++s)
      if ((mi & 31) == (uint32_t)lane && (mi >> 5) == (uint32_t)s) v[s] = -INFINITY;
    if (lane == 0) {
      inds[k - 1 - r] = mi;
      scores[k - 1 - r] = probs[mi];
    }
  }
  __syncwarp();
}

template <int KIND, int M>
__global__ void __launch_bounds__(kFusedThreads, 1) k_moe_up(MoeUpParams P, uint32_t slot_bytes, int depth, int* err) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float* smem = reinterpret_cast<float*>(smem_raw);
  XStage X;
  float* next = stage_carve(smem, KIND, M, P.H, X);
  uint32_t* inds = reinterpret_cast<uint32_t*>(next);  // [M][k], lives through the kernel
  next += M * P.k;
  uint8_t* region = reinterpret_cast<uint8_t*>(smem) + ((((uint8_t*)next - (uint8_t*)smem) + 127) & ~(size_t)127);
  float* lin = reinterpret_cast<float*>(region);       // [M][H]
  float* probs = lin + (size_t)M * P.H;                // [M][E]
  float* red = probs + (size_t)M * P.E;                // [M][32]
  float* scores = red + M * 32;                        // [M][k]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (warp < M)
    warp_softmax_topk(P.logits + (size_t)warp * P.E, P.E, P.k, probs + (size_t)warp * P.E, red + warp * 32,
                      inds + warp * P.k, scores + warp * P.k, lane);
  for (int i = threadIdx.x; i < M * P.H; i += blockDim.x) lin[i] = bf2f(P.x[i]);
  __syncthreads();
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i < M * P.k; i += blockDim.x) {
      P.inds[i] = inds[i];
      P.scores[i] = f2bf(scores[i]);
    }
  stage_fill<KIND>(lin, P.H, X);
  __syncthreads();
  Ring R;
  ring_setup(R, region, slot_bytes, depth, err);
  __syncthreads();
  // task sequence of a warp: (mj, op) = routed row mj, pair op of consecutive expert output rows, starting
  // at flat index gw and stepping by GW, each in `nchunk` chunks; positions advance without divisions
  constexpr int RT = kRowsPerTask;
  const int gw = blockIdx.x * (blockDim.x >> 5) + warp, GW = gridDim.x * (blockDim.x >> 5);
  const int nmj = M * P.k;
  const int npair = (P.I + RT - 1) / RT;
  const int units = X.units;
  const int nchunk = (units + 32 * kChunkSteps - 1) / (32 * kChunkSteps);
  const uint32_t rb0 = units_bytes0(KIND, units), rb1 = units_bytes1(KIND, units);
  struct Pos {
    int mj, op, c;
  };
  auto settle = [&](Pos& q) {
    while (q.mj < nmj && q.op >= npair) { q.op -= npair; ++q.mj; }
  };
  auto advance = [&](Pos& q) {
    if (++q.c == nchunk) { q.c = 0; q.op += GW; settle(q); }
  };
  auto cunits = [&](int c) {
    const int u = units - 32 * kChunkSteps * c;
    return u > 32 * kChunkSteps ? 32 * kChunkSteps : u;
  };
  Pos pp{0, gw, 0}, cp{0, gw, 0};
  settle(pp);
  settle(cp);
  int pslot = 0;
  // slot layout: [gate: RT x stream 0][gate: RT x stream 1][up: RT x stream 0][up: RT x stream 1]
  auto issue = [&]() {
    if (lane == 0) {
      const int o = pp.op * RT;
      const int n = min(RT, P.I - o);
      const int64_t row = (int64_t)inds[pp.mj] * P.I + o;
      const int u = cunits(pp.c);
      const uint32_t b0 = units_bytes0(KIND, u), b1 = units_bytes1(KIND, u);
      const uint32_t bar = R.bar0 + 8 * pslot;
      const uint32_t dst = R.buf0 + pslot * R.slot_bytes;
      const uint32_t half = RT * (b0 + b1);
      mbar_expect_tx(bar, 2 * n * (b0 + b1));
      if (nchunk == 1) {
        bulk_g2s(dst, P.gate.w + row * rb0, n * b0, bar);
        if (b1) bulk_g2s(dst + RT * b0, P.gate.s + row * rb1, n * b1, bar);
        bulk_g2s(dst + half, P.up.w + row * rb0, n * b0, bar);
        if (b1) bulk_g2s(dst + half + RT * b0, P.up.s + row * rb1, n * b1, bar);
      } else {
        for (int r = 0; r < n; ++r) {
          const int64_t o0 = (row + r) * rb0 + (int64_t)pp.c * kChunkSteps * step_bytes0(KIND);
          const int64_t o1 = (row + r) * rb1 + (int64_t)pp.c * kChunkSteps * step_bytes1(KIND);
          bulk_g2s(dst + r * b0, P.gate.w + o0, b0, bar);
          if (b1) bulk_g2s(dst + RT * b0 + r * b1, P.gate.s + o1, b1, bar);
          bulk_g2s(dst + half + r * b0, P.up.w + o0, b0, bar);
          if (b1) bulk_g2s(dst + half + RT * b0 + r * b1, P.up.s + o1, b1, bar);
        }
      }
    }
    advance(pp);
    if (++pslot == depth) pslot = 0;
  };
  for (int i = 0; i < depth && pp.mj < nmj; ++i) issue();
  float g[RT][1], u[RT][1];
  int slot = 0;
  uint32_t parity = 0;
  while (cp.mj < nmj) {
    if (!ring_wait(R, slot, parity)) return;
    int m = 0;
    for (int t = P.k; t <= cp.mj; t += P.k) ++m;  // m = mj / k without a division
    const int o = cp.op * RT;
    const int nvalid = min(RT, P.I - o);
    const int64_t row = (int64_t)inds[cp.mj] * P.I + o;
    const uint8_t* buf = R.buf + (size_t)slot * slot_bytes;
    const int cu = cunits(cp.c);
    const uint32_t cb0 = units_bytes0(KIND, cu), cb1 = units_bytes1(KIND, cu);
    const uint32_t half = RT * (cb0 + cb1);
    if (cp.c == 0) {
#pragma unroll
      for (int r = 0; r < RT; ++r) { g[r][0] = 0.f; u[r][0] = 0.f; }
    }
    warp_chunk_dot_rows<KIND, 1, RT>(buf, cb0, buf + RT * cb0, cb1, P.gate, row, nvalid, cp.c, X, m, lane, g);
    warp_chunk_dot_rows<KIND, 1, RT>(buf + half, cb0, buf + half + RT * cb0, cb1, P.up, row, nvalid, cp.c, X, m, lane, u);
    if (cp.c == nchunk - 1) {
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        const float gs = warp_sum(g[r][0]), us = warp_sum(u[r][0]);
        if (lane == 0 && r < nvalid) P.act[(size_t)cp.mj * P.I + o + r] = f2bf(orn_swiglu_bf(bfr(gs), bfr(us)));
      }
    }
    __syncwarp();
    if (pp.mj < nmj) {
      if (lane == 0) fence_proxy_async();
      issue();
    }
    advance(cp);
    if (++slot == depth) { slot = 0; parity ^= 1; }
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
  int k, H, I, SI, normalize;
};

template <int KIND, int M>
__global__ void __launch_bounds__(kFusedThreads, 1) k_moe_down(MoeDownParams P, uint32_t slot_bytes, int depth, int* err) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float* smem = reinterpret_cast<float*>(smem_raw);
  const int rows = M * P.k;
  XStage X, XS;
  float* next = stage_carve(smem, KIND, rows, P.I, X);
  next = stage_carve(next, KIND, M, P.SI, XS);
  float* wts = next;                                   // [M][k] normalised scores
  float* gsig = wts + rows;                            // [M]
  uint32_t* inds = reinterpret_cast<uint32_t*>(gsig + M);
  next = reinterpret_cast<float*>(inds + rows);
  uint8_t* region = reinterpret_cast<uint8_t*>(smem) + ((((uint8_t*)next - (uint8_t*)smem) + 127) & ~(size_t)127);
  float* lin = reinterpret_cast<float*>(region);       // [rows][I] then [M][SI]
  float* lin2 = lin + (size_t)rows * P.I;
  for (int i = threadIdx.x; i < rows * P.I; i += blockDim.x) lin[i] = bf2f(P.act[i]);
  for (int i = threadIdx.x; i < M * P.SI; i += blockDim.x) lin2[i] = bf2f(P.sact[i]);
  if (threadIdx.x < M) {
    const int m = threadIdx.x;
    float denom = 0.f;
    if (P.normalize)
      for (int j = 0; j < P.k; ++j) denom = bfr(bf2f(P.scores[m * P.k + j]) + denom);
    for (int j = 0; j < P.k; ++j) {
      const float sc = bf2f(P.scores[m * P.k + j]);
      wts[m * P.k + j] = P.normalize ? bfr(sc / denom) : sc;
      inds[m * P.k + j] = P.inds[m * P.k + j];
    }
    gsig[m] = orn_sigmoid_bf(bf2f(P.gs[m]));
  }
  __syncthreads();
  stage_fill<KIND>(lin, P.I, X);
  stage_fill<KIND>(lin2, P.SI, XS);
  __syncthreads();
  Ring R;
  ring_setup(R, region, slot_bytes, depth, err);
  __syncthreads();
  // A warp owns groups of kDownCols consecutive output columns (group gw,
  // gw+GW, ...).  Consecutive columns are consecutive weight rows of one expert,
  // so one pair of bulk copies brings a group's rows of one routed expert.  Per
  // group the warp consumes the M*k routed tiles in (m, j) order and then the
  // shared expert's tile.  Rows here are short (one chunk each, checked at launch).
  const int lane = threadIdx.x & 31;
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), GW = gridDim.x * (blockDim.x >> 5);
  const int ngroups = P.H / kDownCols;
  const uint32_t b0 = units_bytes0(KIND, X.units), b1 = units_bytes1(KIND, X.units);      // routed row
  const uint32_t sb0 = units_bytes0(KIND, XS.units), sb1 = units_bytes1(KIND, XS.units);  // shared row
  struct Pos {
    int g, q;
  };
  auto advance = [&](Pos& t) {
    if (++t.q > rows) { t.q = 0; t.g += GW; }
  };
  Pos pp{gw, 0}, cp{gw, 0};
  int pslot = 0;
  auto issue = [&]() {
    if (lane == 0) {
      const uint32_t bar = R.bar0 + 8 * pslot;
      const uint32_t dst = R.buf0 + pslot * R.slot_bytes;
      const int c0 = pp.g * kDownCols;
      if (pp.q < rows) {
        const int64_t row = (int64_t)inds[pp.q] * P.H + c0;
        mbar_expect_tx(bar, kDownCols * (b0 + b1));
        bulk_g2s(dst, P.down.w + row * b0, kDownCols * b0, bar);
        if (b1) bulk_g2s(dst + kDownCols * b0, P.down.s + row * b1, kDownCols * b1, bar);
      } else {
        mbar_expect_tx(bar, kDownCols * (sb0 + sb1));
        bulk_g2s(dst, P.sh_down.w + (int64_t)c0 * sb0, kDownCols * sb0, bar);
        if (sb1) bulk_g2s(dst + kDownCols * sb0, P.sh_down.s + (int64_t)c0 * sb1, kDownCols * sb1, bar);
      }
    }
    advance(pp);
    if (++pslot == depth) pslot = 0;
  };
  for (int i = 0; i < depth && pp.g < ngroups; ++i) issue();
  float acc[kDownCols][M];
#pragma unroll
  for (int r = 0; r < kDownCols; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
  int slot = 0;
  uint32_t parity = 0;
  while (cp.g < ngroups) {
    if (!ring_wait(R, slot, parity)) return;
    const uint8_t* buf = R.buf + (size_t)slot * slot_bytes;
    const int c0 = cp.g * kDownCols;
    if (cp.q < rows) {
      const int64_t row = (int64_t)inds[cp.q] * P.H + c0;
      const float w = wts[cp.q];
      int m = 0;
      for (int t = P.k; t <= cp.q; t += P.k) ++m;  // m = q / k without a division
      float d[kDownCols][1];
#pragma unroll
      for (int r = 0; r < kDownCols; ++r) d[r][0] = 0.f;
      warp_chunk_dot_rows<KIND, 1, kDownCols>(buf, b0, buf + kDownCols * b0, b1, P.down, row, kDownCols, 0, X, cp.q, lane, d);
#pragma unroll
      for (int r = 0; r < kDownCols; ++r) {
        const float weighted = bfr(bfr(warp_sum(d[r][0])) * w);
#pragma unroll
        for (int mm = 0; mm < M; ++mm)
          if (mm == m) acc[r][mm] = bfr(weighted + acc[r][mm]);
      }
    } else {
      float sd[kDownCols][M];
#pragma unroll
      for (int r = 0; r < kDownCols; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) sd[r][m] = 0.f;
      warp_chunk_dot_rows<KIND, M, kDownCols>(buf, sb0, buf + kDownCols * sb0, sb1, P.sh_down, c0, kDownCols, 0, XS, 0, lane, sd);
#pragma unroll
      for (int r = 0; r < kDownCols; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float v = warp_sum(sd[r][m]);
          if (lane == 0) P.out[(size_t)m * P.H + c0 + r] = f2bf(acc[r][m] + bfr(gsig[m] * bfr(v)));
          acc[r][m] = 0.f;
        }
    }
    __syncwarp();
    if (pp.g < ngroups) {
      if (lane == 0) fence_proxy_async();
      issue();
    }
    advance(cp);
    if (++slot == depth) { slot = 0; parity ^= 1; }
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
};

constexpr int kGdnRows = 16;
constexpr int kGdnMaxT = 4;

__global__ void __launch_bounds__(kGdnRows * 4) k_gdn(GdnParams p) {
  __shared__ float s_q[kGdnMaxT][128], s_k[kGdnMaxT][128], s_v[kGdnMaxT][kGdnRows];
  __shared__ float s_g[kGdnMaxT], s_beta[kGdnMaxT];
  const int hv = blockIdx.y;
  const int hk = hv / (p.Hv / p.Hk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int key_dim = p.Hk * 128;
  // ---- front end (kernels/gdn_front.metal:65-190): warp 0 -> q head, warp 1 -> k head
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
    for (int r = 0; r < 4; ++r) { yv[r] = orn_silu_bf(bfr(acc[r])); sum = fmaf(yv[r], yv[r], sum); }
    sum = warp_sum(sum);
    const float inv = orn_rsqrtf(sum / 128.0f + p.eps);
    const float sc = warp == 0 ? p.q_scale : p.k_scale;
    float* dst = warp == 0 ? s_q[t] : s_k[t];
#pragma unroll
    for (int r = 0; r < 4; ++r) dst[4 * lane + r] = bfr(sc * bfr(yv[r] * inv));
  }
  // value rows of this CTA and the per-head gates
  const int row = blockIdx.x * kGdnRows + (threadIdx.x >> 2);
  const int lir = threadIdx.x & 3;
  if (lir == 0) {
    const int c = 2 * key_dim + hv * 128 + row;
    for (int t = 0; t < p.T; ++t) {
      float acc = 0.f;
      for (int i = 0; i < p.Kc; ++i)
        acc = fmaf(bf2f(p.conv[(size_t)(t + i) * p.D + c]), bf2f(p.cw[(size_t)c * p.Kc + i]), acc);
      s_v[t][threadIdx.x >> 2] = orn_silu_bf(bfr(acc));
    }
  }
  if (threadIdx.x < p.T) {
    const int t = threadIdx.x;
    const size_t i = (size_t)t * p.Hv + hv;
    const float sp = orn_softplus_bf(bfr(bf2f(p.a_in[i]) + bf2f(p.dt_bias[hv])));
    const float decay = orn_expf(bf2f(p.a_log[hv]));
    s_g[t] = orn_expf((-decay) * sp);
    s_beta[t] = orn_sigmoid_bf(bf2f(p.b_in[i]));
  }
  __syncthreads();
  // ---- recurrence (kernels/gated_delta.metal:36-142)
  const size_t ssz = (size_t)p.Hv * 128 * 128;
  const size_t off = ((size_t)hv * 128 + row) * 128 + lir * 32;
  const int cur = *p.cur;
  const float* sin = p.ring + (size_t)(cur % p.nring) * ssz + off;
  float S[32];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 v4 = *reinterpret_cast<const float4*>(sin + 4 * i);
    S[4 * i] = v4.x; S[4 * i + 1] = v4.y; S[4 * i + 2] = v4.z; S[4 * i + 3] = v4.w;
  }
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
      for (int i = 0; i < 8; ++i)
        *reinterpret_cast<float4*>(sout + 4 * i) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
    }
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
    const float inv_freq = orn_expf(-(float)i * lnb);
    const float ang = (float)position * inv_freq;
    float sn, cs;
    orn_sincosf(ang, &sn, &cs);
    const float x1 = dst[i], x2 = dst[i + half];
    const float t1 = x2 * sn, t2 = x2 * cs;
    dst[i] = bfr(fmaf(x1, cs, -t1));
    dst[i + half] = bfr(fmaf(x1, sn, t2));
  }
  __syncwarp();
}

__global__ void __launch_bounds__(1024) k_attn(AttnParams p) {
  constexpr int HD = 256;
  __shared__ float s_o[32][HD];
  __shared__ float s_q[HD];
  __shared__ float s_knew[kGdnMaxT][HD];
  __shared__ float s_max[32], s_sum[32], s_f[32];
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
  for (int n = warp; n < L; n += 32) {
    float kf[8], vf[8];
    if (n >= pos) {
#pragma unroll
      for (int i = 0; i < 8; ++i) kf[i] = s_knew[n - pos][8 * lane + i];
      widen8(ldg128(p.v + ((size_t)(n - pos) * p.Hkv + kvh) * HD + 8 * lane), vf);
    } else {
      const size_t rowoff = ((size_t)kvh * p.cap + n) * HD + 8 * lane;
      widen8(*reinterpret_cast<const uint4*>(p.kc + rowoff), kf);
      widen8(*reinterpret_cast<const uint4*>(p.vc + rowoff), vf);
    }
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(qs[i], kf[i], acc);
    const float score = warp_sum(acc);
    const float nm = fmaxf(mx, score);
    const float factor = orn_expf(mx - nm);
    const float e = orn_expf(score - nm);
    mx = nm;
    sm = fmaf(sm, factor, e);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = fmaf(o[i], factor, e * vf[i]);
  }
  if (lane == 0) { s_max[warp] = mx; s_sum[warp] = sm; }
#pragma unroll
  for (int i = 0; i < 8; ++i) s_o[warp][8 * lane + i] = o[i];
  __syncthreads();
  if (warp == 0) {
    const float M = warp_max(s_max[lane]);
    const float f = orn_expf(s_max[lane] - M);
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
    p.out[((size_t)r * p.Hq + h) * HD + d] = f2bf(orn_sigmoid_bf(gate) * att);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
constexpr size_t kSmemBudget = 220 * 1024;

// launch label for the per-kernel time report (ORN_KTIME=1): kernel, rows, first job's shape
const char* launch_label(orn_ctx* ctx, const char* kern, int M, int kind, int O, int K) {
  if (!ctx->kt) return kern;
  static std::set<std::string> pool;
  char buf[96];
  snprintf(buf, sizeof buf, "%s M=%d kind=%d %dx%d", kern, M, kind, O, K);
  return pool.insert(buf).first->c_str();
}

// raise a kernel's dynamic shared-memory limit once (per kernel, per process)
template <typename Kern>
int set_smem(orn_ctx* ctx, Kern kern, size_t bytes) {
  static std::map<const void*, bool> granted;  // keyed by kernel address (instantiations share a type)
  if (bytes > 227 * 1024) ORN_FAIL(ctx, ORN_ERR_ARG, "fused kernel: staged activations exceed shared memory");
  const void* key = reinterpret_cast<const void*>(kern);
  if (bytes > 48 * 1024 && !granted[key]) {
    ORN_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    granted[key] = true;
  }
  return ORN_OK;
}

// ring depth that fits beside `fixed` bytes of stages, and the dynamic shared
// memory of the launch: max(prologue scratch, rings) shares one region
int plan_smem(orn_ctx* ctx, size_t fixed, size_t scratch, uint32_t slot_bytes, int* depth, size_t* total) {
  const int nwarps = kFusedThreads / 32;
  fixed = (fixed + 127) & ~(size_t)127;
  int d = 8;
  while (d > 1 && fixed + ring_bytes(nwarps, d, slot_bytes) > kSmemBudget) --d;
  const size_t rb = ring_bytes(nwarps, d, slot_bytes);
  *depth = d;
  *total = fixed + (rb > scratch ? rb : scratch) + 128;
  if (*total > 227 * 1024) ORN_FAIL(ctx, ORN_ERR_ARG, "fused kernel: rows too long for the shared-memory rings");
  return ORN_OK;
}

template <int M, int MASK>
int launch_norm_gemv_mask(orn_ctx* ctx, cudaStream_t s, const Prologue& P, const RowJobs& J, uint32_t slot) {
  size_t fixed = 0;
  for (int k = 0; k < 4; ++k)
    if (MASK & (1 << k)) fixed += stage_floats(k, M, P.K) * sizeof(float);
  // stages + prologue scratch stay live beside the rings (the rings are filled while the prologue runs)
  fixed += ((size_t)M * P.K + M * 33 + 64) * sizeof(float);
  fixed = (fixed + 127) & ~(size_t)127;
  int depth;
  size_t bytes;
  int rc = plan_smem(ctx, fixed, 0, slot, &depth, &bytes);
  if (rc != ORN_OK) return rc;
  rc = set_smem(ctx, k_norm_gemv<M, MASK>, bytes);
  if (rc != ORN_OK) return rc;
  k_norm_gemv<M, MASK><<<ctx->sm_count, kFusedThreads, bytes, s>>>(P, J, slot, depth, (uint32_t)fixed, ctx->dev_err);
  return orn_launch_check(ctx, launch_label(ctx, "k_norm_gemv", M, J.job[0].lin.kind, J.job[0].lin.O, P.K));
}

template <int M>
int launch_norm_gemv(orn_ctx* ctx, cudaStream_t s, const Prologue& P, RowJobs& J) {
  J.kinds_mask = 0;
  uint32_t slot = 0;
  if (P.mode == PRO_ADDNORM && P.K > 4 * kFusedThreads)
    ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: hidden size above 2048 is not supported by the norm prologue");
  for (int j = 0; j < J.njobs; ++j) {
    RowJob& job = J.job[j];
    J.kinds_mask |= 1 << job.lin.kind;
    if (job.lin.K != P.K) ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: weight K differs from the staged row");
    if (job.lin.K % 256) ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: K must be a multiple of 256");
    job.tasks = (job.lin.O + kRowsPerTask - 1) / kRowsPerTask;
    job.units = kind_units(job.lin.kind, job.lin.K);
    job.nchunk = row_chunks(job.lin.kind, job.lin.K);
    job.rb0 = units_bytes0(job.lin.kind, job.units);
    job.rb1 = units_bytes1(job.lin.kind, job.units);
    uint32_t rb = kRowsPerTask * chunk_bytes_max(job.lin.kind, job.lin.K);
    if (job.epi == EPI_SWIGLU) {
      if (job.lin2.kind != job.lin.kind || job.lin2.K != job.lin.K || job.lin2.O != job.lin.O)
        ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: gate and up projections must share format and shape");
      rb *= 2;
    }
    slot = rb > slot ? rb : slot;
  }
  // one instantiation per set of formats present, so that a kernel carries only the code it runs
  switch (J.kinds_mask) {
    case 1: return launch_norm_gemv_mask<M, 1>(ctx, s, P, J, slot);
    case 2: return launch_norm_gemv_mask<M, 2>(ctx, s, P, J, slot);
    case 4: return launch_norm_gemv_mask<M, 4>(ctx, s, P, J, slot);
    case 8: return launch_norm_gemv_mask<M, 8>(ctx, s, P, J, slot);
    case 5: return launch_norm_gemv_mask<M, 5>(ctx, s, P, J, slot);    // Q4_K + affine-8
    case 12: return launch_norm_gemv_mask<M, 12>(ctx, s, P, J, slot);  // affine-8 + bf16
    case 9: return launch_norm_gemv_mask<M, 9>(ctx, s, P, J, slot);    // Q4_K + bf16
    case 6: return launch_norm_gemv_mask<M, 6>(ctx, s, P, J, slot);    // Q6_K + affine-8
    default: return launch_norm_gemv_mask<M, 15>(ctx, s, P, J, slot);
  }
}

template <int KIND, int M>
int launch_moe_up_k(orn_ctx* ctx, cudaStream_t s, const MoeUpParams& P) {
  if (P.H % 256) ORN_FAIL(ctx, ORN_ERR_ARG, "moe_up: hidden must be a multiple of 256");
  const size_t fixed = stage_floats(KIND, M, P.H) * sizeof(float) + (size_t)M * P.k * 4;
  const size_t scratch = ((size_t)M * P.H + (size_t)M * P.E + M * 32 + M * P.k + 8) * sizeof(float);
  const uint32_t slot = 2 * kRowsPerTask * chunk_bytes_max(KIND, P.H);
  int depth;
  size_t bytes;
  int rc = plan_smem(ctx, fixed, scratch, slot, &depth, &bytes);
  if (rc != ORN_OK) return rc;
  rc = set_smem(ctx, k_moe_up<KIND, M>, bytes);
  if (rc != ORN_OK) return rc;
  k_moe_up<KIND, M><<<ctx->sm_count, kFusedThreads, bytes, s>>>(P, slot, depth, ctx->dev_err);
  return orn_launch_check(ctx, launch_label(ctx, "k_moe_up", M, KIND, P.I, P.H));
}

template <int KIND, int M>
int launch_moe_down_k(orn_ctx* ctx, cudaStream_t s, const MoeDownParams& P) {
  if (P.I % 256 || P.SI % 256) ORN_FAIL(ctx, ORN_ERR_ARG, "moe_down: intermediate sizes must be multiples of 256");
  const int rows = M * P.k;
  const size_t fixed = (stage_floats(KIND, rows, P.I) + stage_floats(KIND, M, P.SI) + 2 * rows + M) * sizeof(float);
  const size_t scratch = ((size_t)rows * P.I + (size_t)M * P.SI + 8) * sizeof(float);
  if (row_chunks(KIND, P.I) != 1 || row_chunks(KIND, P.SI) != 1)
    ORN_FAIL(ctx, ORN_ERR_ARG, "moe_down: intermediate size too long for one streamed chunk");
  if (P.H % kDownCols) ORN_FAIL(ctx, ORN_ERR_ARG, "moe_down: hidden must be even");
  const uint32_t r0 = chunk_bytes_max(KIND, P.I), r1 = chunk_bytes_max(KIND, P.SI);
  const uint32_t slot = kDownCols * (r0 > r1 ? r0 : r1);
  int depth;
  size_t bytes;
  int rc = plan_smem(ctx, fixed, scratch, slot, &depth, &bytes);
  if (rc != ORN_OK) return rc;
  rc = set_smem(ctx, k_moe_down<KIND, M>, bytes);
  if (rc != ORN_OK) return rc;
  k_moe_down<KIND, M><<<ctx->sm_count, kFusedThreads, bytes, s>>>(P, slot, depth, ctx->dev_err);
  return orn_launch_check(ctx, launch_label(ctx, "k_moe_down", M, KIND, P.H, P.I));
}

}  // namespace

int f_norm_gemv(orn_ctx* ctx, cudaStream_t s, int M, const FusedPrologue& fp, const FusedJob* jobs, int njobs) {
  if (njobs < 1 || njobs > 4) ORN_FAIL(ctx, ORN_ERR_ARG, "fused gemv: 1..4 jobs");
  Prologue P;
  P.mode = fp.mode; P.K = fp.K; P.a = fp.a; P.b = fp.b; P.w = fp.w; P.w2 = fp.w2; P.sum_out = fp.sum_out;
  P.norm_out = fp.norm_out; P.ids = fp.ids; P.eps = fp.eps;
  P.emb = fp.emb ? lin_dev(fp.emb) : LinDev{0, 0, 0, 0, nullptr, nullptr, nullptr};
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
  if (gate->kind != up->kind) ORN_FAIL(ctx, ORN_ERR_ARG, "moe: gate and up experts must share a format");
  MoeUpParams P;
  P.logits = logits; P.x = x; P.gate = lin_dev(gate); P.up = lin_dev(up); P.inds = inds; P.scores = scores;
  P.act = act; P.E = gate->E; P.k = k; P.H = gate->K; P.I = gate->O;
  if (P.E > 512) ORN_FAIL(ctx, ORN_ERR_ARG, "moe: more than 512 experts");
#define ORN_UP(KIND)                                                   \
  switch (M) {                                                         \
    case 1: return launch_moe_up_k<KIND, 1>(ctx, s, P);                \
    case 2: return launch_moe_up_k<KIND, 2>(ctx, s, P);                \
    case 3: return launch_moe_up_k<KIND, 3>(ctx, s, P);                \
    case 4: return launch_moe_up_k<KIND, 4>(ctx, s, P);                \
  }
  switch (gate->kind) {
    case ORN_Q4K: ORN_UP(ORN_Q4K) break;
    case ORN_Q6K: ORN_UP(ORN_Q6K) break;
    case ORN_A8: ORN_UP(ORN_A8) break;
    default: ORN_UP(ORN_BF16) break;
  }
#undef ORN_UP
  ORN_FAIL(ctx, ORN_ERR_ARG, "moe_up: 1..4 rows");
}

int f_moe_down(orn_ctx* ctx, cudaStream_t s, int M, const bf16_t* act, const bf16_t* sact, const uint32_t* inds,
               const bf16_t* scores, const bf16_t* gs, const orn_linear* down, const orn_linear* sh_down, int k,
               int normalize, bf16_t* out) {
  if (down->kind != sh_down->kind) ORN_FAIL(ctx, ORN_ERR_ARG, "moe: routed and shared down projections must share a format");
  MoeDownParams P;
  P.act = act; P.sact = sact; P.inds = inds; P.scores = scores; P.gs = gs; P.down = lin_dev(down);
  P.sh_down = lin_dev(sh_down); P.out = out; P.k = k; P.H = down->O; P.I = down->K; P.SI = sh_down->K;
  P.normalize = normalize;
  if (k > 8) ORN_FAIL(ctx, ORN_ERR_ARG, "moe: top_k above 8");
#define ORN_DN(KIND)                                                   \
  switch (M) {                                                         \
    case 1: return launch_moe_down_k<KIND, 1>(ctx, s, P);              \
    case 2: return launch_moe_down_k<KIND, 2>(ctx, s, P);              \
    case 3: return launch_moe_down_k<KIND, 3>(ctx, s, P);              \
    case 4: return launch_moe_down_k<KIND, 4>(ctx, s, P);              \
  }
  switch (down->kind) {
    case ORN_Q4K: ORN_DN(ORN_Q4K) break;
    case ORN_Q6K: ORN_DN(ORN_Q6K) break;
    case ORN_A8: ORN_DN(ORN_A8) break;
    default: ORN_DN(ORN_BF16) break;
  }
#undef ORN_DN
  ORN_FAIL(ctx, ORN_ERR_ARG, "moe_down: 1..4 rows");
}

int f_gdn(orn_ctx* ctx, cudaStream_t s, const bf16_t* conv, const bf16_t* cw, const bf16_t* a, const bf16_t* b,
          const bf16_t* a_log, const bf16_t* dt_bias, float* ring, int nring, const int* cur, int final_only, int T,
          int Hk, int Hv, int Kc, float eps, bf16_t* y) {
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
  dim3 grid(128 / kGdnRows, Hv);
  k_gdn<<<grid, kGdnRows * 4, 0, s>>>(p);
  return orn_launch_check(ctx, "k_gdn");
}

int f_attn(orn_ctx* ctx, cudaStream_t s, const bf16_t* qg, const bf16_t* k, const bf16_t* v, const bf16_t* q_norm,
           const bf16_t* k_norm, bf16_t* kc, bf16_t* vc, const int* pos, int T, int Hq, int Hkv, int hd, int cap,
           int rope_dims, float lnb, float eps, bf16_t* out) {
  if (hd != 256) ORN_FAIL(ctx, ORN_ERR_ARG, "fused attention: head_dim must be 256");
  if (T > kGdnMaxT) ORN_FAIL(ctx, ORN_ERR_ARG, "fused attention: at most 4 rows");
  AttnParams p;
  p.qg = qg; p.k = k; p.v = v; p.q_norm = q_norm; p.k_norm = k_norm; p.kc = kc; p.vc = vc; p.pos = pos; p.out = out;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.cap = cap; p.rope_dims = rope_dims; p.lnb = lnb;
  p.scale = 1.0f / sqrtf((float)hd);
  p.eps = eps;
  dim3 grid(Hq, T);
  k_attn<<<grid, 1024, 0, s>>>(p);
  return orn_launch_check(ctx, "k_attn");
}
