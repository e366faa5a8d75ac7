// Wide mat-mul on the 5th-generation tensor cores: y[rows, O] = x[rows, K] W^T for rows >= 16,
// with W in any of the library's weight formats.
//
// Replaces kquant::qmm_t / gather_qmm_t (src/ops/kquant.rs:783-812,905-972, kernels/kquant_mm.h:
// 88-360: a tile of weights is dequantised into threadgroup memory and multiplied by simdgroup
// matrices) and the prompt-width side of quantized_matmul / matmul (src/ops/quantized.rs:249-333,
// src/ops/matmul.rs:486-526).  The reference exempts this path from row invariance
// (src/generate.rs:99): a prompt row computed here does not carry the bits of the one-row
// mat-vec, it agrees with it to rounding (weights are rounded to bfloat16 once, products are
// accumulated in float32 by the tensor core).
//
// Shape of the kernel.  The contraction runs with the WEIGHTS as the A operand and the TOKENS as
// the B operand, D[feature, token] = sum_k W[feature, k] x[token, k]: the tensor core's M is always
// a full 128 features, its N is the token-tile width BN (16..256), so a launch with few tokens per
// expert (a routed prompt chunk, a batched decode step) wastes no tensor-core work on padding.
//   - a CTA owns (feature tile of 128, up to NT token tiles) and keeps NT accumulators of
//     128 x BN float32 in tensor memory (NT * BN <= 512 columns);
//   - per block of 64 weights along K: one warp's elected lane brings the NT token tiles
//     [BN, 64] bf16 and the raw bytes of the 128 x 64 weight tile with TMA (cp.async.bulk.tensor.2d,
//     this GPU's memory, no multicast); eight (or four) warps dequantise the tile (one thread per
//     feature row: Q4_K / Q6_K / affine-8 / affine-4 -> bf16) and store it with tcgen05.st into TENSOR
//     MEMORY, where the MMA takes its A operand from (row = lane, two bf16 per column): a 16 KB tile
//     per K block neither crosses shared memory twice nor needs a proxy fence (bf16 weights land in
//     shared memory swizzled and are read from there); another elected lane issues 4 * NT tcgen05.mma
//     (128 x BN x 16, kind::f16, bf16 inputs, f32 accumulate) and commits the stage back to the
//     producers;
//   - the eight dequantising warps then read the accumulators (tcgen05.ld, one TMEM lane = one
//     feature per thread), round to bfloat16 and store y[token, feature].
// Stages are a ring guarded by mbarriers; every wait is bounded and reports through the context's
// device error flag, and the CTA frees its tensor memory on every path.
//
// The grouped form serves rows sorted by expert (counting_sort + switch_glu_rows,
// src/ops/moe.rs:283-314,463-508): a small plan kernel turns the experts' row ranges into work
// items (expert, first row, rows, feature tile) and persistent CTAs walk that list.
#include <cuda.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <set>
#include <string>
#include <utility>

#include "fused.h"
#include "orn_internal.h"
#include "orn_quant.cuh"

namespace {

constexpr int BM = 128;            // features per tile: the tensor core's M
constexpr int BK = 64;             // weights per K block: one 128-byte swizzle row of bf16
// warp 0: TMA, warp 1: MMA, then DQW warps that dequantise and run the epilogue: 8 (two threads per
// feature row of a tile) for launches with one or two CTAs per SM, 4 (one thread per row) for
// launches of narrow items, where up to four small CTAs share an SM
constexpr int gemm_threads(int dqw) { return 64 + 32 * dqw; }
constexpr uint32_t kAccColsMax = 384;   // accumulator columns of an item: the rest of tensor memory holds weight tiles
constexpr uint32_t kWCols = BK / 2;     // tensor-memory columns of one dequantised 128 x 64 tile (two bf16 per column)
constexpr int kSplitMaxRows = 512;                      // dense products up to this many rows may split K
constexpr size_t kSplitPartialBytes = (size_t)64 << 20;  // f32 partials of one launch
constexpr size_t kSplitTiles = 4096;                     // arrival counters
constexpr uint32_t kWTileBytes = BM * BK * 2;
constexpr int kMaxIn = 12;  // IN ring slots (raw weight boxes + token tiles)
constexpr int kMaxW = 4;    // W ring slots (dequantised weight tile)
constexpr uint32_t kGemmWaitLimit = 1u << 16;  // try_wait rounds (each may sleep kGemmHintNs)
constexpr uint32_t kGemmHintNs = 20000;

constexpr int kMaxJobs = 4;  // matrices of one dense launch (projections that share their input rows)
struct GemmJob {
  int O, tile0;        // output features; first feature tile of this matrix in the launch's tile space
  int ldy;             // elements between output rows
  bf16_t* y;
  float* y_f32;        // non-null: float32 output instead of bfloat16
};
struct GemmParams {
  int njobs;
  GemmJob job[kMaxJobs];
  const int4* items;   // grouped: {expert, first row, rows, feature tile}; null = dense
  const int* n_items;  // grouped: device count
  int dense_items;     // dense: feature tiles x token groups
  int rows;            // rows of x (dense) / of the sorted row space (grouped)
  int K;
  const uint32_t* row_map;   // nullable: output row of sorted row p
  int BN, NT, stages /*IN ring*/, w_stages /*W ring*/, f_tiles;
  uint32_t stage_bytes;
  uint32_t tmem_cols;  // power of two >= acc_cols + the W ring's columns (and >= 32): what the CTA takes of tensor memory
  uint32_t acc_cols;   // NT * BN rounded up to 32: the accumulators; the dequantised weight tiles follow
  int splits;          // dense products over few rows: an item is one of `splits` ranges of the K blocks of a tile
  float* partial;      // [tile][split][token][128 features] f32 partial sums of the split items
  int* arrivals;       // [tile] how many splits of the tile have stored their partial (the last one reduces)
  int* err;
};

ORN_D uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
ORN_D void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
ORN_D void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
ORN_D void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
ORN_D bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kGemmHintNs)
      : "memory");
  return ok != 0;
}
// bounded wait: false (and the error flag set) when the phase never completes
ORN_D bool mbar_wait(uint32_t bar, uint32_t parity, int* err) {
  for (uint32_t it = 0; it < kGemmWaitLimit; ++it)
    if (mbar_try(bar, parity)) return true;
  atomicExch(err, 1);
  return false;
}
ORN_D void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
ORN_D void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
ORN_D void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
ORN_D void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
ORN_D void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, 128 x N x 16, bf16 in, f32 out
ORN_D void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// shared-memory operand descriptor: K-major, 128-byte swizzle, rows of 128 bytes, groups of 8 rows
// 1024 bytes apart (start >> 4 | LBO 1 | SBO 64 | version 1 | layout SWIZZLE_128B)
ORN_D uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
ORN_D void tmem_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}
ORN_D void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 16 registers of every lane to 16 columns of the warp's 32 tensor-memory lanes (lane i of the warp = row i)
ORN_D void tmem_st16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
      "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
ORN_D void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]^T: A is 128 lanes x 8 columns (16 bf16 of K per row)
ORN_D void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

ORN_D uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
ORN_D uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
ORN_D uint32_t lds16(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
// Four code bytes of a word -> two words of two bfloat16 each, w = a * q + b per byte q, in two
// packed fused multiply-adds on the code word itself: a code byte dropped into a float's bit
// pattern IS a float that is linear in the code.
//   * codes below 128 go into the third byte of 0x3F000000, already shifted left by s bits so that
//     they fill the byte's top (s = 3 for 4-bit codes, 1 for 6-bit ones): the float is
//     0.5 + (q << s) / 256, hence w = (a 2^(8-s)) * F + (b - a 2^(7-s)); both constants are exact
//     up to one float32 rounding of b - a 2^(7-s), which is of the size of w itself;
//   * 8-bit codes go into the second byte of 0x47000000: the float is 32768 + q and
//     w = a * F + (b - 32768 a), whose constant carries an error of a / 512 at most (far below the
//     bfloat16 rounding of an affine weight, which is of the size of 64 a).
// This path agrees with the mat-vec to rounding, not bit for bit.
template <int I>  // top-aligned code bytes I and I + 1 of w as a packed pair of floats
ORN_D uint64_t code_pair_hi(uint32_t w) {
  // selector nibbles, result byte 3..0: magic byte 3 (0x3F), code byte, magic bytes 1 and 0 (0)
  return pk2(__uint_as_float(__byte_perm(w, 0x3F000000u, 0x7054 + 256 * I)),
             __uint_as_float(__byte_perm(w, 0x3F000000u, 0x7054 + 256 * (I + 1))));
}
template <int I>  // 8-bit code bytes I and I + 1 of w as the packed pair (32768 + q_I, 32768 + q_I+1)
ORN_D uint64_t code_pair_8(uint32_t w) {
  return pk2(__uint_as_float(__byte_perm(w, 0x47000000u, 0x7604 + 16 * I)),
             __uint_as_float(__byte_perm(w, 0x47000000u, 0x7604 + 16 * (I + 1))));
}
ORN_D uint32_t bf2_of(uint64_t p) {  // packed pair of floats -> two bfloat16, the first in the low half
  uint32_t r;
  asm("{\n"
      ".reg .f32 x, y;\n"
      "mov.b64 {x, y}, %1;\n"
      "cvt.rn.bf16x2.f32 %0, y, x;\n"
      "}\n"
      : "=r"(r)
      : "l"(p));
  return r;
}
template <bool kEightBit>
ORN_D void codes4_bf(uint32_t w, uint64_t a2, uint64_t b2, uint32_t& o0, uint32_t& o1) {
  o0 = bf2_of(ffma2(a2, kEightBit ? code_pair_8<0>(w) : code_pair_hi<0>(w), b2));
  o1 = bf2_of(ffma2(a2, kEightBit ? code_pair_8<2>(w) : code_pair_hi<2>(w), b2));
}
// (w >> sh) << up for every byte's field, as one rotation (the bits that wrap land outside the mask)
ORN_D uint32_t field_up(uint32_t w, int sh, int up) { return __funnelshift_r(w, w, (sh - up) & 31); }

// The raw bytes of a K block arrive by TMA as boxes of [128 rows x 16 / 32 / 64 bytes] cut out of
// the row records (no swizzle: row r of a box is at r * box bytes).  A thread dequantises HALF of
// one feature row's K block: 32 weights -> 16 words of two bfloat16 each, in K order (word w of the
// half = weights 2w, 2w + 1), which become 16 tensor-memory columns of the row's lane.
//
// Raw tile layout per format (byte offsets inside the stage's raw area) and the record offsets
// (x coordinates, multiples of 16) the boxes are cut at, for K block kb (b = kb / 4):
//   Q4_K  [0, 4096)      codes, box 32:   x = b*128 + (kb&3)*32
//         [4096, 6144)   header, box 16:  x = b0 + b*16
//   Q6_K  [0, 8192)      ql, box 64:      x = b*192 + 64*half128          (half128 = (kb>>1)&1)
//         [8192, 12288)  qh, box 32:      x = b*192 + 128 + 32*half128
//         [12288, 14336) scales, box 16:  x = b0 + b*16
//         [14336, 16384) d, box 16:       x = b0 + b1 + ((2b) & ~15)
//   A8    [0, 8192)      codes, box 64:   x = kb*64
//         [8192, 10240)  {scale,bias}, box 16: x = b0 + ((4kb) & ~15)
//   A4    [0, 4096)      codes, box 32:   x = kb*32
//         [4096, 6144)   {scale,bias}, box 16: x = b0 + ((8kb) & ~15)
//   BF16  none: the [128 x 64] bf16 box lands in the MMA tile itself (128-byte swizzle)
template <int KIND> struct Fmt;

template <> struct Fmt<ORN_BF16> {
  static constexpr uint32_t kRawBytes = 0;
  ORN_D static void issue(const CUtensorMap*, const CUtensorMap*, const CUtensorMap*, const CUtensorMap* wsw, const RecGeom&,
                          int kb, int row, uint32_t raw, uint32_t wtile, uint32_t bar) {
    tma_load_2d(raw, wsw, kb * BK, row, bar);
  }
  static constexpr uint32_t kTxBytes = kWTileBytes;
  ORN_D static void convert(uint32_t, int, int, int, uint32_t*, const RecGeom&) {}
};

// affine 8-bit, group 64: w = scale * q + bias (one fma, as the embedding lookup computes it)
template <> struct Fmt<ORN_A8> {
  static constexpr uint32_t kRawBytes = 10240, kTxBytes = 8192 + 2048;
  ORN_D static void issue(const CUtensorMap* m64, const CUtensorMap*, const CUtensorMap* m16, const CUtensorMap*, const RecGeom& g,
                          int kb, int row, uint32_t raw, uint32_t, uint32_t bar) {
    tma_load_2d(raw, m64, kb * 64, row, bar);
    tma_load_2d(raw + 8192, m16, (int)g.b0 + ((4 * kb) & ~15), row, bar);
  }
  ORN_D static void convert(uint32_t raw, int r, int kb, int half, uint32_t* out, const RecGeom&) {
    const uint4 q0 = lds128(raw + r * 64 + half * 32), q1 = lds128(raw + r * 64 + half * 32 + 16);
    const uint32_t sb = lds32(raw + 8192 + r * 16 + ((4 * kb) & 15));
    const float sc = bf_lo(sb), bi = fmaf(-32768.0f, sc, bf_hi(sb));
    const uint64_t a2 = pk2(sc, sc), b2 = pk2(bi, bi);
    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) codes4_bf<true>(w[i], a2, b2, out[2 * i], out[2 * i + 1]);
  }
};

// affine 4-bit, group 32: half a K block is one group; byte b holds weights 2b (low nibble), 2b+1 (high)
template <> struct Fmt<ORN_A4> {
  static constexpr uint32_t kRawBytes = 6144, kTxBytes = 4096 + 2048;
  ORN_D static void issue(const CUtensorMap*, const CUtensorMap* m32, const CUtensorMap* m16, const CUtensorMap*, const RecGeom& g,
                          int kb, int row, uint32_t raw, uint32_t, uint32_t bar) {
    tma_load_2d(raw, m32, kb * 32, row, bar);
    tma_load_2d(raw + 4096, m16, (int)g.b0 + ((8 * kb) & ~15), row, bar);
  }
  ORN_D static void convert(uint32_t raw, int r, int kb, int half, uint32_t* out, const RecGeom&) {
    const uint4 q = lds128(raw + r * 32 + half * 16);
    const uint32_t sb = lds32(raw + 4096 + r * 16 + ((8 * kb) & 15) + 4 * half);
    const float sc = bf_lo(sb), a32 = 32.0f * sc, bi = fmaf(-16.0f, sc, bf_hi(sb));
    const uint64_t a2 = pk2(a32, a32), b2 = pk2(bi, bi);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // one word = 8 weights = 4 words of bfloat16 pairs (low nibble first)
      const uint32_t l4 = field_up(w[c], 0, 3) & 0x78787878u, h4 = field_up(w[c], 4, 3) & 0x78787878u;
      // weights 2b, 2b + 1 = (low, high) nibble of byte b: interleave the two nibble words bytewise
      codes4_bf<false>(__byte_perm(l4, h4, 0x5140), a2, b2, out[4 * c], out[4 * c + 1]);
      codes4_bf<false>(__byte_perm(l4, h4, 0x7362), a2, b2, out[4 * c + 2], out[4 * c + 3]);
    }
  }
};

// Q4_K (kernels/q4k.metal:43-96): a K block is 32 code bytes; low nibbles are sub-block 2i (the first
// half of the K block), high nibbles sub-block 2i+1 (the second half); w = (d * sc) * q - dmin * m,
// evaluated as one fma per weight (this path agrees with the mat-vec to rounding, not bit for bit)
template <> struct Fmt<ORN_Q4K> {
  static constexpr uint32_t kRawBytes = 6144, kTxBytes = 4096 + 2048;
  ORN_D static void issue(const CUtensorMap*, const CUtensorMap* m32, const CUtensorMap* m16, const CUtensorMap*, const RecGeom& g,
                          int kb, int row, uint32_t raw, uint32_t, uint32_t bar) {
    tma_load_2d(raw, m32, (kb >> 2) * 128 + (kb & 3) * 32, row, bar);
    tma_load_2d(raw + 4096, m16, (int)g.b0 + (kb >> 2) * 16, row, bar);
  }
  ORN_D static void convert(uint32_t raw, int r, int kb, int half, uint32_t* out, const RecGeom&) {
    const uint4 qa = lds128(raw + r * 32), qb = lds128(raw + r * 32 + 16), hdr = lds128(raw + 4096 + r * 16);
    const float d = h2f((uint16_t)(hdr.x & 0xffff)), dmin = h2f((uint16_t)(hdr.x >> 16));
    float sc, m;
    q4k_scale_min(2 * (kb & 3) + half, hdr.y, hdr.z, hdr.w, &sc, &m);
    const float a = d * sc, a32 = 32.0f * a, nb = fmaf(-16.0f, a, -(dmin * m));
    const uint64_t a2 = pk2(a32, a32), b2 = pk2(nb, nb);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    const int sh = 4 * half;
#pragma unroll
    for (int i = 0; i < 8; ++i) codes4_bf<false>(field_up(w[i], sh, 3) & 0x78787878u, a2, b2, out[2 * i], out[2 * i + 1]);
  }
};

// Q6_K (kernels/q6k.metal:47-77): per 128 weights, byte l of ql / qh gives q1 (weight l), q2 (l + 32),
// q3 (l + 64), q4 (l + 96); a K block of 64 is (q1, q2) or (q3, q4) of one half-block, this thread's
// half of it one of the two code sets; w = (d * sc) * (q - 32)
template <> struct Fmt<ORN_Q6K> {
  static constexpr uint32_t kRawBytes = 16384, kTxBytes = 8192 + 4096 + 2048 + 2048;
  ORN_D static void issue(const CUtensorMap* m64, const CUtensorMap* m32, const CUtensorMap* m16, const CUtensorMap*,
                          const RecGeom& g, int kb, int row, uint32_t raw, uint32_t, uint32_t bar) {
    const int b = kb >> 2, half128 = (kb >> 1) & 1;
    tma_load_2d(raw, m64, b * 192 + 64 * half128, row, bar);
    tma_load_2d(raw + 8192, m32, b * 192 + 128 + 32 * half128, row, bar);
    tma_load_2d(raw + 12288, m16, (int)g.b0 + b * 16, row, bar);
    tma_load_2d(raw + 14336, m16, (int)(g.b0 + g.b1) + ((2 * b) & ~15), row, bar);
  }
  ORN_D static void convert(uint32_t raw, int r, int kb, int set, uint32_t* out, const RecGeom&) {
    const int b = kb >> 2, half128 = (kb >> 1) & 1, hi = kb & 1;
    const uint4 l0 = lds128(raw + r * 64 + 32 * set), l1 = lds128(raw + r * 64 + 32 * set + 16);
    const uint4 h0 = lds128(raw + 8192 + r * 32), h1 = lds128(raw + 8192 + r * 32 + 16);
    const uint32_t sc2 = lds16(raw + 12288 + r * 16 + 8 * half128 + 4 * hi + 2 * set);
    const float d = h2f((uint16_t)lds16(raw + 14336 + r * 16 + ((2 * b) & 15)));
    const float s0 = d * (float)(int8_t)(sc2 & 0xff), s1 = d * (float)(int8_t)(sc2 >> 8);
    // w = s (q - 32) = 128 s (0.5 + q / 128) - 96 s
    const uint64_t a20 = pk2(128.0f * s0, 128.0f * s0), a21 = pk2(128.0f * s1, 128.0f * s1);
    const uint64_t b20 = pk2(-96.0f * s0, -96.0f * s0), b21 = pk2(-96.0f * s1, -96.0f * s1);
    const uint32_t lw[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
    const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
    const int hs = 2 * set + 4 * hi;  // bit position of this code set's two high bits in qh
    const int ls = 4 * hi;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t q = (field_up(lw[i], ls, 1) & 0x1E1E1E1Eu) | (field_up(hw[i], hs, 5) & 0x60606060u);  // code << 1
      codes4_bf<false>(q, i < 4 ? a20 : a21, i < 4 ? b20 : b21, out[2 * i], out[2 * i + 1]);
    }
  }
};

struct Item {
  int e, tok0, ntok, ft;
  int kb0, kb1;  // K blocks of this item
  int tile, split;
  int job;       // which matrix of the launch (ft counts inside it)
};
ORN_D bool get_item(const GemmParams& P, int w, int n_items, Item& it) {
  if (w >= n_items) return false;
  if (P.items != nullptr) {
    const int4 v = P.items[w];
    it.e = v.x; it.tok0 = v.y; it.ntok = v.z; it.ft = v.w;
    it.kb0 = 0; it.kb1 = P.K / BK; it.tile = w; it.split = 0; it.job = 0;
    while (it.job + 1 < P.njobs && it.ft >= P.job[it.job + 1].tile0) ++it.job;
    it.ft -= P.job[it.job].tile0;
  } else {
    const int tile = w / P.splits;
    const int g = tile / P.f_tiles;
    it.e = 0;
    it.ft = tile - g * P.f_tiles;
    it.job = 0;
    while (it.job + 1 < P.njobs && it.ft >= P.job[it.job + 1].tile0) ++it.job;
    it.ft -= P.job[it.job].tile0;
    it.tok0 = g * P.NT * P.BN;
    it.ntok = min(P.NT * P.BN, P.rows - it.tok0);
    const int KB = P.K / BK, per = (KB + P.splits - 1) / P.splits;
    it.tile = tile; it.split = w - tile * P.splits;
    it.kb0 = it.split * per; it.kb1 = min(KB, it.kb0 + per);
  }
  return true;
}

struct WeightMaps {
  CUtensorMap w64;  // row records as bytes [E*O, rec], boxes [128, 64] / [128, 32] / [128, 16], no swizzle
  CUtensorMap w32;
  CUtensorMap w16;
  CUtensorMap wsw;  // bf16 weights only: [E*O, K] bf16, box [128, 64], 128-byte swizzle
};
struct GemmMaps {
  CUtensorMap x;    // tokens [rows, K] bf16, box [BN, 64], 128-byte swizzle
  WeightMaps w[kMaxJobs];
};

// Two rings per CTA.  The IN ring in shared memory (deep: TMA latency is a few thousand cycles) holds
// what TMA brings per K block: the raw weight boxes and the token tiles.  The W ring in tensor memory
// (two or three slots of 32 columns behind the accumulators) holds the dequantised weight tile the
// MMAs read as their A operand.  bf16 weights need no dequantisation: their box lands swizzled in the
// IN ring and the MMAs read it there (A from shared memory).
//   landed[i]   TMA boxes of IN slot i arrived            (producer's expect_tx)
//   full[w]     W slot w dequantised                       (one arrival per dequantising warp)
//   in_free[i]  the MMAs that read IN slot i are done      (tcgen05.commit)
//   w_free[w]   the MMAs that read W slot w are done       (tcgen05.commit)
template <int KIND, int DQW>
__global__ void __launch_bounds__(gemm_threads(DQW), DQW == 4 ? 4 : 1) k_qgemm(const __grid_constant__ GemmMaps maps, GemmParams P) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_bar[2 * kMaxIn + 2 * kMaxW + 2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_last;  // split-K: this CTA stored the last partial of its tile and reduces it
  using F = Fmt<KIND>;
  constexpr bool kDirect = KIND == ORN_BF16;  // the MMA reads the weight box where TMA put it
  constexpr uint32_t kInRaw = kDirect ? kWTileBytes : F::kRawBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem0 = (smem_addr(smem_raw) + 1023u) & ~1023u;  // swizzled tiles want 1024-byte alignment
  const int SI = P.stages, SW = P.w_stages;
  const uint32_t in0 = smem0;
  const uint32_t bar_landed = smem_addr(&s_bar[0]), bar_in_free = smem_addr(&s_bar[kMaxIn]);
  const uint32_t bar_full = smem_addr(&s_bar[2 * kMaxIn]), bar_w_free = smem_addr(&s_bar[2 * kMaxIn + kMaxW]);
  const uint32_t bar_acc_full = smem_addr(&s_bar[2 * kMaxIn + 2 * kMaxW]), bar_acc_empty = bar_acc_full + 8;
  if (threadIdx.x == 0) {
    for (int i = 0; i < SI; ++i) {
      mbar_init(bar_landed + 8 * i, 1);
      mbar_init(bar_in_free + 8 * i, 1);
    }
    for (int i = 0; i < SW; ++i) {
      mbar_init(bar_full + 8 * i, DQW);
      mbar_init(bar_w_free + 8 * i, 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, DQW);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  __syncwarp();
  if (warp == 0) {  // tensor memory: the columns of one item's accumulators (two CTAs of a narrow launch share an SM)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&s_tmem)), "r"(P.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  const int n_items = P.items != nullptr ? *P.n_items : P.dense_items;
  const uint32_t x_tile_bytes = (uint32_t)P.BN * 128u;
  const RecGeom geo = rec_geom(KIND, P.K);

  if (warp == 0) {
    // ---- TMA producer: the raw weight boxes and the token tiles of every K block
    if (lane == 0) {
      // ring positions are counted, not divided: an integer division is a hundred cycles of this one thread
      int si = 0;
      uint32_t si_ph = 0;
      Item w;
      bool ok = true;
      for (int wi = blockIdx.x; ok && get_item(P, wi, n_items, w); wi += gridDim.x) {
        const int nt = (w.ntok + P.BN - 1) / P.BN;
        const int wrow = w.e * P.job[w.job].O + w.ft * BM;
        const WeightMaps& wm = maps.w[w.job];
        for (int kb = w.kb0; kb < w.kb1; ++kb, si = (si + 1 == SI ? 0 : si + 1), si_ph ^= (si == 0 ? 1u : 0u)) {
          ok = mbar_wait(bar_in_free + 8 * si, si_ph ^ 1u, P.err);
          if (!ok) break;
          const uint32_t bar = bar_landed + 8 * si, base = in0 + si * P.stage_bytes;
          mbar_expect_tx(bar, (uint32_t)nt * x_tile_bytes + F::kTxBytes);
          F::issue(&wm.w64, &wm.w32, &wm.w16, &wm.wsw, geo, kb, wrow, base, base, bar);
          for (int t = 0; t < nt; ++t) tma_load_2d(base + kInRaw + t * x_tile_bytes, &maps.x, kb * BK, w.tok0 + t * P.BN, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(P.BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      uint32_t acc_ph = 0, sw_ph = 0;
      int si = 0, sw = 0;
      Item w;
      bool ok = true;
      for (int wi = blockIdx.x; ok && get_item(P, wi, n_items, w); wi += gridDim.x) {
        const int nt = (w.ntok + P.BN - 1) / P.BN;
        ok = mbar_wait(bar_acc_empty, acc_ph ^ 1u, P.err);  // the previous item's accumulators were read
        tc_fence_after();
        for (int kb = w.kb0; kb < w.kb1 && ok;
             ++kb, si = (si + 1 == SI ? 0 : si + 1), sw = (sw + 1 == SW ? 0 : sw + 1), sw_ph ^= (sw == 0 ? 1u : 0u)) {
          ok = mbar_wait(bar_full + 8 * sw, sw_ph, P.err);  // implies landed[si]: the dequantisers waited for it
          if (!ok) break;
          tc_fence_after();
          const uint32_t inb = in0 + si * P.stage_bytes;
          const uint32_t xa = inb + kInRaw;
          const uint32_t wt = tmem + P.acc_cols + (uint32_t)sw * kWCols;  // this K block's weight tile in tensor memory
          for (int t = 0; t < nt; ++t)
#pragma unroll
            for (int j = 0; j < BK / 16; ++j) {
              const uint64_t xb = smem_desc(xa + t * x_tile_bytes + j * 32);
              if (kDirect) tc_mma(tmem + (uint32_t)(t * P.BN), smem_desc(inb + j * 32), xb, idesc, (kb > w.kb0 || j > 0) ? 1u : 0u);
              else tc_mma_ts(tmem + (uint32_t)(t * P.BN), wt + j * 8, xb, idesc, (kb > w.kb0 || j > 0) ? 1u : 0u);
            }
          tc_commit(bar_in_free + 8 * si);  // both slots are free once these MMAs have read them
          tc_commit(bar_w_free + 8 * sw);
        }
        if (!ok) break;
        tc_commit(bar_acc_full);
        acc_ph ^= 1u;
      }
    }
  } else {
    // ---- dequantising warps, then the epilogue of the item
    const int dq = threadIdx.x - 64;   // 0 .. 32 * DQW - 1
    const int q = warp & 3;            // tensor-memory lane quadrant this warp may touch
    const int r = 32 * q + lane;       // feature row of the tile this thread dequantises = its tensor-memory lane
    const int colhalf = (warp - 2) >> 2;  // DQW == 8: the two warps of a quadrant split a K block's weights and the
                                          // epilogue's 16-column groups (DQW == 4: one warp does both halves)
    uint32_t acc_ph = 0, si_ph = 0, sw_ph = 0;
    int si = 0, sw = 0;
    Item w;
    bool ok = true;
    for (int wi = blockIdx.x; ok && get_item(P, wi, n_items, w); wi += gridDim.x) {
      for (int kb = w.kb0; kb < w.kb1; ++kb, si = (si + 1 == SI ? 0 : si + 1), si_ph ^= (si == 0 ? 1u : 0u),
               sw = (sw + 1 == SW ? 0 : sw + 1), sw_ph ^= (sw == 0 ? 1u : 0u)) {
        ok = mbar_wait(bar_w_free + 8 * sw, sw_ph ^ 1u, P.err) && mbar_wait(bar_landed + 8 * si, si_ph, P.err);
        if (!ok) break;
        if (!kDirect) {
          tc_fence_after();  // the MMAs that read this slot's last tile are done (w_free)
          const uint32_t wt = tmem + ((uint32_t)(q * 32) << 16) + P.acc_cols + (uint32_t)sw * kWCols;
          uint32_t o[16];
          if (DQW == 8) {
            F::convert(in0 + si * P.stage_bytes, r, kb, colhalf, o, geo);
            tmem_st16(wt + 16 * colhalf, o);
          } else {
            F::convert(in0 + si * P.stage_bytes, r, kb, 0, o, geo);
            tmem_st16(wt, o);
            F::convert(in0 + si * P.stage_bytes, r, kb, 1, o, geo);
            tmem_st16(wt + 16, o);
          }
          tmem_st_wait();
          tc_fence_before();  // ordered before the MMA thread's reads through the barrier below
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full + 8 * sw);
      }
      if (ok) ok = mbar_wait(bar_acc_full, acc_ph, P.err);
      if (P.splits > 1) {
        // the warps of a split item meet at named barriers below: they leave together or not at all
        // (a warp whose bounded wait ran out still comes here, and its verdict is everybody's)
        uint32_t all;
        asm volatile(
            "{\n"
            ".reg .pred p, q;\n"
            "setp.ne.u32 q, %1, 0;\n"
            "barrier.red.and.pred p, 1, %2, q;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(all)
            : "r"(ok ? 1u : 0u), "n"(DQW * 32)
            : "memory");
        ok = all != 0;
      }
      if (!ok) break;
      acc_ph ^= 1u;
      tc_fence_after();
      const GemmJob& J = P.job[w.job];
      const int fo = w.ft * BM + q * 32 + lane;  // TMEM lane = feature
      const int nt = (w.ntok + P.BN - 1) / P.BN;
      // split-K items store f32 partials [token][128 features] instead of results
      float* part = P.splits > 1 ? P.partial + (size_t)(w.tile * P.splits + w.split) * (size_t)(P.NT * P.BN) * BM : nullptr;
      for (int t = 0; t < nt; ++t) {
        for (int c0 = 16 * colhalf; c0 < P.BN; c0 += (DQW == 8 ? 32 : 16)) {
          if (t * P.BN + c0 >= w.ntok) break;  // warp-uniform
          uint32_t v[16];
          tmem_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(t * P.BN + c0), v);
          tmem_ld_wait();
          if (part != nullptr) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int tok = t * P.BN + c0 + j;
              if (tok < w.ntok) part[(size_t)tok * BM + q * 32 + lane] = __uint_as_float(v[j]);
            }
          } else if (fo < J.O) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int tok = t * P.BN + c0 + j;
              if (tok < w.ntok) {
                const size_t orow = P.row_map != nullptr ? P.row_map[w.tok0 + tok] : (size_t)(w.tok0 + tok);
                if (J.y_f32 != nullptr) J.y_f32[orow * J.ldy + fo] = __uint_as_float(v[j]);
                else J.y[orow * J.ldy + fo] = f2bf(__uint_as_float(v[j]));
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty);
      if (part != nullptr) {
        // the CTA that stores a tile's last partial adds the partials in split order (a fixed order:
        // the result does not depend on which CTA comes last) and writes the tile
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(DQW * 32) : "memory");
        if (dq == 0) s_last = atomicAdd(&P.arrivals[w.tile], 1) == P.splits - 1 ? 1 : 0;
        asm volatile("bar.sync 1, %0;" ::"n"(DQW * 32) : "memory");
        if (s_last) {
          __threadfence();
          const float4* base = reinterpret_cast<const float4*>(P.partial + (size_t)w.tile * P.splits * (size_t)(P.NT * P.BN) * BM);
          const size_t stride4 = (size_t)(P.NT * P.BN) * BM / 4;
          const int n4 = w.ntok * (BM / 4);
          constexpr int kU = 4;  // float4 pieces per thread and round: their loads are in flight together
          for (int i0 = dq; i0 < n4; i0 += kU * DQW * 32) {
            float4 acc[kU];
#pragma unroll
            for (int u = 0; u < kU; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sp = 0; sp < P.splits; ++sp) {
              float4 v[kU];
#pragma unroll
              for (int u = 0; u < kU; ++u) {
                const int i = i0 + u * DQW * 32;
                v[u] = i < n4 ? __ldcg(base + sp * stride4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
              for (int u = 0; u < kU; ++u) { acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w; }
            }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
              const int i = i0 + u * DQW * 32;
              if (i >= n4) continue;
              const int tok = i / (BM / 4), f = 4 * (i - tok * (BM / 4));
              const int feat = w.ft * BM + f;
              const size_t orow = (size_t)(w.tok0 + tok);
              const float r4[4] = {acc[u].x, acc[u].y, acc[u].z, acc[u].w};
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (feat + e < J.O) {
                  if (J.y_f32 != nullptr) J.y_f32[orow * J.ldy + feat + e] = r4[e];
                  else J.y[orow * J.ldy + feat + e] = f2bf(r4[e]);
                }
            }
          }
          if (dq == 0) P.arrivals[w.tile] = 0;  // ready for the next launch
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(P.tmem_cols) : "memory");
  }
}

// ---- grouped form: plan and row movement --------------------------------------------------------
// counts[e] = rows routed to expert e (block-wide histogram), then seg[e] = exclusive scan
__global__ void k_route_count(const uint32_t* rhs, int rows, int E, int* seg /*[E+1]*/, int* cursor /*[E]*/) {
  extern __shared__ int s_cnt[];
  for (int i = threadIdx.x; i < E; i += blockDim.x) s_cnt[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < rows; i += blockDim.x) {
    const uint32_t e = rhs[i];
    if (e < (uint32_t)E) atomicAdd(&s_cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      seg[e] = acc;
      cursor[e] = acc;
      acc += s_cnt[e];
    }
    seg[E] = acc;
  }
}
// stable placement: sorted position of row i = seg[e] + (number of earlier rows with the same expert).
// One warp per expert scans the routing table in order, so the order inside an expert is the
// original order (counting_sort, src/ops/moe.rs:463-508).
__global__ void k_route_place(const uint32_t* rhs, int rows, int E, const int* seg, uint32_t* perm /*[rows]: sorted -> original*/) {
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (e >= E) return;
  int pos = seg[e];
  for (int base = 0; base < rows; base += 32) {
    const int i = base + lane;
    const bool mine = i < rows && rhs[i] == (uint32_t)e;
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (mine) perm[pos + __popc(m & ((1u << lane) - 1u))] = (uint32_t)i;
    pos += __popc(m);
  }
}
// the same placement for long tables, one thread per row: the slot inside an expert is taken from a
// cursor, so the order inside an expert is arbitrary (every row's result is independent of its
// neighbours, and results are stored by original row index)
__global__ void k_route_place_atomic(const uint32_t* rhs, int rows, int E, int* cursor, uint32_t* perm) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows) return;
  const uint32_t e = rhs[i];
  if (e < (uint32_t)E) perm[atomicAdd(&cursor[e], 1)] = (uint32_t)i;
}
// xs[p] = x[lhs[perm[p]]] (rows of K bf16)
__global__ void k_gather_rows(const bf16_t* x, const uint32_t* lhs, const uint32_t* perm, int rows, int K, bf16_t* xs) {
  const int p = blockIdx.x;
  if (p >= rows) return;
  const uint32_t o = perm[p];
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(lhs ? lhs[o] : o) * K);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)p * K);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = src[i];
}
// work items of the grouped launch: expert e's rows in groups of `span`, every feature tile
__global__ void k_plan_items(const int* seg, int E, int span, int f_tiles, int4* items, int* n_items, int max_items) {
  __shared__ int s_off[1025];
  const int e = threadIdx.x;
  int mine = 0;
  if (e < E) mine = ((seg[e + 1] - seg[e] + span - 1) / span) * f_tiles;
  s_off[e + 1] = mine;
  if (e == 0) s_off[0] = 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i <= (int)blockDim.x; ++i) s_off[i] += s_off[i - 1];
    *n_items = min(s_off[blockDim.x], max_items);
  }
  __syncthreads();
  if (e < E) {
    int at = s_off[e];
    const int first = seg[e], n = seg[e + 1] - seg[e];
    for (int g = 0; g * span < n; ++g)
      for (int ft = 0; ft < f_tiles; ++ft, ++at)
        if (at < max_items) items[at] = make_int4(e, first + g * span, min(span, n - g * span), ft);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

std::mutex g_gemm_mu;
std::set<std::pair<int, int>> g_gemm_granted;  // (device, format and warp count): shared-memory limit raised

template <int KIND, int DQW>
int launch_qgemm(orn_ctx* ctx, cudaStream_t s, const GemmMaps& maps, const GemmParams& P, int grid, size_t smem) {
  {
    std::lock_guard<std::mutex> lock(g_gemm_mu);
    if (!g_gemm_granted.count({ctx->device, KIND * 16 + DQW})) {
      ORN_CHECK_CUDA(ctx, cudaFuncSetAttribute(k_qgemm<KIND, DQW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));  // + static barriers
      g_gemm_granted.insert({ctx->device, KIND * 16 + DQW});
    }
  }
  k_qgemm<KIND, DQW><<<grid, gemm_threads(DQW), smem, s>>>(maps, P);
  if (ctx->kt == nullptr) return orn_launch_check(ctx, "k_qgemm");
  // per-kernel timing: one label per shape
  static std::set<std::string> pool;
  char buf[96];
  snprintf(buf, sizeof buf, "k_qgemm kind=%d O=%d%s K=%d rows=%d %s", KIND, P.job[0].O, P.njobs > 1 ? "+" : "", P.K, P.rows, P.items ? "grouped" : "dense");
  std::lock_guard<std::mutex> lock(g_gemm_mu);
  return orn_launch_check(ctx, pool.insert(buf).first->c_str());
}

uint32_t raw_bytes(int kind) {
  switch (kind) {
    case ORN_Q4K: return Fmt<ORN_Q4K>::kRawBytes;
    case ORN_Q6K: return Fmt<ORN_Q6K>::kRawBytes;
    case ORN_A8: return Fmt<ORN_A8>::kRawBytes;
    case ORN_A4: return Fmt<ORN_A4>::kRawBytes;
    default: return 0;
  }
}

}  // namespace

// device scratch of the grouped form: the item count, then the work items (an expert contributes
// one item per feature tile and started group of rows; groups hold at least 128 rows)
size_t qgemm_scratch_bytes(int rows, int E, int O) {
  const int f_tiles = (O + BM - 1) / BM;
  const size_t max_items = (size_t)f_tiles * ((size_t)E + rows / 128 + 1);
  return 256 + max_items * sizeof(int4);
}

// y[rows, O] (row stride ldy) = x[rows, K] W^T.  grp != null: rows are sorted by expert, expert e
// owns rows seg[e] .. seg[e+1]-1 (device array of E + 1 ints) and multiplies by W[e]; row p of the
// result goes to output row row_map[p] when row_map is given.  scratch: qgemm_scratch_bytes() of
// device memory for the grouped form.
int f_qgemm(orn_ctx* ctx, cudaStream_t s, const orn_linear* L, const bf16_t* x, int rows, void* y, int ldy,
            const QGemmGroup* grp, void* scratch, int out_f32, int bn_force) {
  return f_qgemm_multi(ctx, s, &L, &y, &ldy, 1, x, rows, grp, scratch, out_f32, bn_force);
}

// Up to four matrices of one format and row length over the same rows in ONE launch (the projections
// of a layer that share their input): their feature tiles form one tile space.  n == 1 is f_qgemm.
int f_qgemm_multi(orn_ctx* ctx, cudaStream_t s, const orn_linear* const* Ls, void* const* ys, const int* ldys, int n,
                  const bf16_t* x, int rows, const QGemmGroup* grp, void* scratch, int out_f32, int bn_force) {
  if (rows < 1) return ORN_OK;
  if (n < 1 || n > kMaxJobs) ORN_FAIL(ctx, ORN_ERR_ARG, "gemm: 1..4 matrices per launch");
  const orn_linear* L = Ls[0];
  for (int j = 1; j < n; ++j)
    if (Ls[j]->kind != L->kind || Ls[j]->K != L->K || Ls[j]->E != L->E)
      ORN_FAIL(ctx, ORN_ERR_ARG, "gemm: the matrices of one launch share format and row length");
  if (L->K % BK) ORN_FAIL(ctx, ORN_ERR_ARG, "gemm: K must be a multiple of 64");
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) ORN_FAIL(ctx, ORN_ERR_ARG, "gemm: x must be 16-byte aligned");
  if (grp == nullptr && L->E != 1) ORN_FAIL(ctx, ORN_ERR_ARG, "gemm: a routed weight goes through the grouped form");
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr) ORN_FAIL(ctx, ORN_ERR_CUDA, "gemm: the driver has no cuTensorMapEncodeTiled");
  GemmParams P;
  P.njobs = n;
  P.f_tiles = 0;
  for (int j = 0; j < n; ++j) {
    GemmJob& J = P.job[j];
    J.O = Ls[j]->O; J.tile0 = P.f_tiles; J.ldy = ldys[j];
    J.y = out_f32 ? nullptr : reinterpret_cast<bf16_t*>(ys[j]);
    J.y_f32 = out_f32 ? reinterpret_cast<float*>(ys[j]) : nullptr;
    P.f_tiles += (Ls[j]->O + BM - 1) / BM;
  }
  P.K = L->K; P.rows = rows; P.err = ctx->dev_err;
  P.row_map = grp ? grp->row_map : nullptr;
  // token-tile width: wide tiles when there are many tokens per weight tile, narrow ones otherwise
  int per = grp ? (rows + L->E - 1) / L->E : rows;  // expected tokens per weight tile
  if (grp && grp->bn_hint > 0) per = grp->bn_hint;
  int BN = per >= 128 ? 128 : ((per + 15) / 16) * 16;
  if (BN < 16) BN = 16;
  if (bn_force > 0) BN = bn_force;  // a caller that wants one tile shape whatever the row count
  P.BN = BN;
  // tokens per item: 256 for dense products over many rows (a weight tile is dequantised once for
  // all of them; more would leave the IN ring too shallow to cover the TMA latency), a few tiles for
  // routed rows (an expert with more rows than that takes several items)
  P.NT = (int)kAccColsMax / BN;
  if (grp == nullptr) P.NT = std::min(std::min(P.NT, (rows + BN - 1) / BN), BN >= 128 ? 2 : 8);
  else P.NT = std::min(P.NT, BN >= 64 ? 4 : 2);
  if (P.NT > 8) P.NT = 8;
  // shared memory: as many IN slots as fit (TMA latency wants depth); tensor memory: the accumulators, then the W ring
  const uint32_t in_raw = L->kind == ORN_BF16 ? kWTileBytes : raw_bytes(L->kind);
  P.stage_bytes = in_raw + (uint32_t)P.NT * BN * 128u;
  P.acc_cols = ((uint32_t)(P.NT * BN) + 31u) & ~31u;
  const bool direct = L->kind == ORN_BF16;
  auto tmem_need = [&](int ws) {  // power of two that holds the accumulators and ws weight tiles
    uint32_t c = 32;
    while (c < P.acc_cols + (direct ? 0u : (uint32_t)ws * kWCols)) c <<= 1;
    return c;
  };
  P.tmem_cols = tmem_need(2);
  // Dense products over few rows are one token group: the K loop of an item is a chain of short
  // latency-bound steps (about 0.65 us per K block), so the blocks of a tile are split over several
  // CTAs whose f32 partials the last of them adds in split order.  The number of splits depends on
  // (O, K) only, never on the row count, so that a row's bits do not depend on how many rows share
  // the launch.
  P.splits = 1; P.partial = nullptr; P.arrivals = nullptr;
  if (grp == nullptr && rows <= kSplitMaxRows && L->K / BK >= 8) {
    const int tiles = P.f_tiles * ((rows + P.NT * BN - 1) / (P.NT * BN));
    // one round of items over the SMs, two CTAs on each where the tiles alone would leave SMs idle
    // (97 tiles of an input projection: three splits instead of none)
    int sp = std::max(1, (tiles > ctx->sm_count / 2 ? 2 * ctx->sm_count : ctx->sm_count) / tiles);
    sp = std::min(sp, std::min(8, L->K / BK / 4));               // at least 4 K blocks per item
    if (sp > 1) {                                                 // no split may be empty
      const int KBn = L->K / BK, per = (KBn + sp - 1) / sp;
      sp = (KBn + per - 1) / per;
    }
    const int groups = (rows + P.NT * BN - 1) / (P.NT * BN);
    const size_t need = (size_t)P.f_tiles * groups * sp * (size_t)(P.NT * BN) * BM * sizeof(float);
    if (sp > 1 && need <= kSplitPartialBytes && (size_t)P.f_tiles * groups <= kSplitTiles) {
      // products on the side stream run beside products on the main one: a scratch of their own
      const bool on_side = ctx->side != nullptr && s == ctx->side;
      float*& partial = on_side ? ctx->split_partial_side : ctx->split_partial;
      int*& arrivals = on_side ? ctx->split_arrivals_side : ctx->split_arrivals;
      if (partial == nullptr) {
        ORN_CHECK_CUDA(ctx, cudaMalloc((void**)&partial, kSplitPartialBytes));
        ORN_CHECK_CUDA(ctx, cudaMalloc((void**)&arrivals, kSplitTiles * sizeof(int)));
        ORN_CHECK_CUDA(ctx, cudaMemset(arrivals, 0, kSplitTiles * sizeof(int)));
      }
      P.splits = sp; P.partial = partial; P.arrivals = arrivals;
    }
  }
  // A launch of narrow items with more items than SMs runs two CTAs per SM (each with half the
  // shared memory and its own accumulator columns): an item's K loop is a chain of short,
  // latency-bound steps, and two chains per SM overlap.
  const int est_items = P.splits * P.f_tiles * (grp ? std::max(L->E, (rows + P.NT * BN - 1) / (P.NT * BN)) : (rows + P.NT * BN - 1) / (P.NT * BN));
  int ctas = 1, dqw = 8;
  size_t smem = 0;
  // Launches of many narrow items (routed experts with a few rows each): small CTAs of 4 dequantising
  // warps, two-slot rings, up to four per SM: an item's K loop is a latency chain, four chains overlap.
  if (tmem_need(2) <= 128 && est_items > 2 * ctx->sm_count && P.splits == 1) {
    // four CTAs share the SM's 512 tensor-memory columns and its shared memory: up to four IN slots each
    int st = (int)(((226 * 1024) / 4 - 2048) / P.stage_bytes);
    st = std::min(st, 4);
    if (st < 2) st = 2;
    const size_t need = 1024 + (size_t)st * P.stage_bytes;
    const int fit = (int)((226 * 1024) / (need + 1024));  // + static shared memory and the allocation granule
    if (fit >= 3) {
      // the weight ring takes what the accumulators leave of the CTA's 128 columns: hand-offs between the
      // dequantising warps and the MMA thread are a round trip of several hundred cycles per slot
      ctas = std::min(4, fit); dqw = 4; P.w_stages = direct ? 1 : std::min<int>(kMaxW, (128 - (int)P.acc_cols) / (int)kWCols); P.stages = st;
      P.tmem_cols = tmem_need(P.w_stages);
      smem = need;
    }
  }
  if (ctas == 1 && tmem_need(2) <= 256 && est_items > ctx->sm_count) {
    const size_t budget2 = 108 * 1024;
    const int ws = direct ? 1 : std::min<int>(kMaxW, (256 - (int)P.acc_cols) / (int)kWCols);
    const int st = (int)std::min<size_t>(kMaxIn, budget2 / P.stage_bytes);
    if (st >= 3) {
      ctas = 2; P.w_stages = ws; P.stages = st;
      P.tmem_cols = tmem_need(ws);
      smem = 1024 + (size_t)st * P.stage_bytes;
    }
  }
  if (ctas == 1) {
    P.w_stages = direct ? 1 : std::min<int>(kMaxW, (512 - (int)P.acc_cols) / (int)kWCols);
    P.tmem_cols = tmem_need(P.w_stages);
    const size_t budget = 200 * 1024;
    P.stages = (int)std::min<size_t>(kMaxIn, budget / P.stage_bytes);
    if (P.stages < 2) ORN_FAIL(ctx, ORN_ERR_ARG, "gemm: stage does not fit twice into shared memory");
    // one CTA per SM (it may take all of tensor memory): pad the launch's shared memory above half of the SM's
    smem = 1024 + (size_t)P.stages * P.stage_bytes;
    if (smem < 120 * 1024) smem = 120 * 1024;
  }
  GemmMaps maps;
  memset(&maps, 0, sizeof maps);
  auto encode = [&](CUtensorMap* m, CUtensorMapDataType dt, void* base, uint64_t inner, uint64_t outer, uint64_t stride_bytes,
                    uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) -> bool {
    const cuuint64_t gdim[2] = {inner, outer};
    const cuuint64_t gstride[1] = {stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    return enc(m, dt, 2, base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  };
  bool ok = encode(&maps.x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, const_cast<bf16_t*>(x), (uint64_t)L->K, (uint64_t)rows,
                   (uint64_t)L->K * 2, BK, (uint32_t)BN, CU_TENSOR_MAP_SWIZZLE_128B);
  for (int j = 0; j < n; ++j) {
    const orn_linear* Lj = Ls[j];
    WeightMaps& wm = maps.w[j];
    const uint64_t wrows = (uint64_t)Lj->E * Lj->O;
    if (Lj->kind == ORN_BF16) {
      ok = ok && encode(&wm.wsw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, Lj->w, (uint64_t)Lj->K, wrows, (uint64_t)Lj->rec, BK, BM,
                        CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
      ok = ok && encode(&wm.w64, CU_TENSOR_MAP_DATA_TYPE_UINT8, Lj->w, (uint64_t)Lj->rec, wrows, (uint64_t)Lj->rec, 64, BM, CU_TENSOR_MAP_SWIZZLE_NONE);
      ok = ok && encode(&wm.w32, CU_TENSOR_MAP_DATA_TYPE_UINT8, Lj->w, (uint64_t)Lj->rec, wrows, (uint64_t)Lj->rec, 32, BM, CU_TENSOR_MAP_SWIZZLE_NONE);
      ok = ok && encode(&wm.w16, CU_TENSOR_MAP_DATA_TYPE_UINT8, Lj->w, (uint64_t)Lj->rec, wrows, (uint64_t)Lj->rec, 16, BM, CU_TENSOR_MAP_SWIZZLE_NONE);
    }
  }
  if (!ok) ORN_FAIL(ctx, ORN_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed");
  int grid;
  if (grp == nullptr) {
    P.items = nullptr; P.n_items = nullptr;
    const int groups = (rows + P.NT * BN - 1) / (P.NT * BN);
    P.dense_items = P.f_tiles * groups * P.splits;
    grid = std::min(P.dense_items, ctas * ctx->sm_count);
  } else {
    if (L->E > 1024) ORN_FAIL(ctx, ORN_ERR_ARG, "gemm: more than 1024 experts");
    if (scratch == nullptr) ORN_FAIL(ctx, ORN_ERR_ARG, "gemm: the grouped form needs scratch");
    int* n_items = reinterpret_cast<int*>(scratch);
    int4* items = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(scratch) + 256);
    const int max_items = (int)((qgemm_scratch_bytes(rows, L->E, P.f_tiles * BM) - 256) / sizeof(int4));
    int threads = 32;
    while (threads < L->E) threads <<= 1;
    k_plan_items<<<1, threads, 0, s>>>(grp->seg, L->E, P.NT * BN, P.f_tiles, items, n_items, max_items);
    int rc = orn_launch_check(ctx, "k_plan_items");
    if (rc != ORN_OK) return rc;
    P.items = items; P.n_items = n_items; P.dense_items = 0;
    grid = ctas * ctx->sm_count;
  }
  if (dqw == 4) {
    switch (L->kind) {
      case ORN_Q4K: return launch_qgemm<ORN_Q4K, 4>(ctx, s, maps, P, grid, smem);
      case ORN_Q6K: return launch_qgemm<ORN_Q6K, 4>(ctx, s, maps, P, grid, smem);
      case ORN_A8: return launch_qgemm<ORN_A8, 4>(ctx, s, maps, P, grid, smem);
      case ORN_BF16: return launch_qgemm<ORN_BF16, 4>(ctx, s, maps, P, grid, smem);
      case ORN_A4: return launch_qgemm<ORN_A4, 4>(ctx, s, maps, P, grid, smem);
    }
  }
  switch (L->kind) {
    case ORN_Q4K: return launch_qgemm<ORN_Q4K, 8>(ctx, s, maps, P, grid, smem);
    case ORN_Q6K: return launch_qgemm<ORN_Q6K, 8>(ctx, s, maps, P, grid, smem);
    case ORN_A8: return launch_qgemm<ORN_A8, 8>(ctx, s, maps, P, grid, smem);
    case ORN_BF16: return launch_qgemm<ORN_BF16, 8>(ctx, s, maps, P, grid, smem);
    case ORN_A4: return launch_qgemm<ORN_A4, 8>(ctx, s, maps, P, grid, smem);
  }
  ORN_FAIL(ctx, ORN_ERR_ARG, "gemm: unknown weight format");
}

// rows sorted by expert: seg[E+1] and perm[rows] (sorted position -> original row)
int f_route_sort(orn_ctx* ctx, cudaStream_t s, const uint32_t* rhs, int rows, int E, int* seg, int* cursor, uint32_t* perm) {
  if (E > 4096) ORN_FAIL(ctx, ORN_ERR_ARG, "route sort: more than 4096 experts");
  k_route_count<<<1, 1024, E * sizeof(int), s>>>(rhs, rows, E, seg, cursor);
  int rc = orn_launch_check(ctx, "k_route_count");
  if (rc != ORN_OK) return rc;
  if (rows >= 4096) k_route_place_atomic<<<(rows + 255) / 256, 256, 0, s>>>(rhs, rows, E, cursor, perm);
  else k_route_place<<<(E + 7) / 8, 256, 0, s>>>(rhs, rows, E, seg, perm);
  return orn_launch_check(ctx, "k_route_place");
}

int f_gather_rows(orn_ctx* ctx, cudaStream_t s, const bf16_t* x, const uint32_t* lhs, const uint32_t* perm, int rows, int K,
                  bf16_t* xs) {
  if (K % 8) ORN_FAIL(ctx, ORN_ERR_ARG, "gather rows: K must be a multiple of 8");
  k_gather_rows<<<rows, 128, 0, s>>>(x, lhs, perm, rows, K, xs);
  return orn_launch_check(ctx, "k_gather_rows");
}
