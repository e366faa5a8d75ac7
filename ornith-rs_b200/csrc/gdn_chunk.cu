// The gated delta rule over a prompt chunk in chunkwise form, on the warp-level tensor cores.
//
// The recurrence (kernels/gated_delta.metal:36-142; gdn.rs:191-329)
//     S_t = g_t S_{t-1} + beta_t (v_t - g_t S_{t-1} k_t) k_t^T,        o_t = S_t q_t
// is sequential in t, and the row-invariant kernel (gdn.cu) walks it token by token: 0.35 us per
// token, a quarter of a long prompt's time.  Inside a chunk of C = 64 tokens it has a closed form.
// With L_t = sum_{s<=t} log g_s (from the chunk's start) and u_s = beta_s (v_s - g_s S_{s-1} k_s):
//     (I + B A) U = B (V - diag(e^L) K S_0^T),   A[s,r] = e^{L_s - L_r} (k_s . k_r) for r < s,  B = diag(beta)
//     O   = diag(e^L) Q S_0^T + P U,             P[t,s] = e^{L_t - L_s} (q_t . k_s) for s <= t
//     S_C = e^{L_C} S_0 + U^T diag(e^{L_C - L}) K
// (every exponent is <= 0: decays, no overflow).  A, P and T = (I + B A)^{-1} B depend on k, q, g, beta
// only, so a first kernel builds them for all chunks in parallel (the 64 x 64 triangular solve by
// forward substitution); the second kernel carries the state: a warp owns 16 value rows of a head
// (the M = 16 of mma.sync.m16n8k16), state in f32 accumulator fragments, and per chunk computes
// R = V^T - S_0 Kg^T, U^T = R T^T, O^T = S_0 Qg^T + U^T P^T, S_C = e^{L_C} S_0 + U^T Kd with bf16
// operands and f32 accumulation.  Rows of the state are independent, so 8 warps per head (two CTAs)
// run side by side.  Results agree with the sequential kernel to rounding (bf16 operands: about
// 0.25 % rms of the output's rms), which is what the prompt path is granted (src/generate.rs:99).
#include "mma_bf16.cuh"
#include "orn_internal.h"

namespace {

constexpr int kC = 64;                    // tokens per chunk
constexpr int kPitchK = 272;              // bytes per row of a [64][128] bf16 tile in shared memory (256 + 16)
constexpr int kPitchC = 144;              // bytes per row of a [64][64] bf16 tile (128 + 16)
constexpr int kChunkElems = 3 * kC * 128 + 2 * kC * kC;  // Kg, Qg, Kd, T, P of one (head, chunk), bf16

struct PrepParams {
  const bf16_t* q;     // [T][Hk][128]
  const bf16_t* k;     // [T][Hk][128]
  const float* g;      // [T][Hv]
  const bf16_t* beta;  // [T][Hv]
  int T, Hk, Hv, nchunks;
  bf16_t* scratch;     // [Hv][nchunks][kChunkElems]
  float* gc;           // [Hv][nchunks] e^{L_C}
};

// grid (nchunks, Hv), 256 threads.  K K^T and Q K^T of the chunk on mma.sync (the inputs are bf16 already),
// decays and the triangular solve in f32.
constexpr int kPrepTile = kC * kPitchK;  // a [64][128] bf16 tile in shared memory
constexpr int kPrepSmem = 2 * kPrepTile + (2 * kC * 65 + 2 * kC) * (int)sizeof(float);
__global__ void __launch_bounds__(256) gdn_chunk_prep_kernel(PrepParams p) {
  extern __shared__ __align__(128) uint8_t psm[];
  uint8_t* Kb = psm;                                                    // [64][pitch 272] bf16
  uint8_t* Qb = psm + kPrepTile;
  float* BA = reinterpret_cast<float*>(psm + 2 * kPrepTile);            // [64][65]  beta_s A[s][r] (strictly lower)
  float* Tm = BA + kC * 65;                                             // [64][65]
  float* L = Tm + kC * 65;                                              // [64]
  float* bt = L + kC;                                                   // [64]
  const int c = blockIdx.x, hv = blockIdx.y, hk = hv / (p.Hv / p.Hk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, qd = lane & 3;
  const int t0 = c * kC;
  for (int i = threadIdx.x; i < kC * 16; i += blockDim.x) {  // 16-byte pieces of the chunk's k and q rows (zeros beyond T)
    const int s = i >> 4, pc = i & 15, t = t0 + s;
    uint4 kv = make_uint4(0, 0, 0, 0), qv = kv;
    if (t < p.T) {
      kv = ldg128(p.k + ((size_t)t * p.Hk + hk) * 128 + 8 * pc);
      qv = ldg128(p.q + ((size_t)t * p.Hk + hk) * 128 + 8 * pc);
    }
    *reinterpret_cast<uint4*>(Kb + s * kPitchK + 16 * pc) = kv;
    *reinterpret_cast<uint4*>(Qb + s * kPitchK + 16 * pc) = qv;
  }
  if (threadIdx.x < kC) {
    const int t = t0 + threadIdx.x;
    L[threadIdx.x] = t < p.T ? logf(fmaxf(p.g[(size_t)t * p.Hv + hv], 1e-38f)) : 0.f;  // padding: no decay, no update
    bt[threadIdx.x] = t < p.T ? bf2f(p.beta[(size_t)t * p.Hv + hv]) : 0.f;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float acc = 0.f;
    for (int s = 0; s < kC; ++s) { acc += L[s]; L[s] = acc; }
  }
  __syncthreads();
  bf16_t* out = p.scratch + ((size_t)hv * p.nchunks + c) * kChunkElems;
  bf16_t* Kg = out, *Qg = out + kC * 128, *Kd = out + 2 * kC * 128, *To = out + 3 * kC * 128, *Po = To + kC * kC;
  {
    // warp = (row tile mt of 16 tokens s, column half nh of 32 tokens r): 4 n-tiles, two products
    const int mt = warp & 3, nh = warp >> 2;
    const uint32_t kb_s = smem_u32(Kb), qb_s = smem_u32(Qb);
    const uint32_t a_off = (16 * mt + (lane & 7) + 8 * ((lane >> 3) & 1)) * kPitchK + 16 * (lane >> 4);
    const uint32_t b_off = (32 * nh + (lane & 7) + 8 * (lane >> 4)) * kPitchK + 16 * ((lane >> 3) & 1);
    float kk[4][4], qk[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) kk[nt][e] = qk[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t ak[4], aq[4], b0[4], b1[4];
      ldsm4(kb_s + a_off + 32 * ks, ak);
      ldsm4(qb_s + a_off + 32 * ks, aq);
      ldsm4(kb_s + b_off + 32 * ks, b0);                  // tokens r 32nh .. +15
      ldsm4(kb_s + b_off + 16 * kPitchK + 32 * ks, b1);   // tokens r 32nh+16 .. +31
      mma16816(kk[0], ak, b0[0], b0[1]); mma16816(kk[1], ak, b0[2], b0[3]);
      mma16816(kk[2], ak, b1[0], b1[1]); mma16816(kk[3], ak, b1[2], b1[3]);
      mma16816(qk[0], aq, b0[0], b0[1]); mma16816(qk[1], aq, b0[2], b0[3]);
      mma16816(qk[2], aq, b1[0], b1[1]); mma16816(qk[3], aq, b1[2], b1[3]);
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int s = 16 * mt + g + 8 * (e >> 1), r = 32 * nh + 8 * nt + 2 * qd + (e & 1);
        const float dec = r <= s ? expf(L[s] - L[r]) : 0.f;
        BA[s * 65 + r] = r < s ? bt[s] * dec * kk[nt][e] : 0.f;
        Po[s * kC + r] = f2bf(dec * qk[nt][e]);
      }
  }
  for (int i = threadIdx.x; i < kC * 128; i += blockDim.x) {
    const int s = i >> 7, d = i & 127;
    const float kv = bf2f(*reinterpret_cast<const bf16_t*>(Kb + s * kPitchK + 2 * d));
    const float qv = bf2f(*reinterpret_cast<const bf16_t*>(Qb + s * kPitchK + 2 * d));
    const float e = expf(L[s]);
    Kg[i] = f2bf(e * kv);
    Qg[i] = f2bf(e * qv);
    Kd[i] = f2bf(expf(L[kC - 1] - L[s]) * kv);
  }
  if (threadIdx.x == 0) p.gc[(size_t)hv * p.nchunks + c] = expf(L[kC - 1]);
  __syncthreads();
  // T = (I + B A)^{-1} B by forward substitution.  Column `col` of T depends on column `col` only:
  // four adjacent lanes share a column and split the sum over the earlier rows between them.
  {
    const int col = threadIdx.x >> 2, sub = threadIdx.x & 3;
    for (int s = 0; s < kC; ++s) {
      float acc = 0.f;
      for (int r = col + sub; r < s; r += 4) acc = fmaf(-BA[s * 65 + r], Tm[r * 65 + col], acc);  // T[r][col] = 0 for r < col
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (sub == 0) Tm[s * 65 + col] = s >= col ? acc + (s == col ? bt[s] : 0.f) : 0.f;
      __syncwarp();
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kC * kC; i += blockDim.x) To[i] = f2bf(Tm[(i >> 6) * 65 + (i & 63)]);
}

struct ScanParams {
  const bf16_t* v;        // [T][Hv][128]
  const bf16_t* scratch;  // [Hv][nchunks][kChunkElems]
  const float* gc;        // [Hv][nchunks]
  const float* state_in;  // [Hv][128][128] (null: ring)
  float* state_out;
  float* ring;            // [nring][Hv][128][128]
  const int* cur;
  int nring;
  bf16_t* y;              // [T][Hv][128]
  int T, Hv, nchunks;
};

constexpr int kScanWarps = 4;
constexpr int kStageBytes = 3 * kC * kPitchK + 3 * kC * kPitchC;  // Kg, Qg, Kd, T, P, V(64 value rows of this CTA)
constexpr int kScanSmem = 2 * kStageBytes;

ORN_D uint32_t neg2(uint32_t x) { return x ^ 0x80008000u; }

// grid (2, Hv): CTA = 64 value rows of one head, 4 warps x 16 rows
__global__ void __launch_bounds__(kScanWarps * 32) gdn_chunk_scan_kernel(ScanParams p) {
  extern __shared__ __align__(128) uint8_t ssm[];
  const int hv = blockIdx.y, row0 = blockIdx.x * 64;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, qd = lane & 3;
  const size_t ssz = (size_t)p.Hv * 128 * 128;
  const float* sin = p.state_in;
  float* sout = p.state_out;
  if (p.ring != nullptr) {
    const int cur = *p.cur;
    sin = p.ring + (size_t)(cur % p.nring) * ssz;
    sout = p.ring + (size_t)((cur + 1) % p.nring) * ssz;
  }
  const size_t srow = ((size_t)hv * 128 + row0 + 16 * warp) * 128;  // this warp's 16 state rows
  // state in accumulator layout: n-tile nt = key dims 8nt .. 8nt+7; [0],[1] row g, [2],[3] row g + 8
  float S[16][4];
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    const float2 a = *reinterpret_cast<const float2*>(sin + srow + (size_t)g * 128 + 8 * nt + 2 * qd);
    const float2 b = *reinterpret_cast<const float2*>(sin + srow + (size_t)(g + 8) * 128 + 8 * nt + 2 * qd);
    S[nt][0] = a.x; S[nt][1] = a.y; S[nt][2] = b.x; S[nt][3] = b.y;
  }
  const uint32_t sm0 = smem_u32(ssm);
  auto issue = [&](int c) {
    const uint32_t dst = sm0 + (c & 1) * kStageBytes;
    const bf16_t* src = p.scratch + ((size_t)hv * p.nchunks + c) * kChunkElems;
    // Kg, Qg, Kd: 3 x 64 rows x 16 pieces of 16 bytes
    for (int i = threadIdx.x; i < 3 * kC * 16; i += blockDim.x) {
      const int tile = i / (kC * 16), rem = i - tile * kC * 16, r = rem >> 4, pc = rem & 15;
      cp_async16(dst + tile * kC * kPitchK + r * kPitchK + 16 * pc, src + (size_t)tile * kC * 128 + r * 128 + 8 * pc, 16);
    }
    // T, P: 2 x 64 rows x 8 pieces
    for (int i = threadIdx.x; i < 2 * kC * 8; i += blockDim.x) {
      const int tile = i / (kC * 8), rem = i - tile * kC * 8, r = rem >> 3, pc = rem & 7;
      cp_async16(dst + 3 * kC * kPitchK + tile * kC * kPitchC + r * kPitchC + 16 * pc,
                 src + 3 * kC * 128 + (size_t)tile * kC * kC + r * kC + 8 * pc, 16);
    }
    // V: 64 tokens x this CTA's 64 value rows (zeros beyond T)
    for (int i = threadIdx.x; i < kC * 8; i += blockDim.x) {
      const int r = i >> 3, pc = i & 7, t = c * kC + r;
      cp_async16(dst + 3 * kC * kPitchK + 2 * kC * kPitchC + r * kPitchC + 16 * pc,
                 p.v + ((size_t)min(t, p.T - 1) * p.Hv + hv) * 128 + row0 + 8 * pc, t < p.T ? 16 : 0);
    }
    cp_async_commit();
  };
  // ldmatrix lane offsets: B operand from a row-major [n][k] tile (k contiguous), and transposed from [k][n]
  const uint32_t b_row = (lane & 7) + 8 * (lane >> 4), b_k = 8 * ((lane >> 3) & 1);
  const uint32_t t_row = (lane & 7) + 8 * ((lane >> 3) & 1), t_n = 8 * (lane >> 4);
  issue(0);
  for (int c = 0; c < p.nchunks; ++c) {
    if (c + 1 < p.nchunks) {
      issue(c + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t st = sm0 + (c & 1) * kStageBytes;
    const uint32_t kg = st, qg = st + kC * kPitchK, kd = st + 2 * kC * kPitchK;
    const uint32_t tm = st + 3 * kC * kPitchK, pm = tm + kC * kPitchC, vs = pm + kC * kPitchC;
    uint8_t* vptr = ssm + (c & 1) * kStageBytes + 3 * kC * kPitchK + 2 * kC * kPitchC;
    // (1) R = V^T - S_0 Kg^T   [16 rows x 64 tokens]; n-tile = 8 tokens
    float R[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int t = 8 * nt + 2 * qd, col = 16 * warp + g;
      R[nt][0] = bf2f(*reinterpret_cast<const bf16_t*>(vptr + t * kPitchC + 2 * col));
      R[nt][1] = bf2f(*reinterpret_cast<const bf16_t*>(vptr + (t + 1) * kPitchC + 2 * col));
      R[nt][2] = bf2f(*reinterpret_cast<const bf16_t*>(vptr + t * kPitchC + 2 * (col + 8)));
      R[nt][3] = bf2f(*reinterpret_cast<const bf16_t*>(vptr + (t + 1) * kPitchC + 2 * (col + 8)));
    }
    float O[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) O[nt][0] = O[nt][1] = O[nt][2] = O[nt][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      // the state's key dims 16kk .. 16kk+15 as a bf16 A fragment, and its negative
      const uint32_t sa[4] = {pack_bf16x2(S[2 * kk][0], S[2 * kk][1]), pack_bf16x2(S[2 * kk][2], S[2 * kk][3]),
                              pack_bf16x2(S[2 * kk + 1][0], S[2 * kk + 1][1]), pack_bf16x2(S[2 * kk + 1][2], S[2 * kk + 1][3])};
      const uint32_t an[4] = {neg2(sa[0]), neg2(sa[1]), neg2(sa[2]), neg2(sa[3])};
#pragma unroll
      for (int np = 0; np < 4; ++np) {  // pairs of token n-tiles
        uint32_t bk[4], bq[4];
        ldsm4(kg + (16 * np + b_row) * kPitchK + 2 * (16 * kk + b_k), bk);
        ldsm4(qg + (16 * np + b_row) * kPitchK + 2 * (16 * kk + b_k), bq);
        mma16816(R[2 * np], an, bk[0], bk[1]);
        mma16816(R[2 * np + 1], an, bk[2], bk[3]);
        mma16816(O[2 * np], sa, bq[0], bq[1]);      // (3a) S_0 Qg^T
        mma16816(O[2 * np + 1], sa, bq[2], bq[3]);
      }
    }
    // (2) U^T = R T^T: k-steps over tokens s', B rows = s (n), k = s'
    uint32_t Ra[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      Ra[ks][0] = pack_bf16x2(R[2 * ks][0], R[2 * ks][1]);
      Ra[ks][1] = pack_bf16x2(R[2 * ks][2], R[2 * ks][3]);
      Ra[ks][2] = pack_bf16x2(R[2 * ks + 1][0], R[2 * ks + 1][1]);
      Ra[ks][3] = pack_bf16x2(R[2 * ks + 1][2], R[2 * ks + 1][3]);
    }
    float U[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) U[nt][0] = U[nt][1] = U[nt][2] = U[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        if (np < ks) continue;  // T is lower triangular: T[s][s'] = 0 for s' > s
        uint32_t bt4[4];
        ldsm4(tm + (16 * np + b_row) * kPitchC + 2 * (16 * ks + b_k), bt4);
        mma16816(U[2 * np], Ra[ks], bt4[0], bt4[1]);
        mma16816(U[2 * np + 1], Ra[ks], bt4[2], bt4[3]);
      }
    uint32_t Ua[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      Ua[ks][0] = pack_bf16x2(U[2 * ks][0], U[2 * ks][1]);
      Ua[ks][1] = pack_bf16x2(U[2 * ks][2], U[2 * ks][3]);
      Ua[ks][2] = pack_bf16x2(U[2 * ks + 1][0], U[2 * ks + 1][1]);
      Ua[ks][3] = pack_bf16x2(U[2 * ks + 1][2], U[2 * ks + 1][3]);
    }
    // (3b) O^T += U^T P^T: B rows = t (n), k = s; P[t][s] = 0 for s > t
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        if (np < ks) continue;
        uint32_t bp[4];
        ldsm4(pm + (16 * np + b_row) * kPitchC + 2 * (16 * ks + b_k), bp);
        mma16816(O[2 * np], Ua[ks], bp[0], bp[1]);
        mma16816(O[2 * np + 1], Ua[ks], bp[2], bp[3]);
      }
    // (4) S_C = e^{L_C} S_0 + U^T Kd: k-steps over tokens, B from the [token][dim] tile transposed
    const float gcv = p.gc[(size_t)hv * p.nchunks + c];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) { S[nt][0] *= gcv; S[nt][1] *= gcv; S[nt][2] *= gcv; S[nt][3] *= gcv; }
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t bd[4];
        ldsm4t(kd + (16 * ks + t_row) * kPitchK + 2 * (16 * j + t_n), bd);
        mma16816(S[2 * j], Ua[ks], bd[0], bd[1]);
        mma16816(S[2 * j + 1], Ua[ks], bd[2], bd[3]);
      }
    // outputs: this warp's 16 rows x 64 tokens into the V tile's place (each warp reads and writes
    // only its own 16 columns), then the CTA stores whole token rows
    __syncwarp();
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int t = 8 * nt + 2 * qd, col = 16 * warp + g;
      *reinterpret_cast<bf16_t*>(vptr + t * kPitchC + 2 * col) = f2bf(O[nt][0]);
      *reinterpret_cast<bf16_t*>(vptr + (t + 1) * kPitchC + 2 * col) = f2bf(O[nt][1]);
      *reinterpret_cast<bf16_t*>(vptr + t * kPitchC + 2 * (col + 8)) = f2bf(O[nt][2]);
      *reinterpret_cast<bf16_t*>(vptr + (t + 1) * kPitchC + 2 * (col + 8)) = f2bf(O[nt][3]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kC * 8; i += blockDim.x) {
      const int r = i >> 3, pc = i & 7, t = c * kC + r;
      if (t < p.T)
        *reinterpret_cast<uint4*>(p.y + ((size_t)t * p.Hv + hv) * 128 + row0 + 8 * pc) = *reinterpret_cast<const uint4*>(vptr + r * kPitchC + 16 * pc);
    }
    __syncthreads();  // the stage is refilled by the next iteration's issue
  }
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    *reinterpret_cast<float2*>(sout + srow + (size_t)g * 128 + 8 * nt + 2 * qd) = make_float2(S[nt][0], S[nt][1]);
    *reinterpret_cast<float2*>(sout + srow + (size_t)(g + 8) * 128 + 8 * nt + 2 * qd) = make_float2(S[nt][2], S[nt][3]);
  }
}

}  // namespace

size_t gdn_chunk_scratch_bytes(int T, int Hv) {
  const size_t nchunks = (size_t)(T + kC - 1) / kC;
  return (size_t)Hv * nchunks * kChunkElems * sizeof(bf16_t) + (size_t)Hv * nchunks * sizeof(float) + 256;
}

// y[T, Hv, 128] and the state after the last token from q, k [T, Hk, 128], v [T, Hv, 128], g, beta [T, Hv].
// The state comes from `state` (and goes back there) or, in ring mode, from ring slot *cur % nring and goes
// to slot (*cur + 1) % nring.  scratch: gdn_chunk_scratch_bytes(T, Hv) of device memory.
int k_gated_delta_chunked(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* k, const bf16_t* v, const float* g,
                          const bf16_t* beta, float* state, float* ring, int nring, const int* cur, int T, int Hk, int Hv,
                          bf16_t* y, void* scratch) {
  if (T < 1) return ORN_OK;
  if (Hv % Hk != 0) ORN_FAIL(ctx, ORN_ERR_ARG, "gated_delta: Hv % Hk != 0");
  if ((state == nullptr) == (ring == nullptr)) ORN_FAIL(ctx, ORN_ERR_ARG, "gated_delta_chunked: one of state, ring");
  const int nchunks = (T + kC - 1) / kC;
  PrepParams pp;
  pp.q = q; pp.k = k; pp.g = g; pp.beta = beta; pp.T = T; pp.Hk = Hk; pp.Hv = Hv; pp.nchunks = nchunks;
  pp.scratch = reinterpret_cast<bf16_t*>(scratch);
  pp.gc = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + (((size_t)Hv * nchunks * kChunkElems * sizeof(bf16_t) + 255) & ~(size_t)255));
  const size_t psmem = kPrepSmem;
  int rc = orn_grant_smem(ctx, reinterpret_cast<const void*>(gdn_chunk_prep_kernel), psmem);
  if (rc != ORN_OK) return rc;
  gdn_chunk_prep_kernel<<<dim3(nchunks, Hv), 256, psmem, s>>>(pp);
  rc = orn_launch_check(ctx, "gdn_chunk_prep");
  if (rc != ORN_OK) return rc;
  ScanParams sp;
  sp.v = v; sp.scratch = pp.scratch; sp.gc = pp.gc; sp.state_in = state; sp.state_out = state; sp.ring = ring; sp.cur = cur;
  sp.nring = nring; sp.y = y; sp.T = T; sp.Hv = Hv; sp.nchunks = nchunks;
  rc = orn_grant_smem(ctx, reinterpret_cast<const void*>(gdn_chunk_scan_kernel), kScanSmem);
  if (rc != ORN_OK) return rc;
  gdn_chunk_scan_kernel<<<dim3(2, Hv), kScanWarps * 32, kScanSmem, s>>>(sp);
  return orn_launch_check(ctx, "gdn_chunk_scan");
}
