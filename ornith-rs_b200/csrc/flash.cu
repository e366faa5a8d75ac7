// Causal attention of a prompt chunk over the KV cache on the warp-level tensor cores.
//
// The reference runs the prompt through one scaled_dot_product_attention call per layer and chunk
// (src/model/qwen3_5.rs:430-470, mask "causal"); the row-invariant kernel (attn.cu) walks the cache
// once per (query head, row), which at 6621 tokens is most of the prompt's time.  This kernel is the
// prompt path's own: a CTA takes 64 consecutive rows of one query head (4 warps x 16 rows, the A
// operand of mma.sync.m16n8k16), streams the keys of its KV head in tiles of 32 through a two-stage
// cp.async pipeline (rows padded to 528 bytes for conflict-free ldmatrix), and keeps an online
// softmax in the base-2 domain on the accumulator fragments: S = Q K^T (bf16 in, f32 out), P = 2^(S -
// max) rounded to bf16, O += P V with V fragments through ldmatrix.trans.  Row t of the chunk sees
// keys 0 .. pos + t.  Results agree with the row-invariant kernel to rounding (another summation
// order, bf16 probabilities), which is what the reference grants this path (src/generate.rs:99).
#include "mma_bf16.cuh"
#include "orn_internal.h"

namespace {

constexpr int kFaWarps = 4;
constexpr int kFaRows = 16 * kFaWarps;  // query rows per CTA
constexpr int kFaKeys = 32;             // keys per pipeline stage
constexpr int kFaRowB = 528;            // bytes per staged row: 256 bf16 + 16 B pad
constexpr int kFaQBytes = kFaRows * kFaRowB;
constexpr int kFaStage = 2 * kFaKeys * kFaRowB;  // K tile then V tile
constexpr int kFaSmem = kFaQBytes + 2 * kFaStage;

__global__ void __launch_bounds__(kFaWarps * 32, 2) flash_prefill_kernel(const bf16_t* __restrict__ q /*[T, Hq, 256]*/,
                                                                          const bf16_t* __restrict__ kc, const bf16_t* __restrict__ vc,
                                                                          const int* __restrict__ pos, int T, int Hq, int Hkv, int cap,
                                                                          float scale, bf16_t* __restrict__ out /*[T, Hq*256]*/) {
  constexpr int HD = 256;
  extern __shared__ __align__(128) uint8_t fsm[];
  const int qt = gridDim.x - 1 - blockIdx.x;  // the tiles with the most keys start first
  const int h = blockIdx.y, kvh = h / (Hq / Hkv);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, qd = lane & 3;
  const int p0 = *pos;
  const int r0 = qt * kFaRows;
  const int L = min(cap, p0 + T);                        // valid keys of the cache
  const int nkeys = min(L, p0 + min(r0 + kFaRows, T));   // keys any row of this tile sees
  const int tiles = (nkeys + kFaKeys - 1) / kFaKeys;
  const uint32_t q_s = smem_u32(fsm), st_s = q_s + kFaQBytes;
  const size_t base = ((size_t)kvh * cap) * HD;
  // the 64 query rows (zeros beyond T), in the same cp.async group as the first key tile
  for (int i = threadIdx.x; i < kFaRows * 32; i += blockDim.x) {
    const int r = i >> 5, piece = i & 31;
    const int row = r0 + r;
    cp_async16(q_s + r * kFaRowB + 16 * piece, q + ((size_t)min(row, T - 1) * Hq + h) * HD + 8 * piece, row < T ? 16 : 0);
  }
  auto issue = [&](int i) {
    const uint32_t dst = st_s + (i & 1) * kFaStage;
    for (int it = threadIdx.x; it < kFaKeys * 32; it += blockDim.x) {
      const int r = it >> 5, piece = it & 31;
      const int n = i * kFaKeys + r;
      const int ok = n < L ? 16 : 0;
      const size_t src = base + (size_t)min(n, cap - 1) * HD + 8 * piece;
      cp_async16(dst + r * kFaRowB + 16 * piece, kc + src, ok);
      cp_async16(dst + kFaKeys * kFaRowB + r * kFaRowB + 16 * piece, vc + src, ok);
    }
    cp_async_commit();
  };
  issue(0);
  float o[32][4];
#pragma unroll
  for (int nt = 0; nt < 32; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const float sc2 = scale * 1.4426950408889634f;
  const int wrow = r0 + 16 * warp;                       // this warp's first row
  const int lim0 = p0 + wrow + g + 1, lim1 = lim0 + 8;   // keys below these are visible to rows g, g + 8
  const int wlast = p0 + wrow + 15;                      // the last key any row of this warp sees
  const uint32_t a_off = (16 * warp + (lane & 7) + 8 * ((lane >> 3) & 1)) * kFaRowB + 16 * (lane >> 4);
  const uint32_t k_off = ((lane & 7) + 8 * (lane >> 4)) * kFaRowB + 16 * ((lane >> 3) & 1);
  const uint32_t v_off = ((lane & 7) + 8 * ((lane >> 3) & 1)) * kFaRowB + 16 * (lane >> 4);
  for (int i = 0; i < tiles; ++i) {
    if (i + 1 < tiles) {
      issue(i + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t kt = st_s + (i & 1) * kFaStage, vt = kt + kFaKeys * kFaRowB;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int n0 = i * kFaKeys + 16 * half;
      if (n0 > wlast) continue;  // warp-uniform: every key of this step is in the future of every row
      const uint32_t ks = kt + half * 16 * kFaRowB, vs = vt + half * 16 * kFaRowB;
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        uint32_t a[4], bk[4];
        ldsm4(q_s + a_off + 32 * kk, a);
        ldsm4(ks + k_off + 32 * kk, bk);
        mma16816(s[0], a, bk[0], bk[1]);
        mma16816(s[1], a, bk[2], bk[3]);
      }
      const bool all_visible = n0 + 16 <= p0 + wrow + 1;  // warp-uniform: the first row already sees the step's last key
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int key = n0 + 8 * nt + 2 * qd + (c & 1);
          const float v = s[nt][c] * sc2;
          s[nt][c] = (all_visible || key < (c < 2 ? lim0 : lim1)) ? v : -INFINITY;
        }
      float x0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
      float x1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
      x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 1)); x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 2));
      x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 1)); x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 2));
      const float n0m = fmaxf(m0, x0), n1m = fmaxf(m1, x1);
      const float u0 = n0m == -INFINITY ? 0.f : n0m, u1 = n1m == -INFINITY ? 0.f : n1m;
      const float c0 = exp2f(m0 - u0), c1 = exp2f(m1 - u1);
      m0 = n0m; m1 = n1m;
      float pr[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        pr[nt][0] = exp2f(s[nt][0] - u0); pr[nt][1] = exp2f(s[nt][1] - u0);
        pr[nt][2] = exp2f(s[nt][2] - u1); pr[nt][3] = exp2f(s[nt][3] - u1);
      }
      l0 = l0 * c0 + (pr[0][0] + pr[0][1] + pr[1][0] + pr[1][1]);
      l1 = l1 * c1 + (pr[0][2] + pr[0][3] + pr[1][2] + pr[1][3]);
      if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {
#pragma unroll
        for (int nt = 0; nt < 32; ++nt) { o[nt][0] *= c0; o[nt][1] *= c0; o[nt][2] *= c1; o[nt][3] *= c1; }
      }
      uint32_t pa[4] = {pack_bf16x2(pr[0][0], pr[0][1]), pack_bf16x2(pr[0][2], pr[0][3]), pack_bf16x2(pr[1][0], pr[1][1]),
                        pack_bf16x2(pr[1][2], pr[1][3])};
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        uint32_t bv[4];
        ldsm4t(vs + v_off + 32 * j, bv);
        mma16816(o[2 * j], pa, bv[0], bv[1]);
        mma16816(o[2 * j + 1], pa, bv[2], bv[3]);
      }
    }
    __syncthreads();  // the stage is refilled by the next iteration's issue
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const int ra = wrow + g, rb = ra + 8;
  const float i0 = 1.0f / l0, i1 = 1.0f / l1;
#pragma unroll
  for (int nt = 0; nt < 32; ++nt) {
    const int d = 8 * nt + 2 * qd;
    if (ra < T) *reinterpret_cast<uint32_t*>(out + ((size_t)ra * Hq + h) * HD + d) = pack_bf16x2(o[nt][0] * i0, o[nt][1] * i0);
    if (rb < T) *reinterpret_cast<uint32_t*>(out + ((size_t)rb * Hq + h) * HD + d) = pack_bf16x2(o[nt][2] * i1, o[nt][3] * i1);
  }
}

}  // namespace

// att[T, Hq*256] = causal attention of the chunk's T rows (row t at position *pos + t) over cache rows
// 0 .. *pos + T - 1, which the caller has appended already.  head_dim 256 only.
int k_flash_prefill(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* kc, const bf16_t* vc, int T, int Hq, int Hkv, int hd,
                    int cap, const int* pos, float scale, bf16_t* out) {
  if (hd != 256 || Hq % Hkv) ORN_FAIL(ctx, ORN_ERR_ARG, "flash_prefill: head_dim 256 and whole query groups only");
  int rc = orn_grant_smem(ctx, reinterpret_cast<const void*>(flash_prefill_kernel), kFaSmem);
  if (rc != ORN_OK) return rc;
  dim3 grid((T + kFaRows - 1) / kFaRows, Hq);
  flash_prefill_kernel<<<grid, kFaWarps * 32, kFaSmem, s>>>(q, kc, vc, pos, T, Hq, Hkv, cap, scale, out);
  return orn_launch_check(ctx, "flash_prefill");
}
