// Batched decode: B concurrent sequences, each stepping a verify window of T rows (T = 2 for MTP
// depth 1) through the whole trunk in one pass over the weights, the routed experts through the
// expert-parallel block.
//
// The reference decodes one sequence (README.md:217-221); this is the same layer sequence
// (TextModel::forward_capture, src/model/qwen3_5.rs:578-695, and TrunkCapture::rewind, :301-349)
// over rows laid out sequence-major, [B][T].  What is per sequence stays per sequence: a KV cache
// [Hkv, cap, 256] per attention layer, a conv window and a ring of T + 1 recurrent states per
// gated-delta layer, a position and a ring cursor.  What is per row is batched: every projection is
// one wide product over the B * T rows (tensor cores from 16 rows; the row-invariant mat-vec below
// that or with ORN_WIDE_EXACT=1), the MoE block is orn_ep_moe_block over all rows (experts split
// over the ranks of the node when the group has more than one), lm_head is one product and the
// greedy targets of all rows come back together.  Acceptance is per sequence: commit(keep[b]) moves
// position and ring cursor by keep[b] and shifts the conv window; nothing is copied for a rollback.
//
// With row-invariant products the batched pass reproduces the single-sequence engine bit for bit
// (same kernels, a sequence index in their grids); that is how it is tested.  With the tensor-core
// products it agrees to rounding, like the prompt path.
//
// Attention over long contexts: the row-invariant kernel walks a sequence's cache once per (query
// head, row); the batched fast path walks it once per (KV head, 256-key chunk) for the G * T
// queries that share it and merges the chunks in a second kernel (split-KV; 5.4 GB of cache per
// step at 64 sequences x 4096 tokens is the largest HBM stream of the step after the experts).
#include <algorithm>
#include <cstring>
#include <type_traits>

#include "fused.h"
#include "model_types.h"
#include "mma_bf16.cuh"
#include "orn_internal.h"

#define CK(call)                     \
  do {                               \
    int rc__ = (call);               \
    if (rc__ != ORN_OK) return rc__; \
  } while (0)


namespace {

constexpr int kMinChunk = 128, kMaxChunk = 512;  // keys per CTA of the split-KV attention
constexpr int kPartStride = 264;  // floats per (query, chunk) partial: m, s, pad, o[256]

ORN_D float bflo(uint32_t v) { return __uint_as_float(v << 16); }
ORN_D float bfhi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
ORN_D void widen(const uint4& v, float* f) {
  f[0] = bflo(v.x); f[1] = bfhi(v.x); f[2] = bflo(v.y); f[3] = bfhi(v.y);
  f[4] = bflo(v.z); f[5] = bfhi(v.z); f[6] = bflo(v.w); f[7] = bfhi(v.w);
}

// rows of n elements: dst[map[r]] = src[r]
__global__ void scatter_rows_kernel(const bf16_t* src, const uint32_t* map, int n, bf16_t* dst) {
  const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)blockIdx.x * n);
  uint4* d = reinterpret_cast<uint4*>(dst + (size_t)map[blockIdx.x] * n);
  for (int i = threadIdx.x; i < n / 8; i += blockDim.x) d[i] = s[i];
}
__global__ void conv_map_kernel(uint32_t* map, int B, int T, int rows_per_seq, int S) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < B * T) map[r] = (uint32_t)((r / T) * rows_per_seq + S + r % T);
}
// accept keep[b] rows of sequence b's window: position and ring cursor move, the conv windows of
// every gated-delta layer shift so that their first S rows are the last S rows kept
__global__ void commit_kernel(int* pos, int* cur, const int* keep, int B) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) { pos[b] += keep[b]; cur[b] += keep[b]; }
}
__global__ void conv_shift_batched_kernel(bf16_t* const* bufs, const int* keep, int S, int D, int rows_per_seq) {
  bf16_t* buf = bufs[blockIdx.y] + (size_t)blockIdx.z * rows_per_seq * D;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;  // over D/8 16-byte pieces
  if (c >= D / 8) return;
  const int k = keep[blockIdx.z];
  uint4* p = reinterpret_cast<uint4*>(buf);
  for (int j = 0; j < S; ++j) p[(size_t)j * (D / 8) + c] = p[(size_t)(j + k) * (D / 8) + c];
}
__global__ void fill_f32_kernel(float* p, size_t n, uint64_t seed, float std) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint64_t x = seed + i * 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  x ^= x >> 31;
  const float u = ((float)(x >> 40) + 0.5f) * (1.0f / 16777216.0f) - 0.5f;  // uniform (-0.5, 0.5)
  p[i] = std * 3.4641016f * u;
}
__global__ void set_ints_kernel(int* p, int n, int v) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

// ---- split-KV attention over the caches of B sequences (fast path) ------------------------------
// grid (chunks, Hkv, B), 4 warps.  The G * Tb <= 16 queries that share a KV head (query j is head
// kvh * G + j / Tb, window row j % Tb) form the 16-row A operand of mma.sync.m16n8k16 (bf16 in, f32
// out); a CTA owns `chunk` consecutive keys of one (sequence, KV head), its warps take 16-key tiles
// round robin.  Per warp a private 3-stage cp.async pipeline brings a tile's K and V rows (16 x 512 B
// each, rows padded to 528 B so that ldmatrix reads without bank conflicts) into shared memory;
// rows at or beyond the sequence's length arrive as zeros.  Per tile: S = Q K^T (32 MMAs), online
// softmax in the base-2 domain on the accumulator fragments, P (bf16) V (32 MMAs, V fragments through
// ldmatrix.trans).  The warps' partials merge through shared memory and the CTA writes one
// (max, sum, out[256]) per query; battn_merge_kernel folds the chunks.
constexpr int kAttWarps = 4;
constexpr int kAttRowB = 528;                        // bytes per staged row: 256 bf16 + 16 B pad
constexpr int kAttTile = 16 * kAttRowB;              // one 16-key tile of K or of V
constexpr int kAttStages = 3;
constexpr int kAttWarpBytes = kAttStages * 2 * kAttTile;                   // 50688
constexpr int kAttSmem = 16 * kAttRowB + kAttWarps * kAttWarpBytes;        // Q + the warps' pipelines
static_assert(kAttWarpBytes >= 16 * 256 * 4 + 2 * 16 * 4, "a warp's partial must fit its pipeline memory");

__global__ void __launch_bounds__(kAttWarps * 32) battn_partial_kernel(const bf16_t* __restrict__ q /*[B*Tb, Hq, 256]*/,
                                                                       const bf16_t* __restrict__ kc, const bf16_t* __restrict__ vc,
                                                                       const int* __restrict__ pos, int Tb, int Hq, int Hkv, int cap,
                                                                       float scale, float* __restrict__ part, int nchunks, int chunk,
                                                                       int NQ) {
  constexpr int HD = 256;
  extern __shared__ __align__(128) uint8_t asm_[];
  const int ci = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, qd = lane & 3;
  const int G = Hq / Hkv;
  const int p0 = pos[b];
  const int Lmax = min(cap, p0 + Tb);  // keys any row of the window may see
  float* out = part + (((size_t)b * Hkv + kvh) * nchunks + ci) * NQ * kPartStride;
  const int k0 = ci * chunk;
  if (k0 >= Lmax) {  // nothing here for this sequence: an empty partial
    for (int j = threadIdx.x; j < NQ; j += blockDim.x) { out[(size_t)j * kPartStride] = -INFINITY; out[(size_t)j * kPartStride + 1] = 0.f; }
    return;
  }
  const int k1 = min(Lmax, k0 + chunk);
  // the 16 query rows (zeros beyond NQ)
  for (int i = threadIdx.x; i < 16 * 32; i += blockDim.x) {
    const int j = i >> 5, piece = i & 31;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (j < NQ) {
      const int h = kvh * G + j / Tb, tl = j % Tb;
      v = ldg128(q + (((size_t)b * Tb + tl) * Hq + h) * HD + 8 * piece);
    }
    *reinterpret_cast<uint4*>(asm_ + j * kAttRowB + 16 * piece) = v;
  }
  __syncthreads();
  uint8_t* mine = asm_ + 16 * kAttRowB + warp * kAttWarpBytes;
  const uint32_t q_s = smem_u32(asm_), mine_s = smem_u32(mine);
  const size_t base = (((size_t)b * Hkv + kvh) * cap) * HD;
  const int ntiles = (k1 - k0 + 15) / 16;
  const int my_tiles = ntiles > warp ? (ntiles - warp + kAttWarps - 1) / kAttWarps : 0;
  auto issue = [&](int i) {  // this warp's i-th tile into stage i % kAttStages
    if (i < my_tiles) {
      const int n0 = k0 + 16 * (warp + kAttWarps * i);
      const uint32_t dst = mine_s + (i % kAttStages) * 2 * kAttTile;
#pragma unroll
      for (int it = 0; it < 16; ++it) {
        const int p = it * 32 + lane, row = p >> 5, piece = p & 31;
        const int n = n0 + row;
        const int ok = n < Lmax ? 16 : 0;
        const size_t src = base + (size_t)min(n, cap - 1) * HD + 8 * piece;
        cp_async16(dst + row * kAttRowB + 16 * piece, kc + src, ok);
        cp_async16(dst + kAttTile + row * kAttRowB + 16 * piece, vc + src, ok);
      }
    }
    cp_async_commit();
  };
  float o[32][4];
#pragma unroll
  for (int nt = 0; nt < 32; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows g and g + 8, base-2 domain
  const float sc2 = scale * 1.4426950408889634f;
  const int lim0 = p0 + (g % Tb) + 1, lim1 = p0 + ((g + 8) % Tb) + 1;  // keys below these are visible to the row
  // ldmatrix lane addresses: A (queries), B of Q K^T (keys x dims), B of P V (keys x dims, transposed)
  const uint32_t a_off = ((lane & 7) + 8 * ((lane >> 3) & 1)) * kAttRowB + 16 * (lane >> 4);
  const uint32_t k_off = ((lane & 7) + 8 * (lane >> 4)) * kAttRowB + 16 * ((lane >> 3) & 1);
  const uint32_t v_off = ((lane & 7) + 8 * ((lane >> 3) & 1)) * kAttRowB + 16 * (lane >> 4);
  issue(0);
  issue(1);
  for (int i = 0; i < my_tiles; ++i) {
    issue(i + 2);
    cp_async_wait<2>();
    __syncwarp();
    const uint32_t ks = mine_s + (i % kAttStages) * 2 * kAttTile, vs = ks + kAttTile;
    const int n0 = k0 + 16 * (warp + kAttWarps * i);
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      uint32_t a[4], bk[4];
      ldsm4(q_s + a_off + 32 * kk, a);
      ldsm4(ks + k_off + 32 * kk, bk);
      mma16816(s[0], a, bk[0], bk[1]);
      mma16816(s[1], a, bk[2], bk[3]);
    }
    const bool all_visible = n0 + 16 <= p0 + 1;  // warp-uniform: no row of the window masks a key of this tile
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
    const float u0 = n0m == -INFINITY ? 0.f : n0m, u1 = n1m == -INFINITY ? 0.f : n1m;  // a row that has seen no key yet
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
    __syncwarp();  // the stage is refilled by the next iteration's issue
  }
  cp_async_wait<0>();
  __syncwarp();
  // this warp's partial into its own pipeline memory: out[16][256] f32, then max[16], sum[16]
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  float* wo = reinterpret_cast<float*>(mine);
#pragma unroll
  for (int nt = 0; nt < 32; ++nt) {
    *reinterpret_cast<float2*>(wo + g * HD + 8 * nt + 2 * qd) = make_float2(o[nt][0], o[nt][1]);
    *reinterpret_cast<float2*>(wo + (g + 8) * HD + 8 * nt + 2 * qd) = make_float2(o[nt][2], o[nt][3]);
  }
  if (qd == 0) {
    wo[16 * HD + g] = m0; wo[16 * HD + g + 8] = m1;
    wo[16 * HD + 16 + g] = l0; wo[16 * HD + 16 + g + 8] = l1;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < NQ * HD; idx += blockDim.x) {
    const int j = idx / HD, d = idx - j * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttWarps; ++w) M = fmaxf(M, reinterpret_cast<const float*>(asm_ + 16 * kAttRowB + w * kAttWarpBytes)[16 * HD + j]);
    float S = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kAttWarps; ++w) {
      const float* r = reinterpret_cast<const float*>(asm_ + 16 * kAttRowB + w * kAttWarpBytes);
      const float mw = r[16 * HD + j];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
      S = fmaf(r[16 * HD + 16 + j], f, S);
      O = fmaf(r[j * HD + d], f, O);
    }
    float* dst = out + (size_t)j * kPartStride;
    if (d == 0) { dst[0] = M * 0.6931471805599453f; dst[1] = S; }  // the merge works in the natural-log domain
    dst[8 + d] = O;
  }
}

// grid (NQ, Hkv, B), 256 threads (one per dim): merge the chunks, apply the output gate
__global__ void __launch_bounds__(256) battn_merge_kernel(const float* __restrict__ part, const bf16_t* __restrict__ qg /*[B*Tb, Hq, 512]: query | gate*/,
                                                          int Tb, int Hq, int Hkv, int nchunks, int NQ, bf16_t* __restrict__ out /*[B*Tb, Hq*256]*/) {
  constexpr int HD = 256;
  const int j = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, d = threadIdx.x;
  const int G = Hq / Hkv, h = kvh * G + j / Tb, tl = j % Tb;
  const float* p = part + (((size_t)b * Hkv + kvh) * nchunks) * NQ * kPartStride + (size_t)j * kPartStride;
  float M = -INFINITY;
  for (int c = 0; c < nchunks; ++c) M = fmaxf(M, p[(size_t)c * NQ * kPartStride]);
  float S = 0.f, O = 0.f;
  for (int c = 0; c < nchunks; ++c) {
    const float* pc = p + (size_t)c * NQ * kPartStride;
    const float f = pc[0] == -INFINITY ? 0.f : orn_expf(pc[0] - M);
    S = fmaf(pc[1], f, S);
    O = fmaf(pc[8 + d], f, O);
  }
  const float att = bfr(O / S);
  const size_t row = (size_t)b * Tb + tl;
  const float gate = bf2f(qg[(row * Hq + h) * 2 * HD + HD + d]);
  out[(row * Hq + h) * HD + d] = f2bf(orn_sigmoid_bf(gate) * att);
}

int launch_battn(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* kc, const bf16_t* vc, const int* pos, int B, int Tb,
                 int Hq, int Hkv, int cap, float scale, float* part, int nchunks, int chunk, int NQ) {
  int rc = orn_grant_smem(ctx, reinterpret_cast<const void*>(battn_partial_kernel), kAttSmem);
  if (rc != ORN_OK) return rc;
  dim3 grid(nchunks, Hkv, B);
  battn_partial_kernel<<<grid, kAttWarps * 32, kAttSmem, s>>>(q, kc, vc, pos, Tb, Hq, Hkv, cap, scale, part, nchunks, chunk, NQ);
  return orn_launch_check(ctx, "battn_partial");
}

}  // namespace

struct orn_batch {
  orn_model* m = nullptr;
  orn_ep *own_ep = nullptr, *own_ep_exact = nullptr;  // one-rank groups for calls that pass none (made on first use)
  int B = 0, Tmax = 0, cap = 0, nring = 0, conv_rows = 0;
  bool exact = false;  // ORN_BATCH_EXACT or ORN_WIDE_EXACT=1: every product row-invariant
  bool split_attn = false;  // ORN_BATCH_SPLIT_ATTN: the split-KV attention whatever the row count
  std::vector<bf16_t*> kc, vc, conv;  // per layer
  std::vector<float*> ring;           // per layer: [B][nring][Hv,128,128]
  bf16_t** conv_table = nullptr;
  int n_gdn = 0;
  int *pos = nullptr, *cur = nullptr, *keep = nullptr;  // device [B]
  std::vector<int> h_pos;
  std::vector<void*> allocs;
  // activation scratch for R = B * Tmax rows
  uint32_t *ids, *targets, *conv_map;
  bf16_t *x, *n, *r, *h, *n2, *mo, *qkv, *z, *a, *b, *gq, *gk, *gv, *beta, *gy, *gated;
  float* gg;
  bf16_t *qg, *aq, *agate, *ak, *av, *att, *agated, *logits;
  float *greedy_scratch, *part;
  int part_chunks = 0;
  // the MTP head's per-sequence state (depth 1): its own KV cache and positions, the hidden row its next draft reads
  bf16_t *mtp_kc = nullptr, *mtp_vc = nullptr, *hrow = nullptr, *hid0 = nullptr;
  bf16_t *memb = nullptr, *me = nullptr, *mh = nullptr, *mjoined = nullptr, *mx = nullptr, *dhid = nullptr;
  uint32_t *prim = nullptr, *tok1 = nullptr, *drafts = nullptr;
  int* mtp_pos = nullptr;
  std::vector<int> h_mtp_pos;
  bool drafted = false;  // a draft was made for the window in flight: commit re-encodes what it accepts
  std::vector<orn_linear*> mtp_views;  // this rank's slices of the MTP layer's experts
  int last_T = 0;
  uint32_t *ids_h = nullptr, *targets_h = nullptr;  // pinned staging: a captured step copies from / to fixed host addresses
  bf16_t* normed = nullptr;                          // the rows after the final norm of the last step
  struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    int seen = 0;
    int64_t launches = 0;
    orn_ep* group = nullptr;
  };
  std::map<uint64_t, StepGraph> graphs;  // keyed by (rows per window, split-KV launch shape, arithmetic)
  // this rank's slices of the routed experts when the group has several ranks (views, not copies)
  int shard_rank = -1, shard_world = 0;
  std::vector<orn_linear*> views;  // [layer][3]
};

namespace {

int batch_mm(orn_batch* bt, const orn_linear* L, const bf16_t* x, int R, bf16_t* y) {
  orn_ctx* ctx = bt->m->ctx;
  if (R >= 16 && !bt->exact && L->K % 64 == 0) return f_qgemm(ctx, ctx->stream, L, x, R, y, L->O, nullptr, nullptr);
  for (int r = 0; r < R; r += kMaxRows) {
    const int n = std::min(kMaxRows, R - r);
    CK(k_gemv(ctx, ctx->stream, L, x + (size_t)r * L->K, n, y + (size_t)r * L->O, 0));
  }
  return ORN_OK;
}

// several projections of the same rows: consecutive matrices that share format and row length go
// out as one tensor-core launch (their feature tiles form one tile space)
int batch_mm_multi(orn_batch* bt, const orn_linear* const* Ls, bf16_t* const* ys, int n, const bf16_t* x, int R) {
  orn_ctx* ctx = bt->m->ctx;
  if (!(R >= 16 && !bt->exact)) {
    for (int i = 0; i < n; ++i) CK(batch_mm(bt, Ls[i], x, R, ys[i]));
    return ORN_OK;
  }
  // the first group of matrices on the main stream, the others beside it on the side stream (a small
  // projection of another format next to the big one is a launch of a few CTAs that would otherwise wait
  // its turn); the side stream's products have their own split-K scratch
  bool forked = false;
  int i = 0;
  while (i < n) {
    int j = i + 1;
    while (j < n && j - i < 4 && Ls[j]->kind == Ls[i]->kind && Ls[j]->K == Ls[i]->K && Ls[i]->K % 64 == 0) ++j;
    cudaStream_t st = ctx->stream;
    if (i > 0 && Ls[i]->K % 64 == 0 && orn_side_stream(ctx)) {
      if (!forked) {
        ORN_CHECK_CUDA(ctx, cudaEventRecord(ctx->ev_fork, ctx->stream));
        ORN_CHECK_CUDA(ctx, cudaStreamWaitEvent(ctx->side, ctx->ev_fork, 0));
        forked = true;
      }
      st = ctx->side;
    }
    void* yv[4];
    int ld[4];
    for (int k = i; k < j; ++k) { yv[k - i] = ys[k]; ld[k - i] = Ls[k]->O; }
    if (Ls[i]->K % 64 == 0) CK(f_qgemm_multi(ctx, st, Ls + i, yv, ld, j - i, x, R));
    else for (int k = i; k < j; ++k) CK(batch_mm(bt, Ls[k], x, R, ys[k]));
    i = j;
  }
  if (forked) {
    ORN_CHECK_CUDA(ctx, cudaEventRecord(ctx->ev_join, ctx->side));
    ORN_CHECK_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_join, 0));
  }
  return ORN_OK;
}

// views of this rank's E / world experts of every layer's routed matrices
int ensure_shards(orn_batch* bt, int rank, int world) {
  if (bt->shard_rank == rank && bt->shard_world == world) return ORN_OK;
  for (orn_linear* v : bt->views) delete v;
  bt->views.clear();
  orn_model* m = bt->m;
  if (m->cfg.n_experts % world) ORN_FAIL(m->ctx, ORN_ERR_ARG, "batch: the experts do not split evenly over the ranks");
  const int el = m->cfg.n_experts / world;
  for (const Layer& ly : m->layers) {
    const orn_linear* full[3] = {ly.moe.sw_gate, ly.moe.sw_up, ly.moe.sw_down};
    for (const orn_linear* f : full) {
      orn_linear* v = new orn_linear(*f);
      v->E = el;
      const size_t off = (size_t)rank * el * f->O * f->rec;
      v->w = f->w + off; v->s = f->s + off; v->b = f->b + off;
      v->w_bytes = (size_t)el * f->O * f->rec;
      v->owns = false;
      bt->views.push_back(v);
    }
  }
  for (orn_linear* v : bt->mtp_views) delete v;
  bt->mtp_views.clear();
  if (m->mtp.present) {
    const orn_linear* full[3] = {m->mtp.moe.sw_gate, m->mtp.moe.sw_up, m->mtp.moe.sw_down};
    for (const orn_linear* f : full) {
      orn_linear* v = new orn_linear(*f);
      v->E = el;
      const size_t off = (size_t)rank * el * f->O * f->rec;
      v->w = f->w + off; v->s = f->s + off; v->b = f->b + off;
      v->w_bytes = (size_t)el * f->O * f->rec;
      v->owns = false;
      bt->mtp_views.push_back(v);
    }
  }
  bt->shard_rank = rank; bt->shard_world = world;
  return ORN_OK;
}

// the attention sub-block over bt->n for B * T rows (T rows per sequence at positions pos[b] ...):
// projections, per-head norms, RoPE, KV append, attention, output gate, output projection -> bt->r.
// kv_only: stop after the KV rows are in the cache (the MTP head's re-encode of accepted tokens)
int batch_attention(orn_batch* bt, const orn_linear* q_proj, const orn_linear* k_proj, const orn_linear* v_proj,
                    const orn_linear* o_proj, const bf16_t* q_norm, const bf16_t* k_norm, int T, const int* pos, bf16_t* kc,
                    bf16_t* vc, bool exact, int chunk, int nchunks, bool kv_only) {
  orn_model* m = bt->m;
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  const orn_config& c = m->cfg;
  const int B = bt->B, R = B * T, Hq = c.n_heads, Hkv = c.n_kv_heads, hd = c.head_dim, NQ = (Hq / Hkv) * T;
  {
    const orn_linear* pl[3] = {k_proj, v_proj, q_proj};
    bf16_t* py[3] = {bt->ak, bt->av, bt->qg};
    CK(batch_mm_multi(bt, pl, py, kv_only ? 2 : 3, bt->n, R));
  }
  CK(k_rms_norm(ctx, s, bt->ak, k_norm, R * Hkv, hd, c.rms_eps, bt->ak));
  CK(k_rope_batched(ctx, s, bt->ak, B, T, Hkv, hd, c.rope_dims, m->lnb, pos));
  CK(k_kv_append_batched(ctx, s, bt->ak, bt->av, B, T, Hkv, hd, bt->cap, pos, kc, vc));
  if (kv_only) return ORN_OK;
  CK(k_split_qgate(ctx, s, bt->qg, R, Hq, hd, bt->aq, bt->agate));
  CK(k_rms_norm(ctx, s, bt->aq, q_norm, R * Hq, hd, c.rms_eps, bt->aq));
  CK(k_rope_batched(ctx, s, bt->aq, B, T, Hq, hd, c.rope_dims, m->lnb, pos));
  const float scale = 1.0f / sqrtf((float)hd);
  if ((exact && !bt->split_attn) || hd != 256 || NQ > 16) {
    CK(k_sdpa_decode_batched(ctx, s, bt->aq, kc, vc, B, T, Hq, Hkv, hd, bt->cap, pos, scale, bt->att));
    CK(k_sigmoid_gate(ctx, s, bt->agate, bt->att, R * Hq * hd, 1, bt->agated));
  } else {
    CK(launch_battn(ctx, s, bt->aq, kc, vc, pos, B, T, Hq, Hkv, bt->cap, scale, bt->part, nchunks, chunk, NQ));
    dim3 grid(NQ, Hkv, B);
    battn_merge_kernel<<<grid, 256, 0, s>>>(bt->part, bt->qg, T, Hq, Hkv, nchunks, NQ, bt->agated);
    CK(orn_launch_check(ctx, "battn_merge"));
  }
  return batch_mm(bt, o_proj, bt->agated, R, bt->r);
}

// keys per CTA of the split-KV attention: about six CTAs per SM over the whole launch, 128..512, a
// multiple of 64; the launch covers the longest sequence (shorter ones leave chunks empty)
void split_shape(const orn_batch* bt, int maxL, int* chunk, int* nchunks) {
  const orn_ctx* ctx = bt->m->ctx;
  int ch = (int)(((int64_t)maxL * bt->B * bt->m->cfg.n_kv_heads / (ctx->sm_count * 6) + 63) / 64 * 64);
  ch = std::min(kMaxChunk, std::max(kMinChunk, ch));
  *chunk = ch;
  *nchunks = (maxL + ch - 1) / ch;
}

// the MTP head's input for B rows: fc([norm(embed(ids)) | norm(hidden)]) -> bt->mx (MtpHead::hidden, mtp.rs:150-190)
int mtp_join(orn_batch* bt, const uint32_t* dev_ids, const bf16_t* hidden) {
  orn_model* m = bt->m;
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  const orn_config& c = m->cfg;
  const Mtp& h = m->mtp;
  const int B = bt->B, H = c.hidden;
  CK(k_embedding(ctx, s, m->embed, dev_ids, B, bt->memb));
  CK(k_rms_norm(ctx, s, bt->memb, h.pre_fc_norm_embedding, B, H, c.rms_eps, bt->me));
  CK(k_rms_norm(ctx, s, hidden, h.pre_fc_norm_hidden, B, H, c.rms_eps, bt->mh));
  CK(k_concat2(ctx, s, bt->me, bt->mh, B, H, bt->mjoined));
  CK(batch_mm(bt, h.fc, bt->mjoined, B, bt->mx));
  return k_rms_norm(ctx, s, bt->mx, h.input_ln, B, H, c.rms_eps, bt->n);
}

__global__ void gather_window_kernel(const uint32_t* ids, const bf16_t* normed, const int* keep, int T, int H, uint32_t* tok1,
                                     bf16_t* hid0, bf16_t* hrow) {
  // per sequence b: the window's second token, its first hidden row (the re-encode's inputs) and
  // the hidden row of the last kept position (the next draft's input)
  const int b = blockIdx.x;
  if (threadIdx.x == 0 && T > 1) tok1[b] = ids[b * T + 1];
  const uint4* r0 = reinterpret_cast<const uint4*>(normed + (size_t)(b * T) * H);
  const uint4* rk = reinterpret_cast<const uint4*>(normed + (size_t)(b * T + keep[b] - 1) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    reinterpret_cast<uint4*>(hid0 + (size_t)b * H)[i] = r0[i];
    reinterpret_cast<uint4*>(hrow + (size_t)b * H)[i] = rk[i];
  }
}
__global__ void mtp_advance_kernel(int* mtp_pos, const int* keep, int B, int base) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) mtp_pos[b] += base + (keep ? keep[b] - 1 : 0);
}

// the device work of one step: everything between the upload of the ids and the download of the
// targets, with fixed addresses and launch shapes (so that it can be captured once and replayed)
int batch_body(orn_batch* bt, orn_ep* group, int T, int chunk, int nchunks) {
  orn_model* m = bt->m;
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  const orn_config& c = m->cfg;
  const int B = bt->B, R = B * T, H = c.hidden, S = c.gdn_conv_kernel - 1, D = orn_conv_dim(c);
  const int Hq = c.n_heads, Hkv = c.n_kv_heads, hd = c.head_dim;
  const bool exact = bt->exact || R < 16;
  const int world = orn_ep_world(group);
  ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(bt->ids, bt->ids_h, sizeof(uint32_t) * (size_t)R, cudaMemcpyHostToDevice, s));
  conv_map_kernel<<<(R + 127) / 128, 128, 0, s>>>(bt->conv_map, B, T, bt->conv_rows, S);
  CK(orn_launch_check(ctx, "conv_map"));
  CK(k_embedding(ctx, s, m->embed, bt->ids, R, bt->x));
  CK(k_rms_norm(ctx, s, bt->x, m->layers[0].input_ln, R, H, c.rms_eps, bt->n));
  for (int i = 0; i < c.n_layers; ++i) {
    const Layer& ly = m->layers[i];
    if (ly.linear) {
      const orn_linear* pl[4] = {ly.in_qkv, ly.in_z, ly.in_b, ly.in_a};
      bf16_t* py[4] = {bt->qkv, bt->z, bt->b, bt->a};
      CK(batch_mm_multi(bt, pl, py, 4, bt->n, R));
      scatter_rows_kernel<<<R, 128, 0, s>>>(bt->qkv, bt->conv_map, D, bt->conv[i]);  // row (b, t) -> window row S + t of sequence b
      CK(orn_launch_check(ctx, "scatter_rows"));
      CK(k_gdn_front_batched(ctx, s, bt->conv[i], (int64_t)bt->conv_rows * D, ly.conv_w, bt->a, bt->b, ly.a_log, ly.dt_bias, B, T,
                             c.gdn_k_heads, c.gdn_v_heads, c.gdn_head_dim, c.gdn_conv_kernel, 1e-6f, bt->gq, bt->gk, bt->gv,
                             bt->beta, bt->gg));
      CK(k_gated_delta_batched(ctx, s, bt->gq, bt->gk, bt->gv, bt->gg, bt->beta, bt->ring[i], bt->nring, bt->cur, B, T,
                               c.gdn_k_heads, c.gdn_v_heads, bt->gy));
      CK(k_rms_norm_gated(ctx, s, bt->gy, ly.gdn_norm, bt->z, R * c.gdn_v_heads, c.gdn_head_dim, c.rms_eps, bt->gated));
      CK(batch_mm(bt, ly.out_proj, bt->gated, R, bt->r));
    } else {
      CK(batch_attention(bt, ly.q_proj, ly.k_proj, ly.v_proj, ly.o_proj, ly.q_norm, ly.k_norm, T, bt->pos, bt->kc[i], bt->vc[i], exact,
                         chunk, nchunks, false));
    }
    CK(k_add_rms_norm(ctx, s, bt->x, bt->r, ly.post_ln, R, H, c.rms_eps, bt->h, bt->n2));
    const orn_linear* sg = world > 1 ? bt->views[3 * i] : ly.moe.sw_gate;
    const orn_linear* su = world > 1 ? bt->views[3 * i + 1] : ly.moe.sw_up;
    const orn_linear* sd = world > 1 ? bt->views[3 * i + 2] : ly.moe.sw_down;
    CK(orn_ep_moe_block(group, ly.moe.gate, sg, su, sd, ly.moe.sh_gate, ly.moe.sh_up, ly.moe.sh_down, ly.moe.sh_egate, bt->n2, R,
                        c.top_k, c.norm_topk_prob, bt->mo, nullptr));
    const bf16_t* nw = i + 1 < c.n_layers ? m->layers[i + 1].input_ln : m->norm;
    CK(k_add_rms_norm(ctx, s, bt->h, bt->mo, nw, R, H, c.rms_eps, bt->x, bt->n));
  }
  ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(bt->normed, bt->n, sizeof(bf16_t) * (size_t)R * H, cudaMemcpyDeviceToDevice, s));  // the head's input survives it
  CK(batch_mm(bt, m->lm_head, bt->n, R, bt->logits));
  CK(k_greedy(ctx, s, bt->logits, R, c.vocab, 1, bt->targets, bt->greedy_scratch));
  ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(bt->targets_h, bt->targets, sizeof(uint32_t) * (size_t)R, cudaMemcpyDeviceToHost, s));
  return ORN_OK;
}

}  // namespace

extern "C" {

int32_t orn_batch_destroy(orn_batch* bt) {
  if (!bt) return ORN_OK;
  cudaStreamSynchronize(bt->m->ctx->stream);
  for (auto& kv : bt->graphs)
    if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
  for (void* p : bt->allocs) cudaFree(p);
  if (bt->ids_h) cudaFreeHost(bt->ids_h);
  if (bt->targets_h) cudaFreeHost(bt->targets_h);
  for (orn_linear* v : bt->views) delete v;
  for (orn_linear* v : bt->mtp_views) delete v;
  if (bt->own_ep) orn_ep_destroy(bt->own_ep);
  if (bt->own_ep_exact) orn_ep_destroy(bt->own_ep_exact);
  delete bt;
  return ORN_OK;
}

int32_t orn_batch_create(orn_model* m, int32_t B, int32_t T_max, int32_t cap, int32_t flags, orn_batch** out) {
  if (!m || !out) return ORN_ERR_ARG;
  *out = nullptr;
  CK(orn_model_finalize(m));
  orn_ctx* ctx = m->ctx;
  const orn_config& c = m->cfg;
  if (B < 1 || T_max < 1 || T_max > kMaxRows || cap < 8) ORN_FAIL(ctx, ORN_ERR_ARG, "batch_create: 1..4 rows per window, at least one sequence");
  orn_batch* bt = new orn_batch();
  bt->m = m; bt->B = B; bt->Tmax = T_max; bt->cap = cap; bt->nring = T_max + 1;
  bt->exact = (flags & ORN_BATCH_EXACT) != 0 || orn_wide_exact();
  bt->split_attn = (flags & ORN_BATCH_SPLIT_ATTN) != 0;
  const int S = c.gdn_conv_kernel - 1, D = orn_conv_dim(c);
  bt->conv_rows = S + T_max;
  bt->kc.assign(c.n_layers, nullptr); bt->vc.assign(c.n_layers, nullptr);
  bt->conv.assign(c.n_layers, nullptr); bt->ring.assign(c.n_layers, nullptr);
  bt->h_pos.assign(B, 0);
  bt->h_mtp_pos.assign(B, 0);
  int rc = ORN_OK;
  auto A = [&](auto** p, size_t n) {
    if (rc != ORN_OK) return;
    void* d = nullptr;
    rc = orn_alloc(ctx, sizeof(**p) * (n ? n : 1), &d);
    if (rc == ORN_OK) { bt->allocs.push_back(d); *p = (std::remove_reference_t<decltype(**p)>*)d; }
  };
  const size_t kvsz = (size_t)B * c.n_kv_heads * cap * c.head_dim;
  const size_t ssz = (size_t)c.gdn_v_heads * 128 * 128;
  std::vector<bf16_t*> table;
  for (int i = 0; i < c.n_layers; ++i) {
    if (m->layers[i].linear) {
      A(&bt->conv[i], (size_t)B * bt->conv_rows * D);
      A(&bt->ring[i], (size_t)B * bt->nring * ssz);
      table.push_back(bt->conv[i]);
    } else {
      A(&bt->kc[i], kvsz);
      A(&bt->vc[i], kvsz);
    }
  }
  bt->n_gdn = (int)table.size();
  const size_t R = (size_t)B * T_max, H = c.hidden, VD = (size_t)c.gdn_v_heads * c.gdn_head_dim;
  const size_t KD = (size_t)c.gdn_k_heads * c.gdn_head_dim, QD = (size_t)c.n_heads * c.head_dim, KVD = (size_t)c.n_kv_heads * c.head_dim;
  A(&bt->pos, (size_t)B); A(&bt->cur, (size_t)B); A(&bt->keep, (size_t)B);
  A(&bt->ids, R); A(&bt->targets, R); A(&bt->conv_map, R);
  A(&bt->x, R * H); A(&bt->n, R * H); A(&bt->r, R * H); A(&bt->h, R * H); A(&bt->n2, R * H); A(&bt->mo, R * H);
  A(&bt->qkv, R * D); A(&bt->z, R * VD); A(&bt->a, R * c.gdn_v_heads); A(&bt->b, R * c.gdn_v_heads);
  A(&bt->gq, R * KD); A(&bt->gk, R * KD); A(&bt->gv, R * VD); A(&bt->beta, R * c.gdn_v_heads); A(&bt->gg, R * c.gdn_v_heads);
  A(&bt->gy, R * VD); A(&bt->gated, R * VD);
  A(&bt->qg, R * 2 * QD); A(&bt->aq, R * QD); A(&bt->agate, R * QD); A(&bt->ak, R * KVD); A(&bt->av, R * KVD);
  A(&bt->att, R * QD); A(&bt->agated, R * QD);
  A(&bt->logits, R * (size_t)c.vocab);
  A(&bt->normed, R * H);
  if (m->mtp.present) {
    A(&bt->mtp_kc, kvsz); A(&bt->mtp_vc, kvsz); A(&bt->hrow, (size_t)B * H); A(&bt->hid0, (size_t)B * H);
    A(&bt->memb, (size_t)B * H); A(&bt->me, (size_t)B * H); A(&bt->mh, (size_t)B * H); A(&bt->mjoined, (size_t)2 * B * H);
    A(&bt->mx, (size_t)B * H); A(&bt->dhid, (size_t)B * H); A(&bt->prim, (size_t)B); A(&bt->tok1, (size_t)B); A(&bt->drafts, (size_t)B);
    A(&bt->mtp_pos, (size_t)B);
  }
  A(&bt->greedy_scratch, greedy_scratch_floats((int)R, c.vocab));
  bt->part_chunks = (cap + kMinChunk - 1) / kMinChunk;
  A(&bt->part, (size_t)B * c.n_kv_heads * bt->part_chunks * 16 * kPartStride);
  if (rc == ORN_OK && bt->n_gdn) {
    A(&bt->conv_table, table.size());
    if (rc == ORN_OK) rc = orn_upload(ctx, bt->conv_table, table.data(), sizeof(bf16_t*) * table.size());
  }
  if (rc != ORN_OK) { orn_batch_destroy(bt); return rc; }
  if (cudaMallocHost((void**)&bt->ids_h, sizeof(uint32_t) * R) != cudaSuccess ||
      cudaMallocHost((void**)&bt->targets_h, sizeof(uint32_t) * R) != cudaSuccess) {
    ctx->err = "batch_create: pinned staging";
    orn_batch_destroy(bt);
    return ORN_ERR_ALLOC;
  }
  *out = bt;
  return orn_batch_reset(bt);
}

// make_cache for every sequence (cache.rs:160-181): zero conv windows and states, empty KV
int32_t orn_batch_reset(orn_batch* bt) {
  if (!bt) return ORN_ERR_ARG;
  orn_model* m = bt->m;
  const orn_config& c = m->cfg;
  const size_t ssz = sizeof(float) * (size_t)c.gdn_v_heads * 128 * 128;
  for (int i = 0; i < c.n_layers; ++i)
    if (m->layers[i].linear) {
      CK(orn_memset(m->ctx, bt->conv[i], 0, sizeof(bf16_t) * (size_t)bt->B * bt->conv_rows * orn_conv_dim(c)));
      CK(orn_memset(m->ctx, bt->ring[i], 0, ssz * bt->nring * bt->B));
    }
  CK(orn_memset(m->ctx, bt->pos, 0, sizeof(int) * bt->B));
  CK(orn_memset(m->ctx, bt->cur, 0, sizeof(int) * bt->B));
  std::fill(bt->h_pos.begin(), bt->h_pos.end(), 0);
  if (bt->mtp_pos) {
    CK(orn_memset(m->ctx, bt->mtp_pos, 0, sizeof(int) * bt->B));
    CK(orn_memset(m->ctx, bt->hrow, 0, sizeof(bf16_t) * (size_t)bt->B * c.hidden));
    std::fill(bt->h_mtp_pos.begin(), bt->h_mtp_pos.end(), 0);
  }
  bt->drafted = false;
  bt->last_T = 0;
  return orn_sync(m->ctx);
}

// Benchmark set-up: every sequence as if it had decoded ctx_len tokens: seeded random KV rows, conv
// windows and recurrent states (the traffic and arithmetic of a step do not depend on the values).
int32_t orn_batch_fill_random(orn_batch* bt, int32_t ctx_len, uint64_t seed) {
  if (!bt || ctx_len < 0 || ctx_len + bt->Tmax > bt->cap) return ORN_ERR_ARG;
  orn_model* m = bt->m;
  orn_ctx* ctx = m->ctx;
  const orn_config& c = m->cfg;
  const size_t kvsz = (size_t)bt->B * c.n_kv_heads * bt->cap * c.head_dim;
  const size_t ssz = (size_t)c.gdn_v_heads * 128 * 128;
  for (int i = 0; i < c.n_layers; ++i) {
    if (m->layers[i].linear) {
      CK(k_fill_bf16(ctx, ctx->stream, bt->conv[i], (size_t)bt->B * bt->conv_rows * orn_conv_dim(c), seed + 31 * i, 0.f, 0.5f));
      const size_t n = (size_t)bt->B * bt->nring * ssz;
      fill_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(bt->ring[i], n, seed + 77 * i, 0.05f);
      CK(orn_launch_check(ctx, "fill_f32"));
    } else {
      CK(k_fill_bf16(ctx, ctx->stream, bt->kc[i], kvsz, seed + 13 * i, 0.f, 1.0f));
      CK(k_fill_bf16(ctx, ctx->stream, bt->vc[i], kvsz, seed + 17 * i, 0.f, 1.0f));
    }
  }
  set_ints_kernel<<<(bt->B + 127) / 128, 128, 0, ctx->stream>>>(bt->pos, bt->B, ctx_len);
  CK(orn_launch_check(ctx, "set_ints"));
  std::fill(bt->h_pos.begin(), bt->h_pos.end(), ctx_len);
  if (bt->mtp_pos) {  // the MTP head's cache as far along as the trunk's, a random hidden row to draft from
    CK(k_fill_bf16(ctx, ctx->stream, bt->mtp_kc, kvsz, seed + 1001, 0.f, 1.0f));
    CK(k_fill_bf16(ctx, ctx->stream, bt->mtp_vc, kvsz, seed + 1003, 0.f, 1.0f));
    CK(k_fill_bf16(ctx, ctx->stream, bt->hrow, (size_t)bt->B * c.hidden, seed + 1005, 0.f, 1.0f));
    set_ints_kernel<<<(bt->B + 127) / 128, 128, 0, ctx->stream>>>(bt->mtp_pos, bt->B, ctx_len);
    CK(orn_launch_check(ctx, "set_ints"));
    std::fill(bt->h_mtp_pos.begin(), bt->h_mtp_pos.end(), ctx_len);
  }
  return orn_sync(ctx);
}

int32_t orn_batch_positions(orn_batch* bt, int32_t* host_pos) {
  if (!bt || !host_pos) return ORN_ERR_ARG;
  for (int b = 0; b < bt->B; ++b) host_pos[b] = bt->h_pos[b];
  return ORN_OK;
}

int32_t orn_batch_forward(orn_batch* bt, orn_ep* ep, const uint32_t* host_ids, int32_t T, uint16_t* dev_normed,
                          uint32_t* host_targets) {
  if (!bt || !host_ids) return ORN_ERR_ARG;
  orn_model* m = bt->m;
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  const orn_config& c = m->cfg;
  if (T < 1 || T > bt->Tmax) ORN_FAIL(ctx, ORN_ERR_ARG, "batch_forward: window wider than the batch was made for");
  for (int b = 0; b < bt->B; ++b)
    if (bt->h_pos[b] + T > bt->cap) ORN_FAIL(ctx, ORN_ERR_STATE, "batch_forward: a sequence would pass the cache capacity");
  const int B = bt->B, R = B * T;
  const bool exact = bt->exact || R < 16;
  orn_ep* group = ep;
  if (!group) {
    orn_ep** own = exact ? &bt->own_ep_exact : &bt->own_ep;
    if (!*own) CK(orn_ep_init(ctx, nullptr, 0, 1, exact ? ORN_EP_EXACT : 0, own));
    group = *own;
  }
  const int world = orn_ep_world(group), rank = orn_ep_rank(group);
  if (world > 1) CK(ensure_shards(bt, rank, world));
  int max_pos = 0;
  for (int b = 0; b < B; ++b) max_pos = std::max(max_pos, bt->h_pos[b]);
  int chunk, nchunks;
  split_shape(bt, max_pos + T, &chunk, &nchunks);
  // the previous step's targets have been read (its download synchronised) before ids_h is rewritten
  ORN_CHECK_CUDA(ctx, cudaStreamSynchronize(s));
  memcpy(bt->ids_h, host_ids, sizeof(uint32_t) * (size_t)R);
  static int no_graph = -1;
  if (no_graph < 0) { const char* e = getenv("ORN_NO_GRAPH"); no_graph = (e && e[0] == '1') ? 1 : 0; }
  const bool eager = no_graph || ctx->kt != nullptr;
  const uint64_t key = (uint64_t)T | ((uint64_t)nchunks << 8) | ((uint64_t)chunk << 28) | ((uint64_t)(exact ? 1 : 0) << 40);
  orn_batch::StepGraph& g = bt->graphs[key];
  if (g.exec != nullptr && g.group != group) {  // captured for another group: its collectives belong to that one
    cudaGraphExecDestroy(g.exec);
    g = orn_batch::StepGraph();
  }
  int rc = ORN_OK;
  if (g.exec != nullptr && !eager) {
    ORN_CHECK_CUDA(ctx, cudaGraphLaunch(g.exec, s));
    ctx->launches += g.launches;
  } else if (g.seen == 0 || eager) {
    g.seen += 1;  // the first step of a shape runs eagerly (scratch is allocated on first use); the second is captured
    rc = batch_body(bt, group, T, chunk, nchunks);
  } else {
    const int64_t l0 = ctx->launches;
    ORN_CHECK_CUDA(ctx, cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    rc = batch_body(bt, group, T, chunk, nchunks);
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(s, &graph);
    if (rc != ORN_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (e != cudaSuccess) ORN_FAIL(ctx, ORN_ERR_CUDA, std::string("batch_forward: cudaStreamEndCapture: ") + cudaGetErrorString(e));
    e = cudaGraphInstantiate(&g.exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) { g.exec = nullptr; ORN_FAIL(ctx, ORN_ERR_CUDA, std::string("batch_forward: cudaGraphInstantiate: ") + cudaGetErrorString(e)); }
    g.launches = ctx->launches - l0;
    g.group = group;
    ORN_CHECK_CUDA(ctx, cudaGraphLaunch(g.exec, s));
  }
  if (rc != ORN_OK) return rc;
  bt->last_T = T;
  if (dev_normed)
    ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(dev_normed, bt->normed, sizeof(bf16_t) * (size_t)R * c.hidden, cudaMemcpyDeviceToDevice, s));
  if (host_targets) {
    CK(orn_sync(ctx));
    memcpy(host_targets, bt->targets_h, sizeof(uint32_t) * (size_t)R);
  }
  return ORN_OK;
}

// TrunkCapture::rewind per sequence (qwen3_5.rs:324-348): keep[b] in 1..T rows of the last window
int32_t orn_batch_commit(orn_batch* bt, const int32_t* host_keep) {
  if (!bt || !host_keep) return ORN_ERR_ARG;
  orn_model* m = bt->m;
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  if (bt->last_T == 0) ORN_FAIL(ctx, ORN_ERR_STATE, "batch_commit: no window to commit");
  for (int b = 0; b < bt->B; ++b)
    if (host_keep[b] < 1 || host_keep[b] > bt->last_T) ORN_FAIL(ctx, ORN_ERR_ARG, "batch_commit: keep out of range");
  ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(bt->keep, host_keep, sizeof(int) * bt->B, cudaMemcpyHostToDevice, s));
  commit_kernel<<<(bt->B + 127) / 128, 128, 0, s>>>(bt->pos, bt->cur, bt->keep, bt->B);
  CK(orn_launch_check(ctx, "batch_commit"));
  if (bt->n_gdn > 0) {
    const int S = m->cfg.gdn_conv_kernel - 1, D = orn_conv_dim(m->cfg);
    dim3 grid((D / 8 + 127) / 128, bt->n_gdn, bt->B);
    conv_shift_batched_kernel<<<grid, 128, 0, s>>>(bt->conv_table, bt->keep, S, D, bt->conv_rows);
    CK(orn_launch_check(ctx, "conv_shift"));
  }
  for (int b = 0; b < bt->B; ++b) bt->h_pos[b] += host_keep[b];
  if (bt->mtp_pos) {
    // the next draft reads the hidden row of the last kept position; a window that followed a draft
    // re-encodes the accepted draft token into the MTP head's cache (HistoryPolicy::Committed,
    // mtp_generate.rs:292-301): KV row at the head's next position from (window token 1, hidden row 0),
    // computed for every sequence, kept (the position advanced) only where the draft was accepted
    const int T = bt->last_T, H = m->cfg.hidden;
    gather_window_kernel<<<bt->B, 128, 0, s>>>(bt->ids, bt->normed, bt->keep, T, H, bt->tok1, bt->hid0, bt->hrow);
    CK(orn_launch_check(ctx, "gather_window"));
    if (bt->drafted && T == 2) {
      const Mtp& h = m->mtp;
      const bool exact = bt->exact || bt->B < 16;
      CK(mtp_join(bt, bt->tok1, bt->hid0));
      CK(batch_attention(bt, h.q_proj, h.k_proj, h.v_proj, h.o_proj, h.q_norm, h.k_norm, 1, bt->mtp_pos, bt->mtp_kc, bt->mtp_vc, exact,
                         0, 0, true));
      mtp_advance_kernel<<<(bt->B + 127) / 128, 128, 0, s>>>(bt->mtp_pos, bt->keep, bt->B, 0);
      CK(orn_launch_check(ctx, "mtp_advance"));
      for (int b = 0; b < bt->B; ++b) bt->h_mtp_pos[b] += host_keep[b] - 1;
    }
  }
  bt->drafted = false;
  bt->last_T = 0;
  return ORN_OK;
}

// MtpHead::forward at depth 1 for every sequence (mtp.rs:150-262; the draft chain of
// mtp_generate.rs:99-135): from the token each sequence is about to feed (its primary) and the trunk's
// hidden row at the position that produced it, the draft of the token after it (raw-logit argmax).
int32_t orn_batch_mtp_draft(orn_batch* bt, orn_ep* ep, const uint32_t* host_primary, uint32_t* host_drafts) {
  if (!bt || !host_primary || !host_drafts) return ORN_ERR_ARG;
  orn_model* m = bt->m;
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  const orn_config& c = m->cfg;
  const Mtp& h = m->mtp;
  if (!h.present || !bt->mtp_pos) ORN_FAIL(ctx, ORN_ERR_STATE, "batch_mtp_draft: the model has no MTP head");
  if (bt->last_T != 0) ORN_FAIL(ctx, ORN_ERR_STATE, "batch_mtp_draft: a window is waiting for its commit");
  const int B = bt->B, H = c.hidden;
  for (int b = 0; b < B; ++b)
    if (bt->h_mtp_pos[b] + 2 > bt->cap) ORN_FAIL(ctx, ORN_ERR_STATE, "batch_mtp_draft: a sequence would pass the cache capacity");
  const bool exact = bt->exact || B < 16;
  orn_ep* group = ep;
  if (!group) {
    orn_ep** own = exact ? &bt->own_ep_exact : &bt->own_ep;
    if (!*own) CK(orn_ep_init(ctx, nullptr, 0, 1, exact ? ORN_EP_EXACT : 0, own));
    group = *own;
  }
  const int world = orn_ep_world(group), rank = orn_ep_rank(group);
  if (world > 1) CK(ensure_shards(bt, rank, world));
  int max_pos = 0;
  for (int b = 0; b < B; ++b) max_pos = std::max(max_pos, bt->h_mtp_pos[b]);
  int chunk, nchunks;
  split_shape(bt, max_pos + 1, &chunk, &nchunks);
  CK(orn_upload(ctx, bt->prim, host_primary, sizeof(uint32_t) * (size_t)B));
  CK(mtp_join(bt, bt->prim, bt->hrow));
  CK(batch_attention(bt, h.q_proj, h.k_proj, h.v_proj, h.o_proj, h.q_norm, h.k_norm, 1, bt->mtp_pos, bt->mtp_kc, bt->mtp_vc, exact, chunk,
                     nchunks, false));
  CK(k_add_rms_norm(ctx, s, bt->mx, bt->r, h.post_ln, B, H, c.rms_eps, bt->h, bt->n2));
  const orn_linear* sg = world > 1 ? bt->mtp_views[0] : h.moe.sw_gate;
  const orn_linear* su = world > 1 ? bt->mtp_views[1] : h.moe.sw_up;
  const orn_linear* sd = world > 1 ? bt->mtp_views[2] : h.moe.sw_down;
  CK(orn_ep_moe_block(group, h.moe.gate, sg, su, sd, h.moe.sh_gate, h.moe.sh_up, h.moe.sh_down, h.moe.sh_egate, bt->n2, B, c.top_k,
                      c.norm_topk_prob, bt->mo, nullptr));
  CK(k_add_rms_norm(ctx, s, bt->h, bt->mo, h.norm, B, H, c.rms_eps, bt->x, bt->dhid));
  CK(batch_mm(bt, m->lm_head, bt->dhid, B, bt->logits));
  CK(k_greedy(ctx, s, bt->logits, B, c.vocab, 0, bt->drafts, bt->greedy_scratch));
  mtp_advance_kernel<<<(B + 127) / 128, 128, 0, s>>>(bt->mtp_pos, nullptr, B, 1);
  CK(orn_launch_check(ctx, "mtp_advance"));
  for (int b = 0; b < B; ++b) bt->h_mtp_pos[b] += 1;
  bt->drafted = true;
  return orn_download(ctx, host_drafts, bt->drafts, sizeof(uint32_t) * (size_t)B);
}

}  // extern "C"
