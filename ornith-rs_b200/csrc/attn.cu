// Full-attention decode kernels: rotary embedding, KV append and the
// online-softmax attention over the bf16 KV cache.
//
// Replaces kernels/mlx/.../rope.metal:11-60, kernels/cache.metal (cache_copy)
// and kernels/mlx/.../sdpa_vector.h:15-175 as dispatched by src/ops/rope.rs:
// 23-89, src/model/cache.rs:48-84 and src/ops/sdpa.rs:122-229.
//
// Attention layout: one CTA of 32 warps per (query row, query head).  Key n
// belongs to warp n mod 32 whatever the context length or the window width,
// so row r of a T-row verify window visits its keys in the same order, with
// the same arithmetic, as the same token stepped alone.  A lane holds 8 of the
// 256 head dims; K and V rows are read as one 512-byte coalesced request per
// warp.  The 32 partial (max, sum, out) triples merge through shared memory
// with a fixed butterfly.
#include "orn_internal.h"

namespace {
ORN_D float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
ORN_D float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
ORN_D void widen8(const uint4& v, float* f) {
  f[0] = bf_lo(v.x); f[1] = bf_hi(v.x); f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
  f[4] = bf_lo(v.z); f[5] = bf_hi(v.z); f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
}

// x [T, H, hd] rotated in place on the first `dims` dims, pair (i, i+dims/2)
// Tb > 0: the T rows are Tb-row windows of T / Tb sequences, dev_offset holds one position per sequence
__global__ void rope_kernel(bf16_t* x, int T, int H, int hd, int dims, float lnb,
                            const int* dev_offset, int offset_add, int Tb) {
  const int half = dims / 2;
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * H * half) return;
  const int i = idx % half;
  const int h = (idx / half) % H;
  const int t = idx / (half * H);
  const int seq = Tb > 0 ? t / Tb : 0, tl = Tb > 0 ? t - seq * Tb : t;
  const int offset = (dev_offset ? dev_offset[seq] : 0) + offset_add;
  const float inv_freq = orn_expf(-(float)i * lnb);
  const float ang = (float)(offset + tl) * inv_freq;
  float sn, cs;
  orn_sincosf(ang, &sn, &cs);
  bf16_t* p = x + ((int64_t)t * H + h) * hd;
  const float x1 = bf2f(p[i]), x2 = bf2f(p[i + half]);
  const float t1 = x2 * sn;
  const float t2 = x2 * cs;
  p[i] = f2bf(fmaf(x1, cs, -t1));
  p[i + half] = f2bf(fmaf(x1, sn, t2));
}

// k, v [T, Hkv, hd] -> caches [Hkv, cap, hd] at rows offset..offset+T-1
__global__ void kv_append_kernel(const bf16_t* k, const bf16_t* v, int T, int Hkv, int hd, int cap,
                                 const int* dev_offset, int offset_add, bf16_t* kc, bf16_t* vc, int Tb) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;  // over T*Hkv*hd/8 16-byte pieces
  const int per = hd / 8;
  if (idx >= T * Hkv * per) return;
  const int c = idx % per;
  const int h = (idx / per) % Hkv;
  const int t = idx / (per * Hkv);
  const int seq = Tb > 0 ? t / Tb : 0, tl = Tb > 0 ? t - seq * Tb : t;  // Tb > 0: a cache [Hkv, cap, hd] per sequence
  const int offset = (dev_offset ? dev_offset[seq] : 0) + offset_add;
  if (offset + tl >= cap) return;
  const int64_t src = (((int64_t)t * Hkv + h) * hd) / 8 + c;
  const int64_t dst = ((((int64_t)seq * Hkv + h) * cap + offset + tl) * hd) / 8 + c;
  reinterpret_cast<uint4*>(kc)[dst] = reinterpret_cast<const uint4*>(k)[src];
  reinterpret_cast<uint4*>(vc)[dst] = reinterpret_cast<const uint4*>(v)[src];
}

// hd == 256: 8 dims per lane
__global__ void __launch_bounds__(1024)
sdpa_decode_kernel(const bf16_t* __restrict__ q, const bf16_t* __restrict__ kc,
                   const bf16_t* __restrict__ vc, int T, int Hq, int Hkv, int cap,
                   const int* dev_offset, int offset_add, float scale, bf16_t* __restrict__ out, int Tb) {
  constexpr int HD = 256;
  __shared__ float s_o[32][HD];
  __shared__ float s_max[32], s_sum[32], s_f[32];
  const int h = blockIdx.x, r = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kvh = h / (Hq / Hkv);
  const int seq = Tb > 0 ? r / Tb : 0, tl = Tb > 0 ? r - seq * Tb : r;  // Tb > 0: a cache and a position per sequence
  const int offset = (dev_offset ? dev_offset[seq] : 0) + offset_add;
  kc += (int64_t)seq * Hkv * cap * HD;
  vc += (int64_t)seq * Hkv * cap * HD;
  int L = offset + tl + 1;
  if (L > cap) L = cap;
  float qs[8], o[8];
  {
    float qf[8];
    widen8(ldg128(q + ((int64_t)r * Hq + h) * HD + 8 * lane), qf);
#pragma unroll
    for (int i = 0; i < 8; ++i) { qs[i] = qf[i] * scale; o[i] = 0.f; }
  }
  float mx = -INFINITY, sm = 0.f;
  for (int n = warp; n < L; n += 32) {
    const int64_t rowoff = ((int64_t)kvh * cap + n) * HD + 8 * lane;
    float kf[8], vf[8];
    widen8(ldg128(kc + rowoff), kf);
    widen8(ldg128(vc + rowoff), vf);
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
    out[((int64_t)r * Hq + h) * HD + d] = f2bf(a[0] / s_sum[0]);
  }
}
}  // namespace

int k_rope(orn_ctx* ctx, cudaStream_t s, bf16_t* x, int T, int H, int hd, int dims, float lnb,
           const int* dev_offset, int offset_add) {
  int n = T * H * (dims / 2);
  rope_kernel<<<(n + 127) / 128, 128, 0, s>>>(x, T, H, hd, dims, lnb, dev_offset, offset_add, 0);
  return orn_launch_check(ctx, "rope");
}

int k_kv_append(orn_ctx* ctx, cudaStream_t s, const bf16_t* k, const bf16_t* v, int T, int Hkv,
                int hd, int cap, const int* dev_offset, int offset_add, bf16_t* kc, bf16_t* vc) {
  int n = T * Hkv * (hd / 8);
  kv_append_kernel<<<(n + 127) / 128, 128, 0, s>>>(k, v, T, Hkv, hd, cap, dev_offset, offset_add, kc, vc, 0);
  return orn_launch_check(ctx, "kv_append");
}

int k_sdpa_decode(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* kc,
                  const bf16_t* vc, int T, int Hq, int Hkv, int hd, int cap, const int* dev_offset,
                  int offset_add, float scale, bf16_t* out) {
  if (hd != 256) ORN_FAIL(ctx, ORN_ERR_ARG, "sdpa_decode: head_dim must be 256");
  if (Hq % Hkv != 0) ORN_FAIL(ctx, ORN_ERR_ARG, "sdpa_decode: Hq % Hkv != 0");
  dim3 grid(Hq, T);
  sdpa_decode_kernel<<<grid, 1024, 0, s>>>(q, kc, vc, T, Hq, Hkv, cap, dev_offset, offset_add, scale, out, 0);
  return orn_launch_check(ctx, "sdpa_decode");
}

// ---- the same three ops over B sequences at once: rows are sequence-major ([B][Tb] windows), every
// sequence has its own position pos[b] and its own caches [Hkv, cap, hd] laid end to end
int k_rope_batched(orn_ctx* ctx, cudaStream_t s, bf16_t* x, int B, int Tb, int H, int hd, int dims, float lnb, const int* pos) {
  const int n = B * Tb * H * (dims / 2);
  rope_kernel<<<(n + 127) / 128, 128, 0, s>>>(x, B * Tb, H, hd, dims, lnb, pos, 0, Tb);
  return orn_launch_check(ctx, "rope");
}
int k_kv_append_batched(orn_ctx* ctx, cudaStream_t s, const bf16_t* k, const bf16_t* v, int B, int Tb, int Hkv, int hd, int cap,
                        const int* pos, bf16_t* kc, bf16_t* vc) {
  const int n = B * Tb * Hkv * (hd / 8);
  kv_append_kernel<<<(n + 127) / 128, 128, 0, s>>>(k, v, B * Tb, Hkv, hd, cap, pos, 0, kc, vc, Tb);
  return orn_launch_check(ctx, "kv_append");
}
int k_sdpa_decode_batched(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* kc, const bf16_t* vc, int B, int Tb,
                          int Hq, int Hkv, int hd, int cap, const int* pos, float scale, bf16_t* out) {
  if (hd != 256) ORN_FAIL(ctx, ORN_ERR_ARG, "sdpa_decode: head_dim must be 256");
  dim3 grid(Hq, B * Tb);
  sdpa_decode_kernel<<<grid, 1024, 0, s>>>(q, kc, vc, B * Tb, Hq, Hkv, cap, pos, 0, scale, out, Tb);
  return orn_launch_check(ctx, "sdpa_decode");
}
