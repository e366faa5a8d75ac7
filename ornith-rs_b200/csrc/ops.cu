// Norms, elementwise ops and the MoE router/combine kernels of the decode path.
//
// Replaces kernels/ornith_norm.metal, the rms kernels of
// kernels/mlx/.../rms_norm.metal, kernels/ornith_elementwise.metal,
// kernels/mlx/.../softmax.h and the router_top_k / moe_combine kernels of
// kernels/moe.metal, as dispatched by src/ops/norm.rs, elementwise.rs,
// softmax.rs and moe.rs.  All of them are a few KB per call; what matters is
// that their rounding points and reduction orders are fixed (see
// orn_common.cuh), not their bandwidth.
#include "orn_internal.h"

namespace {

// Sum over the block in the order: thread partials -> warp butterfly -> the
// warp sums, zero padded to 32, butterfly again.  `red` is 32 floats of shared
// memory.  Every thread returns the total.
ORN_D float block_sum_ordered(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (threadIdx.x < 32) red[threadIdx.x] = 0.f;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = warp_sum(red[lane]);
  return t;
}
ORN_D float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (threadIdx.x < 32) red[threadIdx.x] = -INFINITY;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  return warp_max(red[lane]);
}

// MODE 0: rms_norm, 1: add + rms_norm (stores h), 2: gated
template <int MODE>
__global__ void rms_kernel(const bf16_t* __restrict__ a, const bf16_t* __restrict__ b,
                           const bf16_t* __restrict__ w, const bf16_t* __restrict__ z, int n,
                           float eps, bf16_t* __restrict__ h, bf16_t* __restrict__ out) {
  __shared__ float red[32];
  const int64_t base = (int64_t)blockIdx.x * n;
  const int i0 = threadIdx.x * 4;
  float xv[4];
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int idx = i0 + i;
    float v = 0.f;
    if (idx < n) {
      v = bf2f(a[base + idx]);
      if (MODE == 1) {
        v = bfr(v + bf2f(b[base + idx]));
        h[base + idx] = f2bf(v);
      }
      acc = fmaf(v, v, acc);
    }
    xv[i] = v;
  }
  float total = block_sum_ordered(acc, red);
  float inv = orn_rsqrtf(total / (float)n + eps);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int idx = i0 + i;
    if (idx < n) {
      float v = bfr(xv[i] * inv);
      if (w != nullptr) v = bfr(bf2f(w[idx]) * v);
      if (MODE == 2) {
        float g = bf2f(z[base + idx]);
        g = g * orn_sigmoid_f32(g);
        v = bfr(g * v);
      }
      out[base + idx] = f2bf(v);
    }
  }
}

__global__ void sigmoid_gate_kernel(const bf16_t* gate, const bf16_t* x, int n, int inner, bf16_t* out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = f2bf(orn_sigmoid_bf(bf2f(gate[i / inner])) * bf2f(x[i]));
}
__global__ void swiglu_kernel(const bf16_t* g, const bf16_t* u, int n, bf16_t* out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = f2bf(orn_swiglu_bf(bf2f(g[i]), bf2f(u[i])));
}
__global__ void add_kernel(const bf16_t* a, const bf16_t* b, int n, bf16_t* out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = f2bf(bf2f(a[i]) + bf2f(b[i]));
}

// mlx softmax.h:10-99, float accumulate; thread t owns 4 consecutive entries
__global__ void softmax_kernel(const bf16_t* __restrict__ x, int n, bf16_t* __restrict__ out) {
  __shared__ float red[32];
  const int64_t base = (int64_t)blockIdx.x * n;
  const int i0 = threadIdx.x * 4;
  float v[4];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] = (i0 + i < n) ? bf2f(x[base + i0 + i]) : -INFINITY;
    m = fmaxf(m, v[i]);
  }
  m = block_max(m, red);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (i0 + i < n) {
      v[i] = orn_expf(v[i] - m);
      acc = acc + v[i];
    }
  float total = block_sum_ordered(acc, red);
  float inv = 1.0f / total;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (i0 + i < n) out[base + i0 + i] = f2bf(v[i] * inv);
}

// kernels/moe.metal:568-614: one warp per row, lane l holds experts l, l+32, ...
constexpr int kRouterMaxPerLane = 16;
__global__ void router_topk_kernel(const bf16_t* __restrict__ gates, int n, int k,
                                   uint32_t* __restrict__ inds, bf16_t* __restrict__ scores) {
  const int row = blockIdx.x, lane = threadIdx.x;
  const bf16_t* g = gates + (int64_t)row * n;
  float v[kRouterMaxPerLane];
  int held = 0;
#pragma unroll
  for (int s = 0; s < kRouterMaxPerLane; ++s) {
    int i = lane + 32 * s;
    v[s] = -INFINITY;
    if (i < n) { v[s] = bf2f(g[i]); held = s + 1; }
  }
  for (int r = 0; r < k; ++r) {
    float best = -INFINITY;
    uint32_t besti = 0;
#pragma unroll
    for (int s = 0; s < kRouterMaxPerLane; ++s) {
      uint32_t i = lane + 32 * s;
      if (s < held && (v[s] > best || (v[s] == best && i > besti))) { best = v[s]; besti = i; }
    }
    float m = warp_max(best);
    uint32_t mi = warp_max_u32(best == m ? besti + 1 : 0u) - 1;
#pragma unroll
    for (int s = 0; s < kRouterMaxPerLane; ++s)
      if ((mi & 31) == (uint32_t)lane && (mi >> 5) == (uint32_t)s) v[s] = -INFINITY;
    if (lane == 0) {
      int slot = row * k + (k - 1 - r);
      inds[slot] = mi;
      scores[slot] = g[mi];
    }
  }
}

// softmax_kernel and router_topk_kernel in one launch (the decode batch's router): the bfloat16
// probabilities stay in shared memory, warp 0 then selects from them.  Same arithmetic, same bits.
__global__ void softmax_topk_kernel(const bf16_t* __restrict__ x, int n, int k, uint32_t* __restrict__ inds,
                                    bf16_t* __restrict__ scores) {
  __shared__ float red[32];
  __shared__ float probs[32 * kRouterMaxPerLane];
  const int row = blockIdx.x;
  const int64_t base = (int64_t)row * n;
  const int i0 = threadIdx.x * 4;
  float v[4];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] = (i0 + i < n) ? bf2f(x[base + i0 + i]) : -INFINITY;
    m = fmaxf(m, v[i]);
  }
  m = block_max(m, red);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (i0 + i < n) {
      v[i] = orn_expf(v[i] - m);
      acc = acc + v[i];
    }
  const float total = block_sum_ordered(acc, red);
  const float inv = 1.0f / total;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (i0 + i < n) probs[i0 + i] = bfr(v[i] * inv);
  __syncthreads();
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  float pv[kRouterMaxPerLane];
  int held = 0;
#pragma unroll
  for (int s = 0; s < kRouterMaxPerLane; ++s) {
    const int i = lane + 32 * s;
    pv[s] = -INFINITY;
    if (i < n) { pv[s] = probs[i]; held = s + 1; }
  }
  for (int r = 0; r < k; ++r) {
    float best = -INFINITY;
    uint32_t besti = 0;
#pragma unroll
    for (int s = 0; s < kRouterMaxPerLane; ++s) {
      const uint32_t i = lane + 32 * s;
      if (s < held && (pv[s] > best || (pv[s] == best && i > besti))) { best = pv[s]; besti = i; }
    }
    const float mm = warp_max(best);
    const uint32_t mi = warp_max_u32(best == mm ? besti + 1 : 0u) - 1;
#pragma unroll
    for (int s = 0; s < kRouterMaxPerLane; ++s)
      if ((mi & 31) == (uint32_t)lane && (mi >> 5) == (uint32_t)s) pv[s] = -INFINITY;
    if (lane == 0) {
      const int slot = row * k + (k - 1 - r);
      inds[slot] = mi;
      scores[slot] = f2bf(probs[mi]);
    }
  }
}

// two SwiGLU jobs in one launch: n1 elements of (g1, u1) and *n2_rows x width2 elements of (g2, u2)
__global__ void swiglu2_kernel(const bf16_t* g1, const bf16_t* u1, size_t n1, bf16_t* out1, const bf16_t* g2, const bf16_t* u2,
                               const int* n2_rows, int width2, bf16_t* out2) {
  const size_t n2 = (size_t)(*n2_rows) * width2;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n1 + n2; i += (size_t)gridDim.x * blockDim.x) {
    if (i < n1) out1[i] = f2bf(orn_swiglu_bf(bf2f(g1[i]), bf2f(u1[i])));
    else out2[i - n1] = f2bf(orn_swiglu_bf(bf2f(g2[i - n1]), bf2f(u2[i - n1])));
  }
}

// kernels/moe.metal:207-244: bfloat16 arithmetic, ascending j
__global__ void moe_combine_kernel(const bf16_t* __restrict__ scores, const bf16_t* __restrict__ y,
                                   const bf16_t* __restrict__ gate, const bf16_t* __restrict__ shared,
                                   int k, int dim, int normalize, bf16_t* __restrict__ out) {
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= dim) return;
  const bf16_t* s = scores + (int64_t)t * k;
  float denom = 0.f;
  if (normalize)
    for (int j = 0; j < k; ++j) denom = bfr(bf2f(s[j]) + denom);
  float acc = 0.f;
  for (int j = 0; j < k; ++j) {
    float w = normalize ? bfr(bf2f(s[j]) / denom) : bf2f(s[j]);
    float weighted = bfr(bf2f(y[((int64_t)t * k + j) * dim + c]) * w);
    acc = bfr(weighted + acc);
  }
  float g = orn_sigmoid_bf(bf2f(gate[t]));
  float gated = bfr(g * bf2f(shared[(int64_t)t * dim + c]));
  out[(int64_t)t * dim + c] = f2bf(acc + gated);
}

// the same arithmetic per element, eight columns per thread (16-byte loads) for many rows
__global__ void __launch_bounds__(128) moe_combine_wide_kernel(const bf16_t* __restrict__ scores, const bf16_t* __restrict__ y,
                                                                const bf16_t* __restrict__ gate, const bf16_t* __restrict__ shared,
                                                                int k, int dim, int normalize, bf16_t* __restrict__ out) {
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= dim) return;
  const bf16_t* s = scores + (int64_t)t * k;
  float denom = 0.f;
  if (normalize)
    for (int j = 0; j < k; ++j) denom = bfr(bf2f(s[j]) + denom);
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int j = 0; j < k; ++j) {
    const float w = normalize ? bfr(bf2f(s[j]) / denom) : bf2f(s[j]);
    const uint4 v = ldg128(y + ((int64_t)t * k + j) * dim + c);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      acc[2 * e] = bfr(bfr(__uint_as_float(u[e] << 16) * w) + acc[2 * e]);
      acc[2 * e + 1] = bfr(bfr(__uint_as_float(u[e] & 0xffff0000u) * w) + acc[2 * e + 1]);
    }
  }
  const float g = orn_sigmoid_bf(bf2f(gate[t]));
  const uint4 sh = ldg128(shared + (int64_t)t * dim + c);
  const uint32_t su[4] = {sh.x, sh.y, sh.z, sh.w};
  uint32_t o[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float lo = acc[2 * e] + bfr(g * __uint_as_float(su[e] << 16));
    const float hi = acc[2 * e + 1] + bfr(g * __uint_as_float(su[e] & 0xffff0000u));
    o[e] = (uint32_t)f2bf(lo) | ((uint32_t)f2bf(hi) << 16);
  }
  *reinterpret_cast<uint4*>(out + (int64_t)t * dim + c) = make_uint4(o[0], o[1], o[2], o[3]);
}

// q_proj output [T, Hq, 2*hd] -> queries [T,Hq,hd], gate [T,Hq,hd]
// (qwen3_5.rs:441-443 slice_inner x2)
__global__ void split_qgate_kernel(const bf16_t* qg, int n /*T*Hq*/, int hd, bf16_t* q, bf16_t* gate) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * hd) return;
  int r = i / hd, d = i - r * hd;
  q[i] = qg[(int64_t)r * 2 * hd + d];
  gate[i] = qg[(int64_t)r * 2 * hd + hd + d];
}
// concat_inner (mtp.rs:186): out[t] = [a[t], b[t]]
__global__ void concat2_kernel(const bf16_t* a, const bf16_t* b, int T, int n, bf16_t* out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * 2 * n) return;
  int t = i / (2 * n), d = i - t * 2 * n;
  out[i] = d < n ? a[(int64_t)t * n + d] : b[(int64_t)t * n + d - n];
}

int norm_threads(int n) {
  int t = (n + 3) / 4;
  return ((t + 31) / 32) * 32;
}
}  // namespace

int k_rms_norm(orn_ctx* ctx, cudaStream_t s, const bf16_t* x, const bf16_t* w, int rows, int n,
               float eps, bf16_t* out) {
  if (n > 4096) ORN_FAIL(ctx, ORN_ERR_ARG, "rms_norm: n > 4096");
  rms_kernel<0><<<rows, norm_threads(n), 0, s>>>(x, nullptr, w, nullptr, n, eps, nullptr, out);
  return orn_launch_check(ctx, "rms_norm");
}
int k_add_rms_norm(orn_ctx* ctx, cudaStream_t s, const bf16_t* a, const bf16_t* b, const bf16_t* w,
                   int rows, int n, float eps, bf16_t* h, bf16_t* out) {
  if (n > 4096) ORN_FAIL(ctx, ORN_ERR_ARG, "add_rms_norm: n > 4096");
  rms_kernel<1><<<rows, norm_threads(n), 0, s>>>(a, b, w, nullptr, n, eps, h, out);
  return orn_launch_check(ctx, "add_rms_norm");
}
int k_rms_norm_gated(orn_ctx* ctx, cudaStream_t s, const bf16_t* x, const bf16_t* w,
                     const bf16_t* z, int rows, int n, float eps, bf16_t* out) {
  if (n > 4096) ORN_FAIL(ctx, ORN_ERR_ARG, "rms_norm_gated: n > 4096");
  rms_kernel<2><<<rows, norm_threads(n), 0, s>>>(x, nullptr, w, z, n, eps, nullptr, out);
  return orn_launch_check(ctx, "rms_norm_gated");
}
int k_sigmoid_gate(orn_ctx* ctx, cudaStream_t s, const bf16_t* gate, const bf16_t* x, int n,
                   int inner, bf16_t* out) {
  sigmoid_gate_kernel<<<(n + 255) / 256, 256, 0, s>>>(gate, x, n, inner, out);
  return orn_launch_check(ctx, "sigmoid_gate");
}
int k_swiglu(orn_ctx* ctx, cudaStream_t s, const bf16_t* g, const bf16_t* u, int n, bf16_t* out) {
  swiglu_kernel<<<(n + 255) / 256, 256, 0, s>>>(g, u, n, out);
  return orn_launch_check(ctx, "swiglu");
}
int k_add(orn_ctx* ctx, cudaStream_t s, const bf16_t* a, const bf16_t* b, int n, bf16_t* out) {
  add_kernel<<<(n + 255) / 256, 256, 0, s>>>(a, b, n, out);
  return orn_launch_check(ctx, "add");
}
int k_softmax_precise(orn_ctx* ctx, cudaStream_t s, const bf16_t* x, int rows, int n, bf16_t* out) {
  if (n > 4096) ORN_FAIL(ctx, ORN_ERR_ARG, "softmax: n > 4096");
  softmax_kernel<<<rows, norm_threads(n), 0, s>>>(x, n, out);
  return orn_launch_check(ctx, "softmax");
}
int k_router_topk(orn_ctx* ctx, cudaStream_t s, const bf16_t* gates, int rows, int n, int k,
                  uint32_t* inds, bf16_t* scores) {
  if (n > 32 * kRouterMaxPerLane || k > n) ORN_FAIL(ctx, ORN_ERR_ARG, "router_topk: n > 512 or k > n");
  router_topk_kernel<<<rows, 32, 0, s>>>(gates, n, k, inds, scores);
  return orn_launch_check(ctx, "router_topk");
}
int k_softmax_topk(orn_ctx* ctx, cudaStream_t s, const bf16_t* x, int rows, int n, int k, uint32_t* inds, bf16_t* scores) {
  if (n > 32 * kRouterMaxPerLane || k > n) ORN_FAIL(ctx, ORN_ERR_ARG, "softmax_topk: n > 512 or k > n");
  softmax_topk_kernel<<<rows, norm_threads(n), 0, s>>>(x, n, k, inds, scores);
  return orn_launch_check(ctx, "softmax_topk");
}
int k_swiglu2(orn_ctx* ctx, cudaStream_t s, const bf16_t* g1, const bf16_t* u1, size_t n1, bf16_t* out1, const bf16_t* g2,
              const bf16_t* u2, const int* n2_rows, int width2, bf16_t* out2) {
  swiglu2_kernel<<<ctx->sm_count * 4, 256, 0, s>>>(g1, u1, n1, out1, g2, u2, n2_rows, width2, out2);
  return orn_launch_check(ctx, "swiglu2");
}
int k_moe_combine(orn_ctx* ctx, cudaStream_t s, const bf16_t* scores, const bf16_t* y,
                  const bf16_t* gate, const bf16_t* shared, int T, int k, int dim, int normalize,
                  bf16_t* out) {
  const bool aligned = dim % 8 == 0 && ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(shared) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (T >= 16 && aligned) {
    dim3 wgrid((dim / 8 + 127) / 128, T);
    moe_combine_wide_kernel<<<wgrid, 128, 0, s>>>(scores, y, gate, shared, k, dim, normalize, out);
    return orn_launch_check(ctx, "moe_combine");
  }
  dim3 grid((dim + 255) / 256, T);
  moe_combine_kernel<<<grid, 256, 0, s>>>(scores, y, gate, shared, k, dim, normalize, out);
  return orn_launch_check(ctx, "moe_combine");
}
int k_split_qgate(orn_ctx* ctx, cudaStream_t s, const bf16_t* qg, int T, int Hq, int hd, bf16_t* q,
                  bf16_t* gate) {
  int n = T * Hq;
  split_qgate_kernel<<<(n * hd + 255) / 256, 256, 0, s>>>(qg, n, hd, q, gate);
  return orn_launch_check(ctx, "split_qgate");
}
int k_concat2(orn_ctx* ctx, cudaStream_t s, const bf16_t* a, const bf16_t* b, int T, int n,
              bf16_t* out) {
  concat2_kernel<<<(T * 2 * n + 255) / 256, 256, 0, s>>>(a, b, T, n, out);
  return orn_launch_check(ctx, "concat2");
}
