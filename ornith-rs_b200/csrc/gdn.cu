// Gated-delta (linear attention) kernels: the fused front end and the fp32
// recurrent delta rule.
//
// Replaces kernels/gdn_front.metal:65-190 (conv window + depthwise causal
// conv k=4 + SiLU + q/k RMS norm and scale + beta + decay gate) and
// kernels/gated_delta.metal:36-142 (gated_delta_step_packed_btree), as
// dispatched by src/ops/gdn.rs:191-413.
//
// Recurrence layout: the state of one value head is [Dv=128][Dk=128] fp32
// (64 KB).  Value rows are independent, so the work is cut by (head, 16-row
// slice): a CTA of 64 threads holds a 16 x 128 slice entirely in registers
// (4 lanes per row, 32 consecutive state floats per lane, read and written as
// 128-bit accesses that cover whole 512-byte rows).  Every state element is
// read once and written once per token: the kernel moves exactly the
// algorithmic bytes.  The dot products use the reference's tree: eight chains
// of four fmas per lane, pairwise fold, then xor-1 and xor-2 across the four
// lanes of a row.
#include "orn_internal.h"

namespace {

ORN_D float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
ORN_D float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

struct FrontParams {
  const bf16_t* conv_state;  // [S, D]
  const bf16_t* qkv;         // [T, D]
  const bf16_t* cw;          // [D, Kc]
  const bf16_t* a_in;        // [T, Hv]
  const bf16_t* b_in;        // [T, Hv]
  const bf16_t* a_log;       // [Hv]
  const bf16_t* dt_bias;     // [Hv]
  bf16_t* conv_next;         // [S, D] or null
  bf16_t* conv_input;        // [S+T, D] or null
  bf16_t* q;                 // [T, Hk, Dh]
  bf16_t* k;                 // [T, Hk, Dh]
  bf16_t* v;                 // [T, Hv, Dh]
  bf16_t* beta;              // [T, Hv]
  float* g;                  // [T, Hv]
  int T, S, Kc, D, Dh, Hk, Hv;
  float q_scale, k_scale, eps;
  int Tb;         // > 0: the T rows are Tb-row windows of T / Tb sequences ...
  int64_t seq_stride;  // ... whose conv buffers [S + Tcap, D] lie seq_stride elements apart (qkv = rows S.. of each)
};

// one warp per (token, 128-channel head slot); lane owns 4 channels
__global__ void gdn_front_kernel(FrontParams p) {
  const int lane = threadIdx.x & 31;
  const int slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int t = blockIdx.y;
  const int slots = p.D / p.Dh;
  if (slot >= slots) return;
  const int c0 = slot * p.Dh + lane * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int seq = p.Tb > 0 ? t / p.Tb : 0, tl = p.Tb > 0 ? t - seq * p.Tb : t;
  const bf16_t* cs = p.conv_state + seq * p.seq_stride;
  const bf16_t* qk = p.qkv + seq * p.seq_stride;
  for (int i = 0; i < p.Kc; ++i) {
    const int j = tl + i;
    const bf16_t* src = (j < p.S) ? (cs + (int64_t)j * p.D) : (qk + (int64_t)(j - p.S) * p.D);
    uint2 xv = *reinterpret_cast<const uint2*>(src + c0);
    float xs[4] = {bf_lo(xv.x), bf_hi(xv.x), bf_lo(xv.y), bf_hi(xv.y)};
#pragma unroll
    for (int r = 0; r < 4; ++r) acc[r] = fmaf(xs[r], bf2f(p.cw[(int64_t)(c0 + r) * p.Kc + i]), acc[r]);
  }
  float y[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) y[r] = orn_silu_bf(bfr(acc[r]));

  if (t + 1 == p.T && p.conv_next != nullptr) {
    for (int j = 0; j < p.S; ++j) {
      const int row = p.T + j;
      const bf16_t* src = (row < p.S) ? (p.conv_state + (int64_t)row * p.D)
                                      : (p.qkv + (int64_t)(row - p.S) * p.D);
      *reinterpret_cast<uint2*>(p.conv_next + (int64_t)j * p.D + c0) =
          *reinterpret_cast<const uint2*>(src + c0);
    }
  }
  if (p.conv_input != nullptr) {
    *reinterpret_cast<uint2*>(p.conv_input + (int64_t)(p.S + t) * p.D + c0) =
        *reinterpret_cast<const uint2*>(p.qkv + (int64_t)t * p.D + c0);
    if (t == 0)
      for (int j = 0; j < p.S; ++j)
        *reinterpret_cast<uint2*>(p.conv_input + (int64_t)j * p.D + c0) =
            *reinterpret_cast<const uint2*>(p.conv_state + (int64_t)j * p.D + c0);
  }

  const int key_dim = p.Hk * p.Dh;
  if (slot < 2 * p.Hk) {
    float sum = 0.f;
#pragma unroll
    for (int r = 0; r < 4; ++r) sum = fmaf(y[r], y[r], sum);
    sum = warp_sum(sum);
    const float inv = orn_rsqrtf(sum / (float)p.Dh + p.eps);
    const bool is_q = slot < p.Hk;
    bf16_t* dst = (is_q ? p.q : p.k) + (int64_t)t * key_dim + (is_q ? c0 : c0 - key_dim);
    const float sc = is_q ? p.q_scale : p.k_scale;
#pragma unroll
    for (int r = 0; r < 4; ++r) dst[r] = f2bf(sc * bfr(y[r] * inv));
  } else {
    bf16_t* dst = p.v + (int64_t)t * (p.D - 2 * key_dim) + (c0 - 2 * key_dim);
#pragma unroll
    for (int r = 0; r < 4; ++r) dst[r] = f2bf(y[r]);
  }

  if (slot == 0) {
    for (int h = lane; h < p.Hv; h += 32) {
      const int64_t i = (int64_t)t * p.Hv + h;
      float sp = orn_softplus_bf(bfr(bf2f(p.a_in[i]) + bf2f(p.dt_bias[h])));
      float decay = orn_expf(bf2f(p.a_log[h]));
      p.g[i] = orn_expf((-decay) * sp);
      p.beta[i] = f2bf(orn_sigmoid_bf(bf2f(p.b_in[i])));
    }
  }
}

struct DeltaParams {
  const bf16_t* q;     // [T, Hk, 128]
  const bf16_t* k;     // [T, Hk, 128]
  const bf16_t* v;     // [T, Hv, 128]
  const float* g;      // [T, Hv]
  const bf16_t* beta;  // [T, Hv]
  float* state;        // in-place mode: [Hv,128,128]
  float* snaps;        // in-place mode: [T][Hv,128,128] or null
  float* ring;         // ring mode: [nring][Hv,128,128]; in = ring[cur%nring], out_t = ring[(cur+1+t)%nring]
  const int* cur;      // ring mode selector (device)
  int nring;           // ring mode: number of state buffers
  int ring_final;      // ring mode: only the state after the last token is kept, in ring[(cur+1)%nring]
  bf16_t* y;           // [T, Hv, 128]
  int T, Hk, Hv;
  int batched;         // ring mode over sequences: blockIdx.z = sequence, a ring and a cursor per sequence, T rows each
};

constexpr int kRowsPerCta = 16;

// 32 bytes per request: a thread's 32 state floats are one 128-byte line, which four requests of a whole
// sector each move instead of eight half sectors
ORN_D void ld256(const float* p, float* v) {
  asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
               : "l"(p));
}
ORN_D void st256(float* p, const float* v) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]),
               "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}

__global__ void __launch_bounds__(kRowsPerCta * 4) gated_delta_kernel(DeltaParams p) {
  const int hv = blockIdx.y;
  const int hk = hv / (p.Hv / p.Hk);
  const int row = blockIdx.x * kRowsPerCta + (threadIdx.x >> 2);
  const int lir = threadIdx.x & 3;  // lane in row
  const size_t ssz = (size_t)p.Hv * 128 * 128;
  const size_t off = ((size_t)hv * 128 + row) * 128 + lir * 32;
  const float* sin;
  int cur = 0;
  if (p.batched) {  // this sequence's rows, ring and cursor
    const size_t z = blockIdx.z;
    p.q += z * p.T * p.Hk * 128; p.k += z * p.T * p.Hk * 128; p.v += z * p.T * p.Hv * 128;
    p.g += z * p.T * p.Hv; p.beta += z * p.T * p.Hv; p.y += z * p.T * p.Hv * 128;
    p.ring += z * p.nring * ssz; p.cur += z;
  }
  if (p.ring != nullptr) {
    cur = *p.cur;
    sin = p.ring + (size_t)(cur % p.nring) * ssz + off;
  } else {
    sin = p.state + off;
  }
  float S[32];
#pragma unroll
  for (int i = 0; i < 4; ++i) ld256(sin + 8 * i, S + 8 * i);
  // the inputs of step t + 1 are requested before step t's arithmetic: a long window (a prompt
  // chunk) otherwise pays one memory round trip per token on top of the recurrence's own chain
  struct StepIn {
    uint4 kv[4], qv[4];
    float g;
    bf16_t beta, v;
  };
  auto fetch = [&](int t, StepIn& in) {
    const bf16_t* kp = p.k + ((size_t)t * p.Hk + hk) * 128 + lir * 32;
    const bf16_t* qp = p.q + ((size_t)t * p.Hk + hk) * 128 + lir * 32;
#pragma unroll
    for (int i = 0; i < 4; ++i) { in.kv[i] = ldg128(kp + 8 * i); in.qv[i] = ldg128(qp + 8 * i); }
    in.g = p.g[(size_t)t * p.Hv + hv];
    in.beta = p.beta[(size_t)t * p.Hv + hv];
    in.v = p.v[((size_t)t * p.Hv + hv) * 128 + row];
  };
  StepIn now, nxt;
  fetch(0, now);
  for (int t = 0; t < p.T; ++t) {
    if (t + 1 < p.T) fetch(t + 1, nxt);
    float kf[32], qf[32];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 kv = now.kv[i], qv = now.qv[i];
      kf[8 * i] = bf_lo(kv.x); kf[8 * i + 1] = bf_hi(kv.x); kf[8 * i + 2] = bf_lo(kv.y); kf[8 * i + 3] = bf_hi(kv.y);
      kf[8 * i + 4] = bf_lo(kv.z); kf[8 * i + 5] = bf_hi(kv.z); kf[8 * i + 6] = bf_lo(kv.w); kf[8 * i + 7] = bf_hi(kv.w);
      qf[8 * i] = bf_lo(qv.x); qf[8 * i + 1] = bf_hi(qv.x); qf[8 * i + 2] = bf_lo(qv.y); qf[8 * i + 3] = bf_hi(qv.y);
      qf[8 * i + 4] = bf_lo(qv.z); qf[8 * i + 5] = bf_hi(qv.z); qf[8 * i + 6] = bf_lo(qv.w); qf[8 * i + 7] = bf_hi(qv.w);
    }
    const float gt = now.g;
    const float bt = bf2f(now.beta);
    const float vt = bf2f(now.v);
    now = nxt;
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
    if (p.ring != nullptr) {
      if (!p.ring_final) sout = p.ring + (size_t)((cur + 1 + t) % p.nring) * ssz + off;
      else if (t + 1 == p.T) sout = p.ring + (size_t)((cur + 1) % p.nring) * ssz + off;
    }
    else if (p.snaps != nullptr) sout = p.snaps + (size_t)t * ssz + off;
    else if (t + 1 == p.T) sout = p.state + off;
    if (sout != nullptr) {
#pragma unroll
      for (int i = 0; i < 4; ++i) st256(sout + 8 * i, S + 8 * i);
    }
    if (p.ring == nullptr && p.snaps != nullptr && t + 1 == p.T) {
      float* so = p.state + off;
#pragma unroll
      for (int i = 0; i < 4; ++i) st256(so + 8 * i, S + 8 * i);
    }
  }
}
}  // namespace

int k_gdn_front(orn_ctx* ctx, cudaStream_t s, const bf16_t* conv_state, const bf16_t* qkv,
                const bf16_t* cw, const bf16_t* a, const bf16_t* b, const bf16_t* a_log,
                const bf16_t* dt_bias, int T, int Hk, int Hv, int Dh, int Kc, float eps,
                bf16_t* conv_next, bf16_t* q, bf16_t* k, bf16_t* v, bf16_t* beta, float* g,
                bf16_t* conv_input_keep) {
  if (Dh != 128) ORN_FAIL(ctx, ORN_ERR_ARG, "gdn_front: head dim must be 128");
  if (conv_next == conv_state) ORN_FAIL(ctx, ORN_ERR_ARG, "gdn_front: conv_next must not alias conv_state");
  FrontParams p;
  p.conv_state = conv_state; p.qkv = qkv; p.cw = cw; p.a_in = a; p.b_in = b; p.a_log = a_log;
  p.dt_bias = dt_bias; p.conv_next = conv_next; p.conv_input = conv_input_keep;
  p.q = q; p.k = k; p.v = v; p.beta = beta; p.g = g;
  p.T = T; p.S = Kc - 1; p.Kc = Kc; p.D = 2 * Hk * Dh + Hv * Dh; p.Dh = Dh; p.Hk = Hk; p.Hv = Hv;
  p.Tb = 0; p.seq_stride = 0;
  // powf(dk, -0.5) and its square, cast to bfloat16 (qwen3_5.rs:506,524-525)
  float inv_scale = 1.0f / sqrtf((float)Dh);
  p.q_scale = bfr(inv_scale * inv_scale);
  p.k_scale = bfr(inv_scale);
  p.eps = eps;
  int slots = p.D / Dh;
  dim3 grid((slots + 3) / 4, T);
  gdn_front_kernel<<<grid, 128, 0, s>>>(p);
  return orn_launch_check(ctx, "gdn_front");
}

static int launch_delta(orn_ctx* ctx, cudaStream_t s, DeltaParams& p, int B = 1) {
  if (p.Hv % p.Hk != 0) ORN_FAIL(ctx, ORN_ERR_ARG, "gated_delta: Hv % Hk != 0");
  dim3 grid(128 / kRowsPerCta, p.Hv, B);
  gated_delta_kernel<<<grid, kRowsPerCta * 4, 0, s>>>(p);
  return orn_launch_check(ctx, "gated_delta");
}

int k_gated_delta(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* k, const bf16_t* v,
                  const float* g, const bf16_t* beta, float* state, int T, int Hk, int Hv,
                  bf16_t* y, float* snaps) {
  DeltaParams p;
  p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta; p.state = state; p.snaps = snaps;
  p.ring = nullptr; p.cur = nullptr; p.nring = 1; p.ring_final = 0; p.y = y; p.T = T; p.Hk = Hk; p.Hv = Hv;
  p.batched = 0;
  return launch_delta(ctx, s, p);
}

// ring mode for the model: nring state buffers per layer, selected by a device
// counter so that accepting `keep` tokens is `cur += keep` and never a copy
int k_gated_delta_ring(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* k,
                       const bf16_t* v, const float* g, const bf16_t* beta, float* ring,
                       int nring, const int* cur, int final_only, int T, int Hk, int Hv,
                       bf16_t* y) {
  if (T + 1 > nring && !final_only) ORN_FAIL(ctx, ORN_ERR_ARG, "gated_delta ring mode: window wider than the ring");
  DeltaParams p;
  p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta; p.state = nullptr; p.snaps = nullptr;
  p.ring = ring; p.cur = cur; p.nring = nring; p.ring_final = final_only; p.y = y; p.T = T; p.Hk = Hk; p.Hv = Hv;
  p.batched = 0;
  return launch_delta(ctx, s, p);
}

// ---- B sequences at once: rows sequence-major ([B][Tb] windows); conv buffers [B][S + Tcap, D] with the
// window's qkv rows already in place behind each sequence's S cached rows; state rings [B][nring][Hv,128,128]
// with one cursor per sequence, the state after window row t written to slot (cur + 1 + t) % nring
int k_gdn_front_batched(orn_ctx* ctx, cudaStream_t s, const bf16_t* conv, int64_t seq_stride, const bf16_t* cw,
                        const bf16_t* a, const bf16_t* b, const bf16_t* a_log, const bf16_t* dt_bias, int B, int Tb, int Hk,
                        int Hv, int Dh, int Kc, float eps, bf16_t* q, bf16_t* k, bf16_t* v, bf16_t* beta, float* g) {
  if (Dh != 128) ORN_FAIL(ctx, ORN_ERR_ARG, "gdn_front: head dim must be 128");
  FrontParams p;
  p.D = 2 * Hk * Dh + Hv * Dh;
  p.conv_state = conv; p.qkv = conv + (int64_t)(Kc - 1) * p.D; p.cw = cw; p.a_in = a; p.b_in = b; p.a_log = a_log;
  p.dt_bias = dt_bias; p.conv_next = nullptr; p.conv_input = nullptr;
  p.q = q; p.k = k; p.v = v; p.beta = beta; p.g = g;
  p.T = B * Tb; p.S = Kc - 1; p.Kc = Kc; p.Dh = Dh; p.Hk = Hk; p.Hv = Hv;
  p.Tb = Tb; p.seq_stride = seq_stride;
  const float inv_scale = 1.0f / sqrtf((float)Dh);
  p.q_scale = bfr(inv_scale * inv_scale);
  p.k_scale = bfr(inv_scale);
  p.eps = eps;
  const int slots = p.D / Dh;
  dim3 grid((slots + 3) / 4, B * Tb);
  gdn_front_kernel<<<grid, 128, 0, s>>>(p);
  return orn_launch_check(ctx, "gdn_front");
}
int k_gated_delta_batched(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* k, const bf16_t* v, const float* g,
                          const bf16_t* beta, float* rings, int nring, const int* cur, int B, int Tb, int Hk, int Hv, bf16_t* y) {
  if (Tb + 1 > nring) ORN_FAIL(ctx, ORN_ERR_ARG, "gated_delta: window wider than the ring");
  DeltaParams p;
  p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta; p.state = nullptr; p.snaps = nullptr;
  p.ring = rings; p.cur = cur; p.nring = nring; p.ring_final = 0; p.y = y; p.T = Tb; p.Hk = Hk; p.Hv = Hv;
  p.batched = 1;
  return launch_delta(ctx, s, p, B);
}
