// Internal types shared by the translation units of libornith_cuda.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <set>
#include <string>
#include <utility>
#include <vector>

#include "../../include/ornith_cuda.h"
#include "orn_common.cuh"

struct orn_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  // a second stream for work that does not depend on the main chain (the shared expert beside the routed
  // experts of an expert-parallel block): forked and joined with the two events, also inside a capture
  cudaStream_t side = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  std::string err;
  int64_t launches = 0;  // kernels launched through this context
  int sm_count = 148;
  cudaEvent_t t0 = nullptr, t1 = nullptr;  // orn_timer_start / orn_timer_stop
  int* dev_err = nullptr;  // set by a kernel whose bounded wait ran out
  struct orn_ktime* kt = nullptr;  // per-kernel device times when ORN_KTIME=1 (eager launches only)
  // Kernel classes launched as programmatic dependents (bit 0 norm + mat-vec, 1 expert up, 2 expert
  // down, 3 gated-delta, 4 attention).  Measured on the replayed decode graph: bit 0 alone +3 %;
  // the gated-delta kernel +0.6 % once it is capped at two CTAs per SM (uncapped -8 %: its small
  // CTAs pile onto the first SMs the previous kernel leaves); expert up and attention +0.3 %;
  // expert down -4 %, so it stays a plain launch.  ORN_PDL_MASK overrides, ORN_NO_PDL=1 clears it.
  int pdl_mask = 27;
  // split-K scratch of the tensor-core product (gemm.cu): partial sums and per-tile arrival counters,
  // allocated once at the first product that splits (never inside a stream capture: callers run a
  // shape eagerly before they capture it)
  // group partials and arrival counters of the fused attention's long-context form (fused.cu)
  float* attn_partial = nullptr;
  int* attn_arrivals = nullptr;
  float* split_partial = nullptr;
  int* split_arrivals = nullptr;
  float* split_partial_side = nullptr;  // the same for products launched on the side stream
  int* split_arrivals_side = nullptr;
};

// Records an event after the launch just made and attributes the device time
// since the previous mark to `what` (api.cu).
void orn_ktime_mark(orn_ctx* ctx, const char* what);

// Device-resident weight matrix [E, O, K] as ROW RECORDS: every weight row is
// one contiguous, 16-byte aligned record
//   [stream 0: codes][stream 1: scales / headers][stream 2: Q6_K super-scales][pad]
// so that one bulk copy brings everything a consecutive run of rows needs.
//   Q4_K: nibble bytes K/2 | one 16-byte header {d f16, dmin f16, scales[12]} per block
//   Q6_K: ql|qh 192 bytes per block | int8 scales 16 per block | d f16 per block
//   A8  : codes K | u32 {scale bf16, bias bf16} per 64 weights
//   A4  : nibble codes K/2 | u32 {scale bf16, bias bf16} per 32 weights
//   BF16: bf16 K
// w points at row 0's record; s and b point at its streams 1 and 2 (same
// allocation), so row r's streams are w + r*rec, s + r*rec, b + r*rec.
struct RecGeom {
  uint32_t b0, b1, b2, rec;
};
__host__ __device__ inline RecGeom rec_geom(int kind, int K) {
  RecGeom g;
  const uint32_t nb = (uint32_t)K >> 8;
  switch (kind) {
    case ORN_Q4K: g.b0 = (uint32_t)K / 2; g.b1 = nb * 16; g.b2 = 0; break;
    case ORN_Q6K: g.b0 = nb * 192; g.b1 = nb * 16; g.b2 = nb * 2; break;
    case ORN_A8: g.b0 = (uint32_t)K; g.b1 = ((uint32_t)K >> 6) * 4; g.b2 = 0; break;
    case ORN_A4: g.b0 = (uint32_t)K / 2; g.b1 = ((uint32_t)K >> 5) * 4; g.b2 = 0; break;
    default: g.b0 = 2u * (uint32_t)K; g.b1 = 0; g.b2 = 0; break;
  }
  g.rec = (g.b0 + g.b1 + g.b2 + 15u) & ~15u;
  return g;
}

struct orn_linear {
  int kind = 0, E = 1, O = 0, K = 0;
  uint8_t* w = nullptr;  // the allocation: E*O records
  uint8_t* s = nullptr;  // w + b0
  uint8_t* b = nullptr;  // w + b0 + b1
  uint32_t rec = 0;      // bytes per row record
  size_t w_bytes = 0;    // device size of the allocation
  bool owns = true;
};

// POD view passed to kernels by value
struct LinDev {
  int kind, E, O, K;
  const uint8_t* w;
  const uint8_t* s;
  const uint8_t* b;
  uint32_t rec;
};
static inline LinDev lin_dev(const orn_linear* l) {
  return LinDev{l->kind, l->E, l->O, l->K, l->w, l->s, l->b, l->rec};
}

#define ORN_CHECK_CUDA(ctx, call)                                              \
  do {                                                                         \
    cudaError_t e__ = (call);                                                  \
    if (e__ != cudaSuccess) {                                                  \
      (ctx)->err = std::string(#call) + ": " + cudaGetErrorString(e__);        \
      return ORN_ERR_CUDA;                                                     \
    }                                                                          \
  } while (0)

#define ORN_FAIL(ctx, code, msg) \
  do {                           \
    (ctx)->err = (msg);          \
    return (code);               \
  } while (0)

// the context's side stream and its fork / join events, made on first use (never inside a capture); false
// when they cannot be had, inside a capture that began before they existed, with per-kernel timing on, or
// when ORN_NO_SIDE_STREAM=1 asks for one stream
bool orn_side_stream(orn_ctx* ctx);

static inline int orn_launch_check(orn_ctx* ctx, const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    ctx->err = std::string(what) + ": " + cudaGetErrorString(e);
    return ORN_ERR_CUDA;
  }
  ctx->launches += 1;
  if (ctx->kt) orn_ktime_mark(ctx, what);
  return ORN_OK;
}

// Raises a kernel's dynamic shared-memory limit once per (device, kernel).  The attribute belongs to
// the device's copy of the function, so the table is keyed by both and guarded for concurrent contexts.
inline int orn_grant_smem(orn_ctx* ctx, const void* kern, size_t bytes) {
  static std::mutex mu;
  static std::set<std::pair<int, const void*>> granted;
  const std::pair<int, const void*> key(ctx->device, kern);
  std::lock_guard<std::mutex> lock(mu);
  if (granted.count(key)) return ORN_OK;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) {
    ctx->err = std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e);
    return ORN_ERR_CUDA;
  }
  granted.insert(key);
  return ORN_OK;
}

// Launch `kern` so that it may begin while the previous kernel of the stream is still draining
// (programmatic dependent launch).  Such a kernel runs its set-up and its weight prefetch at
// once and executes griddepcontrol.wait before it touches anything an earlier kernel wrote or
// still reads.  Without the attribute the same kernel runs as an ordinary launch (the wait
// returns immediately).
template <typename... KArgs, typename... Args>
inline cudaError_t orn_launch_dependent(orn_ctx* ctx, cudaStream_t s, int cls, void (*kern)(KArgs...), dim3 grid,
                                        dim3 block, size_t smem, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = (ctx->pdl_mask >> cls) & 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// ---- kernel launchers (each returns ORN_OK or an error, work on s) ---------
// linear.cu
int k_gemv(orn_ctx* ctx, cudaStream_t s, const orn_linear* L, const bf16_t* x, int M, void* y,
           int out_f32);
int k_gather_gemv(orn_ctx* ctx, cudaStream_t s, const orn_linear* L, const bf16_t* x,
                  const uint32_t* lhs, const uint32_t* rhs, int rows, bf16_t* y);
int k_grouped_gemv(orn_ctx* ctx, cudaStream_t s, const orn_linear* L, const bf16_t* xs, const int* seg, bf16_t* y,
                   const uint32_t* row_map /*nullable*/, int max_rows /*upper bound of the rows of one expert*/);
int k_grouped_gemv2(orn_ctx* ctx, cudaStream_t st, const orn_linear* L1, bf16_t* y1, const orn_linear* L2, bf16_t* y2,
                    const bf16_t* xs, const int* seg, int max_rows);
int k_kq_dequantize(orn_ctx* ctx, cudaStream_t s, const orn_linear* L, int e, float* out);
int k_embedding(orn_ctx* ctx, cudaStream_t s, const orn_linear* L, const uint32_t* ids, int T,
                bf16_t* out);
int k_linear_pack(orn_ctx* ctx, cudaStream_t s, orn_linear* L, const uint8_t* dw,
                  const uint8_t* ds, const uint8_t* db);
int k_linear_unpack(orn_ctx* ctx, cudaStream_t s, const orn_linear* L, uint8_t* dw, uint8_t* ds,
                    uint8_t* db);
int k_linear_random(orn_ctx* ctx, cudaStream_t s, orn_linear* L, uint64_t seed, float std);
int k_linear_gather_rows(orn_ctx* ctx, cudaStream_t s, const orn_linear* L, const uint32_t* ids,
                         int n, orn_linear* out);
int k_fill_bf16(orn_ctx* ctx, cudaStream_t s, bf16_t* p, size_t n, uint64_t seed, float mean,
                float std);
void linear_artifact_sizes(int kind, int E, int O, int K, size_t* w, size_t* s, size_t* b);

// ops.cu
int k_rms_norm(orn_ctx* ctx, cudaStream_t s, const bf16_t* x, const bf16_t* w, int rows, int n,
               float eps, bf16_t* out);
int k_add_rms_norm(orn_ctx* ctx, cudaStream_t s, const bf16_t* a, const bf16_t* b,
                   const bf16_t* w, int rows, int n, float eps, bf16_t* h, bf16_t* out);
int k_rms_norm_gated(orn_ctx* ctx, cudaStream_t s, const bf16_t* x, const bf16_t* w,
                     const bf16_t* z, int rows, int n, float eps, bf16_t* out);
int k_sigmoid_gate(orn_ctx* ctx, cudaStream_t s, const bf16_t* gate, const bf16_t* x, int n,
                   int inner, bf16_t* out);
int k_swiglu(orn_ctx* ctx, cudaStream_t s, const bf16_t* g, const bf16_t* u, int n, bf16_t* out);
int k_add(orn_ctx* ctx, cudaStream_t s, const bf16_t* a, const bf16_t* b, int n, bf16_t* out);
int k_softmax_precise(orn_ctx* ctx, cudaStream_t s, const bf16_t* x, int rows, int n, bf16_t* out);
int k_softmax_topk(orn_ctx* ctx, cudaStream_t s, const bf16_t* x, int rows, int n, int k, uint32_t* inds, bf16_t* scores);
int k_swiglu2(orn_ctx* ctx, cudaStream_t s, const bf16_t* g1, const bf16_t* u1, size_t n1, bf16_t* out1, const bf16_t* g2,
              const bf16_t* u2, const int* n2_rows, int width2, bf16_t* out2);
int k_router_topk(orn_ctx* ctx, cudaStream_t s, const bf16_t* gates, int rows, int n, int k,
                  uint32_t* inds, bf16_t* scores);
int k_moe_combine(orn_ctx* ctx, cudaStream_t s, const bf16_t* scores, const bf16_t* y,
                  const bf16_t* gate, const bf16_t* shared, int T, int k, int dim, int normalize,
                  bf16_t* out);
int k_split_qgate(orn_ctx* ctx, cudaStream_t s, const bf16_t* qg, int T, int Hq, int hd, bf16_t* q,
                  bf16_t* gate);
int k_concat2(orn_ctx* ctx, cudaStream_t s, const bf16_t* a, const bf16_t* b, int T, int n,
              bf16_t* out);

// gdn.cu
int k_gdn_front(orn_ctx* ctx, cudaStream_t s, const bf16_t* conv_state, const bf16_t* qkv,
                const bf16_t* cw, const bf16_t* a, const bf16_t* b, const bf16_t* a_log,
                const bf16_t* dt_bias, int T, int Hk, int Hv, int Dh, int Kc, float eps,
                bf16_t* conv_next, bf16_t* q, bf16_t* k, bf16_t* v, bf16_t* beta, float* g,
                bf16_t* conv_input_keep);
int k_gated_delta(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* k, const bf16_t* v,
                  const float* g, const bf16_t* beta, float* state, int T, int Hk, int Hv,
                  bf16_t* y, float* snaps);
int k_gated_delta_ring(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* k,
                       const bf16_t* v, const float* g, const bf16_t* beta, float* ring,
                       int nring, const int* cur, int final_only, int T, int Hk, int Hv,
                       bf16_t* y);

int k_gdn_front_batched(orn_ctx* ctx, cudaStream_t s, const bf16_t* conv, int64_t seq_stride, const bf16_t* cw,
                        const bf16_t* a, const bf16_t* b, const bf16_t* a_log, const bf16_t* dt_bias, int B, int Tb, int Hk,
                        int Hv, int Dh, int Kc, float eps, bf16_t* q, bf16_t* k, bf16_t* v, bf16_t* beta, float* g);
int k_gated_delta_batched(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* k, const bf16_t* v, const float* g,
                          const bf16_t* beta, float* rings, int nring, const int* cur, int B, int Tb, int Hk, int Hv, bf16_t* y);

// gdn_chunk.cu: the recurrence over a prompt chunk in chunkwise form on the tensor cores (to rounding)
size_t gdn_chunk_scratch_bytes(int T, int Hv);
int k_gated_delta_chunked(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* k, const bf16_t* v, const float* g,
                          const bf16_t* beta, float* state, float* ring, int nring, const int* cur, int T, int Hk, int Hv,
                          bf16_t* y, void* scratch);

// attn.cu
int k_rope_batched(orn_ctx* ctx, cudaStream_t s, bf16_t* x, int B, int Tb, int H, int hd, int dims, float lnb, const int* pos);
int k_kv_append_batched(orn_ctx* ctx, cudaStream_t s, const bf16_t* k, const bf16_t* v, int B, int Tb, int Hkv, int hd, int cap,
                        const int* pos, bf16_t* kc, bf16_t* vc);
int k_sdpa_decode_batched(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* kc, const bf16_t* vc, int B, int Tb,
                          int Hq, int Hkv, int hd, int cap, const int* pos, float scale, bf16_t* out);
// flash.cu
int k_flash_prefill(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* kc, const bf16_t* vc, int T, int Hq, int Hkv, int hd,
                    int cap, const int* pos, float scale, bf16_t* out);
int k_rope(orn_ctx* ctx, cudaStream_t s, bf16_t* x, int T, int H, int hd, int dims, float lnb,
           const int* dev_offset, int offset_add);
int k_kv_append(orn_ctx* ctx, cudaStream_t s, const bf16_t* k, const bf16_t* v, int T, int Hkv,
                int hd, int cap, const int* dev_offset, int offset_add, bf16_t* kc, bf16_t* vc);
int k_sdpa_decode(orn_ctx* ctx, cudaStream_t s, const bf16_t* q, const bf16_t* kc,
                  const bf16_t* vc, int T, int Hq, int Hkv, int hd, int cap, const int* dev_offset,
                  int offset_add, float scale, bf16_t* out);

// sample.cu
int k_greedy(orn_ctx* ctx, cudaStream_t s, const bf16_t* logits, int T, int V, int normalize,
             uint32_t* tokens, float* scratch /* [T, 2*ceil(V/1024)] */);
size_t greedy_scratch_floats(int T, int V);
