// Greedy sampling over the vocabulary: bf16 log-softmax then argmax with the
// lowest index winning ties, and the raw-logit argmax of the draft chain.
//
// Replaces looped_logsumexp / vs_Subtract / argmax of the reference
// (kernels/mlx/.../logsumexp.h:3-74, arg_reduce.metal:53-66) as dispatched by
// src/ops/sample.rs:134-147,186-191.
//
// lp_i = bf(x_i - lse) with lse = bf(max + log sum exp(x - max)).  Because the
// subtraction is monotone, argmax(lp) is the lowest index whose lp equals
// bf(max - lse); so one pass produces per-1024-logit chunk (max, sum), and a
// second, single-CTA pass merges the chunks in ascending order and scans only
// the first chunk whose maximum reaches the winning lp value.
#include <atomic>

#include "orn_internal.h"

namespace {

__global__ void __launch_bounds__(256)
lse_chunk_kernel(const bf16_t* __restrict__ logits, int V, int nc, float* __restrict__ scratch) {
  __shared__ float red[32];
  const int b = blockIdx.x, t = blockIdx.y;
  const bf16_t* x = logits + (int64_t)t * V + (int64_t)b * 1024;
  const int n = min(1024, V - b * 1024);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float v[4];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int idx = 4 * threadIdx.x + i;
    v[i] = idx < n ? bf2f(x[idx]) : -INFINITY;
    m = fmaxf(m, v[i]);
  }
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = warp_max(red[lane & 7]);
  __syncthreads();
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (4 * threadIdx.x + i < n) acc = acc + orn_expf(v[i] - m);
  acc = warp_sum(acc);
  if (threadIdx.x < 32) red[threadIdx.x] = 0.f;
  __syncthreads();
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    float s = warp_sum(red[lane]);
    if (lane == 0) {
      scratch[((int64_t)t * nc + b) * 2 + 0] = m;
      scratch[((int64_t)t * nc + b) * 2 + 1] = s;
    }
  }
}

__global__ void __launch_bounds__(256)
greedy_finish_kernel(const bf16_t* __restrict__ logits, int V, int nc, int normalize,
                     const float* __restrict__ scratch, uint32_t* __restrict__ tokens) {
  extern __shared__ float sh[];  // m[nc], e[nc]
  __shared__ float red[32];
  __shared__ float s_lse, s_target;
  __shared__ int s_chunk;
  __shared__ unsigned int s_best;
  const int t = blockIdx.x;
  const float* sc = scratch + (int64_t)t * nc * 2;
  float* sm = sh;
  float* se = sh + nc;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float m = -INFINITY;
  for (int b = threadIdx.x; b < nc; b += blockDim.x) {
    sm[b] = sc[2 * b];
    m = fmaxf(m, sm[b]);
  }
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  const float M = warp_max(red[lane & 7]);
  for (int b = threadIdx.x; b < nc; b += blockDim.x) se[b] = orn_expf(sm[b] - M);
  __syncthreads();
  if (threadIdx.x == 0) {
    float lse = 0.f, target = M;
    if (normalize) {
      float S = 0.f;
      for (int b = 0; b < nc; ++b) S = fmaf(sc[2 * b + 1], se[b], S);
      lse = bfr(M + orn_logf(S));
      target = bfr(M - lse);
    }
    int chunk = 0;
    for (int b = 0; b < nc; ++b) {
      float lp = normalize ? bfr(sm[b] - lse) : sm[b];
      if (lp == target) { chunk = b; break; }
    }
    s_lse = lse; s_target = target; s_chunk = chunk; s_best = 0xffffffffu;
  }
  __syncthreads();
  const int b = s_chunk;
  const bf16_t* x = logits + (int64_t)t * V + (int64_t)b * 1024;
  const int n = min(1024, V - b * 1024);
  unsigned int best = 0xffffffffu;
#pragma unroll
  for (int i = 3; i >= 0; --i) {
    int idx = 4 * threadIdx.x + i;
    if (idx < n) {
      float lp = normalize ? bfr(bf2f(x[idx]) - s_lse) : bf2f(x[idx]);
      if (lp == s_target) best = (unsigned int)(b * 1024 + idx);
    }
  }
  best = warp_min_u32(best);
  if (lane == 0) atomicMin(&s_best, best);
  __syncthreads();
  if (threadIdx.x == 0) tokens[t] = s_best;
}
}  // namespace

size_t greedy_scratch_floats(int T, int V) { return (size_t)T * 2 * ((V + 1023) / 1024); }

int k_greedy(orn_ctx* ctx, cudaStream_t s, const bf16_t* logits, int T, int V, int normalize,
             uint32_t* tokens, float* scratch) {
  const int nc = (V + 1023) / 1024;
  dim3 grid(nc, T);
  lse_chunk_kernel<<<grid, 256, 0, s>>>(logits, V, nc, scratch);
  int rc = orn_launch_check(ctx, "lse_chunk");
  if (rc != ORN_OK) return rc;
  size_t shm = sizeof(float) * 2 * (size_t)nc;
  if (shm > 40000) ORN_FAIL(ctx, ORN_ERR_ARG, "greedy: vocabulary too large");
  greedy_finish_kernel<<<T, 256, shm, s>>>(logits, V, nc, normalize, scratch, tokens);
  return orn_launch_check(ctx, "greedy_finish");
}

// ---------------------------------------------------------------------------
// Greedy sampling without any allocation.
//
// orn_greedy borrows its [T, 2*ceil(V/1024)] floats of scratch from the device
// allocator on every call.  Some callers must not touch the allocator at all: a
// decode loop that runs with the allocator's device-wide lock held elsewhere
// (another thread loading weights), a host thread whose latency budget cannot
// absorb an allocation that may synchronise the whole device, or code that is
// about to record work on its stream (the first call on a device looks the
// array's address up and must come before any stream capture begins; later
// calls only launch the two kernels).  For them the same two kernels run on a fixed scratch array
// that lives in the module's global memory.
//
// The array is sized for the largest decode window and vocabulary the engine
// serves: 4 rows of at most 262144 logits = 2048 floats (8 KB).  Larger inputs
// are refused; orn_greedy serves them.
//
// Nothing in the array has to start at zero: the first kernel writes every
// element the second one reads.
//
// Every call on a device shares the one array.  Two calls whose kernels may
// overlap in time (different streams or contexts of the same device, or two
// host threads) race on it; callers serialise them, e.g. by using one stream.
// ---------------------------------------------------------------------------
namespace {
constexpr int kStaticGreedyMaxT = 4;
constexpr int kStaticGreedyMaxV = 262144;
constexpr size_t kStaticGreedyFloats = (size_t)kStaticGreedyMaxT * 2 * (kStaticGreedyMaxV / 1024);
constexpr int kMaxDevices = 64;
// Device address of the array per device; null = not looked up yet.  Published with release /
// read with acquire, so a second host thread on the same device never sees a half-made entry
// (two threads that race on the first call both look the address up and store the same value).
std::atomic<float*> g_static_scratch_ptr[kMaxDevices];
}  // namespace

static __device__ __align__(256) float g_greedy_static_scratch[kStaticGreedyFloats];

extern "C" int32_t orn_greedy_static(orn_ctx* ctx, const uint16_t* logits, int32_t T, int32_t V, int32_t normalize,
                                     uint32_t* tokens) {
  if (!ctx || !logits || !tokens || T < 1 || V < 1) return ORN_ERR_ARG;
  if (T > kStaticGreedyMaxT || V > kStaticGreedyMaxV)
    ORN_FAIL(ctx, ORN_ERR_ARG,
             "orn_greedy_static: at most 4 rows of at most 262144 logits fit the fixed 8 KB scratch; "
             "use orn_greedy for larger inputs");
  const int dev = ctx->device;
  if (dev < 0 || dev >= kMaxDevices) ORN_FAIL(ctx, ORN_ERR_ARG, "orn_greedy_static: device index above 63");
  float* scratch = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // one-time set-up per device, with that device current: ask the runtime where this
    // device's copy of the array lives (the array's name is not a device address on the host).
    // The calling thread's current device is put back afterwards.
    int prev = -1;
    ORN_CHECK_CUDA(ctx, cudaGetDevice(&prev));
    ORN_CHECK_CUDA(ctx, cudaSetDevice(dev));
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&p, g_greedy_static_scratch);
    if (prev >= 0 && prev != dev) cudaSetDevice(prev);
    if (e != cudaSuccess) ORN_FAIL(ctx, ORN_ERR_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    if (p == nullptr) ORN_FAIL(ctx, ORN_ERR_CUDA, "orn_greedy_static: no device address for the scratch array");
    g_static_scratch_ptr[dev].store(p, std::memory_order_release);
    scratch = p;
  }
  return k_greedy(ctx, ctx->stream, (const bf16_t*)logits, T, V, normalize, tokens, scratch);
}
