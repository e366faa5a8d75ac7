// C ABI: context, memory, weight handles and the op-level entry points.
// The model-level entry points live in model.cu.
#include <cuda_fp16.h>

#include <cstdio>
#include <cstring>

#include "orn_internal.h"
#include "fused.h"

#define CK(call)                     \
  do {                               \
    int rc__ = (call);               \
    if (rc__ != ORN_OK) return rc__; \
  } while (0)

// ---- ORN_KTIME=1: device time per kernel name, printed when the context is destroyed ----
struct orn_ktime {
  std::vector<cudaEvent_t> ev;
  std::vector<const char*> name;
  size_t n = 0;
  std::map<std::string, std::pair<double, long>> agg;
};

static void ktime_flush(orn_ctx* ctx) {
  orn_ktime* k = ctx->kt;
  if (k->n == 0) return;
  cudaEventSynchronize(k->ev[k->n - 1]);
  for (size_t i = 1; i < k->n; ++i) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, k->ev[i - 1], k->ev[i]) == cudaSuccess) {
      auto& a = k->agg[k->name[i]];
      a.first += ms;
      a.second += 1;
    }
  }
  k->n = 0;
}

void orn_ktime_mark(orn_ctx* ctx, const char* what) {
  orn_ktime* k = ctx->kt;
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(ctx->stream, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) return;
  if (k->n == k->ev.size()) {
    if (k->ev.size() < 16384) {
      cudaEvent_t e;
      if (cudaEventCreate(&e) != cudaSuccess) return;
      k->ev.push_back(e);
      k->name.push_back(what);
    } else {
      ktime_flush(ctx);
    }
  }
  k->name[k->n] = what;
  cudaEventRecord(k->ev[k->n], ctx->stream);
  k->n += 1;
}

static void ktime_report(orn_ctx* ctx) {
  ktime_flush(ctx);
  double total = 0;
  for (auto& kv : ctx->kt->agg) total += kv.second.first;
  fprintf(stderr, "[ORN_KTIME] %-28s %10s %10s %8s %6s\n", "kernel", "launches", "total ms", "avg us", "share");
  for (auto& kv : ctx->kt->agg)
    fprintf(stderr, "[ORN_KTIME] %-28s %10ld %10.3f %8.2f %5.1f%%\n", kv.first.c_str(), kv.second.second,
            kv.second.first, 1e3 * kv.second.first / kv.second.second, 100.0 * kv.second.first / total);
  for (cudaEvent_t e : ctx->kt->ev) cudaEventDestroy(e);
  delete ctx->kt;
  ctx->kt = nullptr;
}

extern "C" {

int32_t orn_ctx_create(int32_t device, orn_ctx** out) {
  if (!out) return ORN_ERR_ARG;
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) return ORN_ERR_CUDA;
  if (device < 0 || device >= count) return ORN_ERR_ARG;
  if (cudaSetDevice(device) != cudaSuccess) return ORN_ERR_CUDA;
  orn_ctx* c = new orn_ctx();
  c->device = device;
  if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete c;
    return ORN_ERR_CUDA;
  }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) c->sm_count = prop.multiProcessorCount;
  // [0] the error flag of bounded waits; [64 ..) arrival counters of the gated-delta kernel's heads
  if (cudaMalloc((void**)&c->dev_err, 1024 * sizeof(int)) != cudaSuccess ||
      cudaMemset(c->dev_err, 0, 1024 * sizeof(int)) != cudaSuccess) {
    cudaStreamDestroy(c->stream);
    delete c;
    return ORN_ERR_ALLOC;
  }
  const char* np = getenv("ORN_NO_PDL");
  const char* pg = getenv("ORN_PDL_MASK");
  if (pg) c->pdl_mask = atoi(pg);
  if (np && np[0] == '1') c->pdl_mask = 0;
  const char* kt = getenv("ORN_KTIME");
  if (kt && kt[0] == '1') c->kt = new orn_ktime();
  *out = c;
  return ORN_OK;
}

int32_t orn_ctx_destroy(orn_ctx* ctx) {
  if (!ctx) return ORN_ERR_ARG;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->kt) ktime_report(ctx);
  if (ctx->t0) cudaEventDestroy(ctx->t0);
  if (ctx->t1) cudaEventDestroy(ctx->t1);
  cudaFree(ctx->dev_err);
  cudaFree(ctx->split_partial_side);
  cudaFree(ctx->split_arrivals_side);
  cudaFree(ctx->split_partial);
  cudaFree(ctx->attn_partial);
  cudaFree(ctx->attn_arrivals);
  cudaFree(ctx->split_arrivals);
  if (ctx->side) cudaStreamDestroy(ctx->side);
  if (ctx->ev_fork) cudaEventDestroy(ctx->ev_fork);
  if (ctx->ev_join) cudaEventDestroy(ctx->ev_join);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return ORN_OK;
}

}  // extern "C"

bool orn_side_stream(orn_ctx* ctx) {
  static const bool one = [] { const char* e = getenv("ORN_NO_SIDE_STREAM"); return e && e[0] == '1'; }();  // set once, thread-safe
  if (one || ctx->kt != nullptr) return false;
  if (ctx->side != nullptr) return true;
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(ctx->stream, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) return false;
  cudaStream_t side = nullptr;
  cudaEvent_t a = nullptr, b = nullptr;
  if (cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&a, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&b, cudaEventDisableTiming) != cudaSuccess) {
    if (side) cudaStreamDestroy(side);
    if (a) cudaEventDestroy(a);
    cudaGetLastError();
    return false;
  }
  ctx->side = side; ctx->ev_fork = a; ctx->ev_join = b;
  return true;
}

extern "C" {

int32_t orn_sync(orn_ctx* ctx) {
  if (!ctx) return ORN_ERR_ARG;
  int flag = 0;
  ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(&flag, ctx->dev_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  ORN_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (flag != 0) {
    cudaMemsetAsync(ctx->dev_err, 0, sizeof(int), ctx->stream);
    ORN_FAIL(ctx, ORN_ERR_TIMEOUT, "a kernel gave up waiting (for its own asynchronous copies, or for a peer of an expert-parallel group)");
  }
  return ORN_OK;
}

int32_t orn_ctx_ktime_begin(orn_ctx* ctx) {
  if (!ctx) return ORN_ERR_ARG;
  ORN_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->kt) ktime_flush(ctx);
  else ctx->kt = new orn_ktime();
  ctx->kt->agg.clear();
  return ORN_OK;
}

int32_t orn_ctx_ktime_end(orn_ctx* ctx, char* host_buf, size_t nbytes) {
  if (!ctx || !host_buf || nbytes < 2) return ORN_ERR_ARG;
  if (!ctx->kt) ORN_FAIL(ctx, ORN_ERR_STATE, "ktime_end without ktime_begin");
  ktime_flush(ctx);
  std::string out;
  char line[192];
  for (auto& kv : ctx->kt->agg) {
    snprintf(line, sizeof line, "%s\t%ld\t%.6f\n", kv.first.c_str(), kv.second.second, kv.second.first);
    out += line;
  }
  for (cudaEvent_t e : ctx->kt->ev) cudaEventDestroy(e);
  delete ctx->kt;
  ctx->kt = nullptr;
  if (out.size() + 1 > nbytes) ORN_FAIL(ctx, ORN_ERR_ARG, "ktime_end: buffer too small");
  memcpy(host_buf, out.c_str(), out.size() + 1);
  return ORN_OK;
}

int32_t orn_debug_wait_probe(orn_ctx* ctx, uint32_t rounds) {
  if (!ctx) return ORN_ERR_ARG;
  if (rounds < 1 || rounds > 64) ORN_FAIL(ctx, ORN_ERR_ARG, "wait probe: 1..64 rounds");
  return f_wait_probe(ctx, ctx->stream, rounds, ctx->dev_err + 32);
}

int32_t orn_timer_start(orn_ctx* ctx) {
  if (!ctx) return ORN_ERR_ARG;
  if (!ctx->t0) {
    ORN_CHECK_CUDA(ctx, cudaEventCreate(&ctx->t0));
    ORN_CHECK_CUDA(ctx, cudaEventCreate(&ctx->t1));
  }
  ORN_CHECK_CUDA(ctx, cudaEventRecord(ctx->t0, ctx->stream));
  return ORN_OK;
}

int32_t orn_timer_stop(orn_ctx* ctx, float* ms_out) {
  if (!ctx || !ms_out || !ctx->t0) return ORN_ERR_ARG;
  ORN_CHECK_CUDA(ctx, cudaEventRecord(ctx->t1, ctx->stream));
  ORN_CHECK_CUDA(ctx, cudaEventSynchronize(ctx->t1));
  ORN_CHECK_CUDA(ctx, cudaEventElapsedTime(ms_out, ctx->t0, ctx->t1));
  return ORN_OK;
}

const char* orn_last_error(orn_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }

int32_t orn_alloc(orn_ctx* ctx, size_t nbytes, void** dev_out) {
  if (!ctx || !dev_out) return ORN_ERR_ARG;
  *dev_out = nullptr;
  cudaSetDevice(ctx->device);
  cudaError_t e = cudaMalloc(dev_out, nbytes ? nbytes : 16);
  if (e != cudaSuccess) {
    ctx->err = std::string("cudaMalloc: ") + cudaGetErrorString(e);
    cudaGetLastError();
    return ORN_ERR_ALLOC;
  }
  return ORN_OK;
}

int32_t orn_free(orn_ctx* ctx, void* dev) {
  if (!ctx) return ORN_ERR_ARG;
  if (!dev) return ORN_OK;
  ORN_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ORN_CHECK_CUDA(ctx, cudaFree(dev));
  return ORN_OK;
}

int32_t orn_ctx_stream(orn_ctx* ctx, void** stream_out) {
  if (!ctx || !stream_out) return ORN_ERR_ARG;
  *stream_out = (void*)ctx->stream;
  return ORN_OK;
}

int32_t orn_ctx_launches(orn_ctx* ctx, int64_t* count_out) {
  if (!ctx || !count_out) return ORN_ERR_ARG;
  *count_out = (int64_t)ctx->launches;
  return ORN_OK;
}

int32_t orn_memset(orn_ctx* ctx, void* dev, int32_t byte, size_t nbytes) {
  if (!ctx || !dev) return ORN_ERR_ARG;
  ORN_CHECK_CUDA(ctx, cudaMemsetAsync(dev, byte, nbytes, ctx->stream));
  return ORN_OK;
}

int32_t orn_upload(orn_ctx* ctx, void* dev, const void* host, size_t nbytes) {
  if (!ctx || !dev || !host) return ORN_ERR_ARG;
  ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(dev, host, nbytes, cudaMemcpyHostToDevice, ctx->stream));
  // the host buffer may be pageable and reused by the caller right away
  ORN_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return ORN_OK;
}

int32_t orn_download(orn_ctx* ctx, void* host, const void* dev, size_t nbytes) {
  if (!ctx || !dev || !host) return ORN_ERR_ARG;
  ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(host, dev, nbytes, cudaMemcpyDeviceToHost, ctx->stream));
  ORN_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return ORN_OK;
}

// ---------------------------------------------------------------- weights
static int check_linear_shape(orn_ctx* ctx, int kind, int E, int O, int K) {
  if (E < 1 || O < 1 || K < 1) ORN_FAIL(ctx, ORN_ERR_ARG, "linear: non-positive dimension");
  if ((kind == ORN_Q4K || kind == ORN_Q6K) && K % 256 != 0)
    ORN_FAIL(ctx, ORN_ERR_ARG, "k-quant matrix: K must be a multiple of 256");
  if (kind == ORN_A8 && K % 64 != 0) ORN_FAIL(ctx, ORN_ERR_ARG, "affine-8 matrix: K must be a multiple of 64");
  if (kind == ORN_BF16 && K % 8 != 0) ORN_FAIL(ctx, ORN_ERR_ARG, "bf16 matrix: K must be a multiple of 8");
  if (kind == ORN_A4 && K % 32 != 0) ORN_FAIL(ctx, ORN_ERR_ARG, "affine-4 matrix: K must be a multiple of 32");
  if (kind < ORN_Q4K || kind > ORN_A4) ORN_FAIL(ctx, ORN_ERR_ARG, "linear: unknown kind");
  return ORN_OK;
}

static int linear_alloc(orn_ctx* ctx, int kind, int E, int O, int K, orn_linear** out) {
  CK(check_linear_shape(ctx, kind, E, O, K));
  orn_linear* L = new orn_linear();
  L->kind = kind; L->E = E; L->O = O; L->K = K;
  const RecGeom g = rec_geom(kind, K);
  L->rec = g.rec;
  L->w_bytes = (size_t)E * O * g.rec;
  int rc = orn_alloc(ctx, L->w_bytes, (void**)&L->w);
  if (rc != ORN_OK) {
    delete L;
    return rc;
  }
  L->s = L->w + g.b0;
  L->b = L->w + g.b0 + g.b1;
  *out = L;
  return ORN_OK;
}

int32_t orn_linear_create(orn_ctx* ctx, int32_t kind, int32_t E, int32_t O, int32_t K,
                          const void* host_w, const void* host_s, const void* host_b,
                          orn_linear** out) {
  if (!ctx || !out || !host_w) return ORN_ERR_ARG;
  *out = nullptr;
  CK(check_linear_shape(ctx, kind, E, O, K));
  if (kind != ORN_BF16 && (!host_s || !host_b)) ORN_FAIL(ctx, ORN_ERR_ARG, "quantised matrix needs three tensors");
  size_t aw, as, ab;
  linear_artifact_sizes(kind, E, O, K, &aw, &as, &ab);
  orn_linear* L = nullptr;
  CK(linear_alloc(ctx, kind, E, O, K, &L));
  int rc = ORN_OK;
  if (kind == ORN_BF16) {
    rc = orn_upload(ctx, L->w, host_w, aw);  // a bf16 record is the row itself
  } else {
    // stage the artifact tensors on the device, then build the row records there
    uint8_t *dw = nullptr, *ds = nullptr, *db = nullptr;
    rc = orn_alloc(ctx, aw, (void**)&dw);
    if (rc == ORN_OK) rc = orn_alloc(ctx, as, (void**)&ds);
    if (rc == ORN_OK) rc = orn_alloc(ctx, ab, (void**)&db);
    if (rc == ORN_OK) rc = orn_upload(ctx, dw, host_w, aw);
    if (rc == ORN_OK) rc = orn_upload(ctx, ds, host_s, as);
    if (rc == ORN_OK) rc = orn_upload(ctx, db, host_b, ab);
    if (rc == ORN_OK) rc = k_linear_pack(ctx, ctx->stream, L, dw, ds, db);
    if (rc == ORN_OK) rc = orn_sync(ctx);
    cudaFree(dw); cudaFree(ds); cudaFree(db);
  }
  if (rc != ORN_OK) {
    orn_linear_destroy(ctx, L);
    return rc;
  }
  *out = L;
  return ORN_OK;
}

int32_t orn_linear_create_random(orn_ctx* ctx, int32_t kind, int32_t E, int32_t O, int32_t K,
                                 uint64_t seed, float std, orn_linear** out) {
  if (!ctx || !out) return ORN_ERR_ARG;
  *out = nullptr;
  orn_linear* L = nullptr;
  CK(linear_alloc(ctx, kind, E, O, K, &L));
  int rc = k_linear_random(ctx, ctx->stream, L, seed, std);
  if (rc != ORN_OK) {
    orn_linear_destroy(ctx, L);
    return rc;
  }
  *out = L;
  return ORN_OK;
}

int32_t orn_linear_sizes(const orn_linear* lin, size_t* w, size_t* s, size_t* b) {
  if (!lin || !w || !s || !b) return ORN_ERR_ARG;
  linear_artifact_sizes(lin->kind, lin->E, lin->O, lin->K, w, s, b);
  return ORN_OK;
}

int32_t orn_linear_info(const orn_linear* lin, int32_t* kind, int32_t* E, int32_t* O, int32_t* K) {
  if (!lin || !kind || !E || !O || !K) return ORN_ERR_ARG;
  *kind = lin->kind; *E = lin->E; *O = lin->O; *K = lin->K;
  return ORN_OK;
}

int32_t orn_linear_export(orn_ctx* ctx, const orn_linear* lin, void* host_w, void* host_s,
                          void* host_b) {
  if (!ctx || !lin || !host_w) return ORN_ERR_ARG;
  size_t aw, as, ab;
  linear_artifact_sizes(lin->kind, lin->E, lin->O, lin->K, &aw, &as, &ab);
  if (lin->kind == ORN_BF16) return orn_download(ctx, host_w, lin->w, aw);
  if (!host_s || !host_b) return ORN_ERR_ARG;
  uint8_t *dw = nullptr, *ds = nullptr, *db = nullptr;
  int rc = orn_alloc(ctx, aw, (void**)&dw);
  if (rc == ORN_OK) rc = orn_alloc(ctx, as, (void**)&ds);
  if (rc == ORN_OK) rc = orn_alloc(ctx, ab, (void**)&db);
  if (rc == ORN_OK) rc = k_linear_unpack(ctx, ctx->stream, lin, dw, ds, db);
  if (rc == ORN_OK) rc = orn_download(ctx, host_w, dw, aw);
  if (rc == ORN_OK) rc = orn_download(ctx, host_s, ds, as);
  if (rc == ORN_OK) rc = orn_download(ctx, host_b, db, ab);
  cudaFree(dw); cudaFree(ds); cudaFree(db);
  return rc;
}

int32_t orn_linear_destroy(orn_ctx* ctx, orn_linear* lin) {
  if (!lin) return ORN_OK;
  if (ctx) cudaStreamSynchronize(ctx->stream);
  if (lin->owns) cudaFree(lin->w);
  delete lin;
  return ORN_OK;
}

int32_t orn_linear_gather_rows(orn_ctx* ctx, const orn_linear* lin, const uint32_t* host_ids,
                               int32_t n, orn_linear** out) {
  if (!ctx || !lin || !host_ids || !out || n < 1) return ORN_ERR_ARG;
  if (lin->E != 1) ORN_FAIL(ctx, ORN_ERR_ARG, "gather_rows: dense matrices only");
  for (int i = 0; i < n; ++i)
    if (host_ids[i] >= (uint32_t)lin->O) ORN_FAIL(ctx, ORN_ERR_ARG, "gather_rows: id out of range");
  orn_linear* L = nullptr;
  CK(linear_alloc(ctx, lin->kind, 1, n, lin->K, &L));
  uint32_t* dids = nullptr;
  int rc = orn_alloc(ctx, sizeof(uint32_t) * (size_t)n, (void**)&dids);
  if (rc == ORN_OK) rc = orn_upload(ctx, dids, host_ids, sizeof(uint32_t) * (size_t)n);
  if (rc == ORN_OK) rc = k_linear_gather_rows(ctx, ctx->stream, lin, dids, n, L);
  if (rc == ORN_OK) rc = orn_sync(ctx);
  cudaFree(dids);
  if (rc != ORN_OK) { orn_linear_destroy(ctx, L); return rc; }
  *out = L;
  return ORN_OK;
}

// ---------------------------------------------------------------- ops
int32_t orn_kq_dequantize(orn_ctx* ctx, const orn_linear* lin, int32_t e, float* dev_out) {
  if (!ctx || !lin || !dev_out) return ORN_ERR_ARG;
  if (e < 0 || e >= lin->E) ORN_FAIL(ctx, ORN_ERR_ARG, "kq_dequantize: expert out of range");
  return k_kq_dequantize(ctx, ctx->stream, lin, e, dev_out);
}

int32_t orn_gemv(orn_ctx* ctx, const orn_linear* lin, const uint16_t* dev_x, int32_t M, void* dev_y,
                 int32_t out_f32) {
  if (!ctx || !lin || !dev_x || !dev_y || M < 1) return ORN_ERR_ARG;
  if (lin->E != 1) ORN_FAIL(ctx, ORN_ERR_ARG, "gemv: expert-stacked matrix needs gather_gemv");
  return k_gemv(ctx, ctx->stream, lin, dev_x, M, dev_y, out_f32);
}

int32_t orn_gather_gemv(orn_ctx* ctx, const orn_linear* lin, const uint16_t* dev_x,
                        const uint32_t* dev_lhs, const uint32_t* dev_rhs, int32_t rows,
                        uint16_t* dev_y) {
  if (!ctx || !lin || !dev_x || !dev_lhs || !dev_rhs || !dev_y || rows < 0) return ORN_ERR_ARG;
  if (rows > 65535) ORN_FAIL(ctx, ORN_ERR_ARG, "gather_gemv: more than 65535 routed rows");
  return k_gather_gemv(ctx, ctx->stream, lin, dev_x, dev_lhs, dev_rhs, rows, dev_y);
}

int32_t orn_gemm(orn_ctx* ctx, const orn_linear* lin, const uint16_t* dev_x, int32_t M, void* dev_y, int32_t out_f32) {
  if (!ctx || !lin || !dev_x || !dev_y || M < 1) return ORN_ERR_ARG;
  return f_qgemm(ctx, ctx->stream, lin, dev_x, M, dev_y, lin->O, nullptr, nullptr, out_f32);
}

int32_t orn_gemm_multi(orn_ctx* ctx, const orn_linear* const* lins, int32_t n, const uint16_t* x, int32_t M,
                       void* const* ys, int32_t out_f32) {
  if (!ctx || !lins || !x || !ys || M < 1 || n < 1 || n > 4) return ORN_ERR_ARG;
  int ld[4];
  for (int j = 0; j < n; ++j) {
    if (!lins[j] || !ys[j]) return ORN_ERR_ARG;
    ld[j] = lins[j]->O;
  }
  return f_qgemm_multi(ctx, ctx->stream, lins, ys, ld, n, x, M, nullptr, nullptr, out_f32, 0);
}

int32_t orn_gather_gemm(orn_ctx* ctx, const orn_linear* lin, const uint16_t* dev_x, const uint32_t* dev_lhs,
                        const uint32_t* dev_rhs, int32_t rows, void* dev_y, int32_t out_f32) {
  if (!ctx || !lin || !dev_x || !dev_lhs || !dev_rhs || !dev_y || rows < 1) return ORN_ERR_ARG;
  // sort the rows by expert, gather their inputs, run the grouped product, results back in row order
  cudaStream_t s = ctx->stream;
  const size_t seg_b = ((size_t)(2 * lin->E + 2) * sizeof(int) + 255) & ~(size_t)255;
  const size_t perm_b = ((size_t)rows * sizeof(uint32_t) + 255) & ~(size_t)255;
  const size_t xs_b = ((size_t)rows * lin->K * sizeof(bf16_t) + 255) & ~(size_t)255;
  const size_t sc_b = qgemm_scratch_bytes(rows, lin->E, lin->O);
  uint8_t* buf = nullptr;
  CK(orn_alloc(ctx, seg_b + perm_b + xs_b + sc_b, (void**)&buf));
  int* seg = reinterpret_cast<int*>(buf);
  uint32_t* perm = reinterpret_cast<uint32_t*>(buf + seg_b);
  bf16_t* xs = reinterpret_cast<bf16_t*>(buf + seg_b + perm_b);
  int rc = f_route_sort(ctx, s, dev_rhs, rows, lin->E, seg, seg + lin->E + 1, perm);
  if (rc == ORN_OK) rc = f_gather_rows(ctx, s, dev_x, dev_lhs, perm, rows, lin->K, xs);
  QGemmGroup g{seg, perm, 0};
  if (rc == ORN_OK) rc = f_qgemm(ctx, s, lin, xs, rows, dev_y, lin->O, &g, buf + seg_b + perm_b + xs_b, out_f32);
  if (rc == ORN_OK) rc = orn_sync(ctx);
  else cudaStreamSynchronize(s);
  cudaFree(buf);
  return rc;
}

int32_t orn_embedding(orn_ctx* ctx, const orn_linear* table, const uint32_t* dev_ids, int32_t T,
                      uint16_t* dev_out) {
  if (!ctx || !table || !dev_ids || !dev_out || T < 1) return ORN_ERR_ARG;
  return k_embedding(ctx, ctx->stream, table, dev_ids, T, dev_out);
}

int32_t orn_rms_norm(orn_ctx* ctx, const uint16_t* x, const uint16_t* w, int32_t rows, int32_t n,
                     float eps, uint16_t* out) {
  if (!ctx || !x || !out || rows < 1 || n < 1) return ORN_ERR_ARG;
  return k_rms_norm(ctx, ctx->stream, x, w, rows, n, eps, out);
}
int32_t orn_add_rms_norm(orn_ctx* ctx, const uint16_t* a, const uint16_t* b, const uint16_t* w,
                         int32_t rows, int32_t n, float eps, uint16_t* h, uint16_t* out) {
  if (!ctx || !a || !b || !h || !out || rows < 1 || n < 1) return ORN_ERR_ARG;
  return k_add_rms_norm(ctx, ctx->stream, a, b, w, rows, n, eps, h, out);
}
int32_t orn_add_norm_gemv(orn_ctx* ctx, const uint16_t* a, const uint16_t* b, const uint16_t* w, int32_t M,
                          int32_t K, float eps, const orn_linear* const* lins, uint16_t* const* outs,
                          int32_t njobs, uint16_t* h, uint16_t* normed) {
  if (!ctx || !a || !w || !lins || !outs || M < 1 || M > 4 || njobs < 1 || njobs > 4) return ORN_ERR_ARG;
  FusedPrologue fp;
  fp.mode = PRO_ADDNORM; fp.K = K; fp.a = a; fp.b = b; fp.w = w; fp.eps = eps; fp.sum_out = h; fp.norm_out = normed;
  FusedJob jobs[4];
  for (int j = 0; j < njobs; ++j) {
    if (!lins[j] || !outs[j] || lins[j]->E != 1) return ORN_ERR_ARG;
    jobs[j].lin = lins[j];
    jobs[j].out = outs[j];
  }
  return f_norm_gemv(ctx, ctx->stream, M, fp, jobs, njobs);
}
int32_t orn_rms_norm_gated(orn_ctx* ctx, const uint16_t* x, const uint16_t* w, const uint16_t* z,
                           int32_t rows, int32_t n, float eps, uint16_t* out) {
  if (!ctx || !x || !w || !z || !out || rows < 1 || n < 1) return ORN_ERR_ARG;
  return k_rms_norm_gated(ctx, ctx->stream, x, w, z, rows, n, eps, out);
}
int32_t orn_sigmoid_gate(orn_ctx* ctx, const uint16_t* gate, const uint16_t* x, int32_t n,
                         int32_t inner, uint16_t* out) {
  if (!ctx || !gate || !x || !out || n < 1 || inner < 1) return ORN_ERR_ARG;
  return k_sigmoid_gate(ctx, ctx->stream, gate, x, n, inner, out);
}
int32_t orn_swiglu(orn_ctx* ctx, const uint16_t* g, const uint16_t* u, int32_t n, uint16_t* out) {
  if (!ctx || !g || !u || !out || n < 1) return ORN_ERR_ARG;
  return k_swiglu(ctx, ctx->stream, g, u, n, out);
}
int32_t orn_softmax_precise(orn_ctx* ctx, const uint16_t* x, int32_t rows, int32_t n, uint16_t* out) {
  if (!ctx || !x || !out || rows < 1 || n < 1) return ORN_ERR_ARG;
  return k_softmax_precise(ctx, ctx->stream, x, rows, n, out);
}
int32_t orn_router_topk(orn_ctx* ctx, const uint16_t* gates, int32_t rows, int32_t n, int32_t k,
                        uint32_t* inds, uint16_t* scores) {
  if (!ctx || !gates || !inds || !scores || rows < 1 || k < 1) return ORN_ERR_ARG;
  return k_router_topk(ctx, ctx->stream, gates, rows, n, k, inds, scores);
}
int32_t orn_moe_combine(orn_ctx* ctx, const uint16_t* scores, const uint16_t* y,
                        const uint16_t* gate, const uint16_t* shared, int32_t T, int32_t k,
                        int32_t dim, int32_t normalize, uint16_t* out) {
  if (!ctx || !scores || !y || !gate || !shared || !out || T < 1) return ORN_ERR_ARG;
  return k_moe_combine(ctx, ctx->stream, scores, y, gate, shared, T, k, dim, normalize, out);
}

int32_t orn_gdn_front(orn_ctx* ctx, const uint16_t* conv_state, const uint16_t* qkv,
                      const uint16_t* conv_w, const uint16_t* a, const uint16_t* b,
                      const uint16_t* a_log, const uint16_t* dt_bias, int32_t T, int32_t Hk,
                      int32_t Hv, int32_t Dh, int32_t Kc, float eps, uint16_t* conv_next,
                      uint16_t* q, uint16_t* k, uint16_t* v, uint16_t* beta, float* g) {
  if (!ctx || !conv_state || !qkv || !conv_w || !a || !b || !a_log || !dt_bias || !conv_next ||
      !q || !k || !v || !beta || !g || T < 1)
    return ORN_ERR_ARG;
  return k_gdn_front(ctx, ctx->stream, conv_state, qkv, conv_w, a, b, a_log, dt_bias, T, Hk, Hv, Dh,
                     Kc, eps, conv_next, q, k, v, beta, g, nullptr);
}
int32_t orn_gated_delta(orn_ctx* ctx, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                        const float* g, const uint16_t* beta, float* state, int32_t T, int32_t Hk,
                        int32_t Hv, uint16_t* y, float* snaps) {
  if (!ctx || !q || !k || !v || !g || !beta || !state || !y || T < 1) return ORN_ERR_ARG;
  return k_gated_delta(ctx, ctx->stream, q, k, v, g, beta, state, T, Hk, Hv, y, snaps);
}

int32_t orn_gated_delta_prefill(orn_ctx* ctx, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                const float* g, const uint16_t* beta, float* state, int32_t T, int32_t Hk,
                                int32_t Hv, uint16_t* y) {
  if (!ctx || !q || !k || !v || !g || !beta || !state || !y || T < 1) return ORN_ERR_ARG;
  void* scratch = nullptr;
  CK(orn_alloc(ctx, gdn_chunk_scratch_bytes(T, Hv), &scratch));
  int rc = k_gated_delta_chunked(ctx, ctx->stream, q, k, v, g, beta, state, nullptr, 1, nullptr, T, Hk, Hv, y, scratch);
  if (rc == ORN_OK) rc = orn_sync(ctx);
  orn_free(ctx, scratch);
  return rc;
}

int32_t orn_rope(orn_ctx* ctx, uint16_t* x, int32_t T, int32_t H, int32_t hd, int32_t dims,
                 float theta, int32_t offset) {
  if (!ctx || !x || T < 1 || dims > hd || dims % 2) return ORN_ERR_ARG;
  float lnb = (float)(log((double)theta) / (double)(dims / 2));
  return k_rope(ctx, ctx->stream, x, T, H, hd, dims, lnb, nullptr, offset);
}
int32_t orn_sdpa_decode(orn_ctx* ctx, const uint16_t* q, const uint16_t* kc, const uint16_t* vc,
                        int32_t T, int32_t Hq, int32_t Hkv, int32_t hd, int32_t cap,
                        int32_t offset, float scale, uint16_t* out) {
  if (!ctx || !q || !kc || !vc || !out || T < 1) return ORN_ERR_ARG;
  if (offset + T > cap) ORN_FAIL(ctx, ORN_ERR_ARG, "sdpa_decode: window exceeds the cache capacity");
  return k_sdpa_decode(ctx, ctx->stream, q, kc, vc, T, Hq, Hkv, hd, cap, nullptr, offset, scale, out);
}

int32_t orn_sdpa_prefill(orn_ctx* ctx, const uint16_t* q, const uint16_t* kc, const uint16_t* vc,
                         int32_t T, int32_t Hq, int32_t Hkv, int32_t hd, int32_t cap,
                         int32_t offset, float scale, uint16_t* out) {
  if (!ctx || !q || !kc || !vc || !out || T < 1 || offset < 0) return ORN_ERR_ARG;
  if (offset + T > cap) ORN_FAIL(ctx, ORN_ERR_ARG, "sdpa_prefill: chunk exceeds the cache capacity");
  int* pos = nullptr;
  CK(orn_alloc(ctx, sizeof(int), (void**)&pos));
  int rc = orn_upload(ctx, pos, &offset, sizeof(int));
  if (rc == ORN_OK) rc = k_flash_prefill(ctx, ctx->stream, q, kc, vc, T, Hq, Hkv, hd, cap, pos, scale, out);
  if (rc == ORN_OK) rc = orn_sync(ctx);
  orn_free(ctx, pos);
  return rc;
}

int32_t orn_greedy(orn_ctx* ctx, const uint16_t* logits, int32_t T, int32_t V, int32_t normalize,
                   uint32_t* tokens) {
  if (!ctx || !logits || !tokens || T < 1 || V < 1) return ORN_ERR_ARG;
  float* scratch = nullptr;
  CK(orn_alloc(ctx, sizeof(float) * greedy_scratch_floats(T, V), (void**)&scratch));
  int rc = k_greedy(ctx, ctx->stream, logits, T, V, normalize, tokens, scratch);
  if (rc == ORN_OK) rc = orn_sync(ctx);
  cudaFree(scratch);
  return rc;
}

// host copies of the elementary functions
float orn_host_expf(float x) { return orn_expf(x); }
float orn_host_logf(float x) { return orn_logf(x); }
float orn_host_log1pf(float x) { return orn_log1pf(x); }
void orn_host_sincosf(float a, float* s, float* c) { orn_sincosf(a, s, c); }
float orn_host_sigmoid_bf(float x) { return orn_sigmoid_bf(x); }
float orn_host_softplus_bf(float x) { return orn_softplus_bf(x); }

}  // extern "C"
