/* C ABI of libornith_cuda.so: the sm_100a replacement for ornith-rs's device
 * layer (src/metal/mod.rs, `Context` + `Dispatch`) and everything that layer
 * runs on the decode hot path.
 *
 * The reference binds kernels one dispatch at a time
 * (`ctx.kernel(name).arr(..).out(..).bytes(..).groups(..)`, e.g.
 * src/ops/kquant.rs:578-593).  This ABI is op-level instead: one entry point
 * per function of src/ops/ and src/model/ that the MTP depth-1 decode step
 * calls, so the Rust crate keeps its public API (generate_step,
 * generate_step_mtp, FrSpec, WeightStore) and forwards here.
 *
 * Conventions
 *   - every function returns an int32 status: 0 ok, negative = error
 *     (ORN_ERR_*); nothing aborts.  orn_last_error() gives the message.
 *   - handles are opaque and owned by the library; one orn_ctx per (thread,
 *     device); not thread-safe; all work is ordered on the context's stream.
 *   - "dev" pointers are device memory from orn_alloc (or any CUDA
 *     allocation on the context's device); "host" pointers are host memory.
 *   - activations are bfloat16 (raw uint16), accumulators float32.
 *   - a compute entry point never touches host memory and never falls back to
 *     the CPU.
 */
#ifndef ORNITH_CUDA_H
#define ORNITH_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORN_OK 0
#define ORN_ERR_ARG (-1)
#define ORN_ERR_ALLOC (-2)
#define ORN_ERR_CUDA (-3)
#define ORN_ERR_TIMEOUT (-4)
#define ORN_ERR_IO (-5)
#define ORN_ERR_STATE (-6)

/* weight formats (src/ops/linear.rs:23-40 `Linear = Mlx | K`, src/ops/kquant.rs:298-347) */
#define ORN_Q4K 0  /* ggml Q4_K, three tensors: qs / scales / dm       */
#define ORN_Q6K 1  /* ggml Q6_K, three tensors: ql|qh / scales / d     */
#define ORN_A8 2   /* mlx affine, 8 bits, group 64: codes/scales/biases */
#define ORN_BF16 3 /* dense bfloat16                                    */
#define ORN_A4 4   /* mlx affine, 4 bits, group 32 (src/ops/quantized.rs:249-278, QuantMode::Affine;
                      the shared-expert modules of the published q6k-full artifact,
                      tools/forge_q4k.py:131-152): codes/scales/biases       */

typedef struct orn_ctx orn_ctx;
typedef struct orn_linear orn_linear;
typedef struct orn_model orn_model;
typedef struct orn_cache orn_cache;
typedef struct orn_ep orn_ep;

/* model dimensions (src/model/config.rs:9-158) */
typedef struct {
  int32_t hidden, n_layers, full_attn_interval;
  int32_t n_heads, n_kv_heads, head_dim, rope_dims;
  float rope_theta;
  int32_t gdn_k_heads, gdn_v_heads, gdn_head_dim, gdn_conv_kernel;
  int32_t n_experts, top_k, expert_inter, shared_inter, norm_topk_prob;
  int32_t vocab;
  float rms_eps;
  int32_t max_ctx;
} orn_config;

/* ---- context and memory: replaces metal::Context (src/metal/mod.rs:433-519,612-646) */
int32_t orn_ctx_create(int32_t device, orn_ctx** out);
int32_t orn_ctx_destroy(orn_ctx* ctx);
int32_t orn_sync(orn_ctx* ctx);                        /* Context::sync */
const char* orn_last_error(orn_ctx* ctx);
/* The context's queue (metal::Context's one command queue, src/metal/mod.rs:433-519) as a
 * cudaStream_t: every entry point enqueues on it in call order.  A caller that interleaves its
 * own device work (an expert-parallel exchange between two ops, say) enqueues that work on this
 * stream instead of synchronising. */
int32_t orn_ctx_stream(orn_ctx* ctx, void** stream_out);
/* kernels this context has launched so far (the per-dispatch count of the reference's
 * ORNITH_PROF report, src/metal/mod.rs:197-284) */
int32_t orn_ctx_launches(orn_ctx* ctx, int64_t* count_out);
int32_t orn_alloc(orn_ctx* ctx, size_t nbytes, void** dev_out);   /* Context::alloc */
int32_t orn_free(orn_ctx* ctx, void* dev);
int32_t orn_memset(orn_ctx* ctx, void* dev, int32_t byte, size_t nbytes);
int32_t orn_upload(orn_ctx* ctx, void* dev, const void* host, size_t nbytes);   /* Array::from_slice */
int32_t orn_download(orn_ctx* ctx, void* host, const void* dev, size_t nbytes); /* Array::to_vec (syncs) */

/* Per-kernel device time on demand (the reference's ORNITH_PROF per-dispatch report,
 * src/metal/mod.rs:197-284).  Between begin and end every launch of this context is followed by a
 * CUDA event on its stream and the generation loops launch eagerly instead of replaying graphs; the
 * time between two events is charged to the later kernel.  end writes one line per kernel label,
 * "label<TAB>launches<TAB>total milliseconds", as a NUL-terminated string.  ORN_KTIME=1 in the
 * environment does the same for a whole context and prints the table when it is destroyed. */
int32_t orn_ctx_ktime_begin(orn_ctx* ctx);
int32_t orn_ctx_ktime_end(orn_ctx* ctx, char* host_buf, size_t nbytes);

/* Test hook for the library's only device-side failure report (no reference counterpart: Metal
 * command buffers report errors through their completion handler, src/metal/mod.rs:612-646).
 * Every streaming kernel waits for its own asynchronous copies with a bounded number of tries and,
 * if they run out, sets a flag that the next orn_sync turns into ORN_ERR_TIMEOUT.  This call queues
 * a one-warp kernel that waits `rounds` (1..64) tries for a copy that was never requested, so the
 * give-up path runs with nothing in flight; the following orn_sync returns ORN_ERR_TIMEOUT once and
 * the context stays usable. */
int32_t orn_debug_wait_probe(orn_ctx* ctx, uint32_t rounds);
/* the same for the expert-parallel exchange over peer memory: the gather kernel of a group of two, run
 * against a window of this process in which nobody plays the second rank; it raises its own flag, waits
 * a few seconds for the peer's, gives up, and the following orn_sync returns ORN_ERR_TIMEOUT once.
 * One GPU, one process, no peer. */
int32_t orn_debug_ep_wait_probe(orn_ctx* ctx);

/* device-side stopwatch on the context's stream (CUDA events; the reference's
 * ORNITH_PROF GPUStart/GPUEnd sums, src/metal/mod.rs:197-284) */
int32_t orn_timer_start(orn_ctx* ctx);
int32_t orn_timer_stop(orn_ctx* ctx, float* ms_out); /* synchronises */

/* ---- weights: replaces KMatrix / QuantMatrix / dense Array (src/ops/kquant.rs:349-411,
 * src/weights.rs:132-279).  Tensors are in the artifact's layout:
 *   Q4_K: w = qs bytes [E,O,K/2], s = scales u8 [E,O,K/256,12], b = dm f16 [E,O,K/256,2]
 *   Q6_K: w = ql|qh bytes [E,O,K/256*192], s = i8 [E,O,K/256,16], b = d f16 [E,O,K/256]
 *   A8  : w = codes u8 [E,O,K], s = scales bf16 [E,O,K/64], b = biases bf16 [E,O,K/64]
 *   BF16: w = bf16 [E,O,K]
 *   A4  : w = codes, 8 per u32, lowest nibble first [E,O,K/8 words], s = scales bf16 [E,O,K/32],
 *         b = biases bf16 [E,O,K/32]
 * The library copies them into its own HBM layout (16-byte-aligned streams).
 * Shape rules follow KMatrix::new: K % 256 == 0 for k-quants, K % 64 == 0 for
 * A8, K % 32 == 0 for A4, K % 8 == 0 for BF16; violations return ORN_ERR_ARG.
 * A4 matrices run through the per-op kernels and the wide product; a model that holds one outside
 * its MoE blocks runs unfused, a MoE block that holds one runs its block unfused. */
int32_t orn_linear_create(orn_ctx* ctx, int32_t kind, int32_t E, int32_t O, int32_t K,
                          const void* host_w, const void* host_s, const void* host_b,
                          orn_linear** out);
/* seeded synthetic weights ~ N(0, std) quantised on the GPU (no reference
 * counterpart: the reference's artifacts come from tools/forge_q4k.py) */
int32_t orn_linear_create_random(orn_ctx* ctx, int32_t kind, int32_t E, int32_t O, int32_t K,
                                 uint64_t seed, float std, orn_linear** out);
/* copy a matrix back to host in the artifact layout (for checkers) */
int32_t orn_linear_export(orn_ctx* ctx, const orn_linear* lin, void* host_w, void* host_s,
                          void* host_b);
int32_t orn_linear_sizes(const orn_linear* lin, size_t* w_bytes, size_t* s_bytes, size_t* b_bytes);
int32_t orn_linear_info(const orn_linear* lin, int32_t* kind, int32_t* E, int32_t* O, int32_t* K);
int32_t orn_linear_destroy(orn_ctx* ctx, orn_linear* lin);
/* FrSpec::prune (src/frspec.rs:115-135): row gather of every head tensor */
int32_t orn_linear_gather_rows(orn_ctx* ctx, const orn_linear* lin, const uint32_t* host_ids,
                               int32_t n, orn_linear** out);

/* ---- k-quant ops (src/ops/kquant.rs) */
/* kquant::dequantize -> q4k_dequantize / q6k_dequantize (kernels/q4k.metal:64-96,
 * kernels/q6k.metal:47-77): expert e of lin to float [O,K] */
int32_t orn_kq_dequantize(orn_ctx* ctx, const orn_linear* lin, int32_t e, float* dev_out);
/* Linear::matmul at M <= 4 rows -> kquant::qmv / quantized_matmul / matmul
 * (src/ops/linear.rs:23-80, kquant.rs:539-595, quantized.rs:249-333,
 * matmul.rs:334-437): y[M,O] = x[M,K] W^T.  Every row is computed with the
 * one-row arithmetic (src/ops/invariant.rs:78-116).  out_f32 != 0 stores
 * float, else bfloat16.  M > 4 is processed in groups of 4. */
int32_t orn_gemv(orn_ctx* ctx, const orn_linear* lin, const uint16_t* dev_x, int32_t M,
                 void* dev_y, int32_t out_f32);
/* Linear::gather_matmul -> kquant::gather_qmv / gather_mv (kquant.rs:741-770,
 * matmul.rs:649-711): row r = W[rhs[r]] . x[lhs[r]], bf16 out [rows,O] */
int32_t orn_gather_gemv(orn_ctx* ctx, const orn_linear* lin, const uint16_t* dev_x,
                        const uint32_t* dev_lhs, const uint32_t* dev_rhs, int32_t rows,
                        uint16_t* dev_y);
/* Linear::matmul at prompt width -> kquant::qmm_t (src/ops/kquant.rs:783-812, kernels/kquant_mm.h:
 * 88-360) / quantized_matmul / matmul above the row limit (kquant.rs:MM_ROW_LIMIT = 16):
 * y[M,O] = x[M,K] W^T on the tensor cores, weights dequantised to bfloat16 tile by tile, float32
 * accumulation, bfloat16 out (float32 when out_f32 != 0).  Any M >= 1 is accepted; the result agrees with orn_gemv to rounding,
 * not bit for bit (the reference exempts this path from row invariance, src/generate.rs:99).
 * K must be a multiple of 64. */
int32_t orn_gemm(orn_ctx* ctx, const orn_linear* lin, const uint16_t* dev_x, int32_t M,
                 void* dev_y, int32_t out_f32);
/* Linear::gather_matmul at prompt width -> kquant::gather_qmm_t (kquant.rs:905-972): row r =
 * W[rhs[r]] . x[lhs[r]].  Rows are counting-sorted by expert on the device (moe.rs:463-508), each
 * expert's rows multiply its matrix once, results land in row order.  Synchronises. */
int32_t orn_gather_gemm(orn_ctx* ctx, const orn_linear* lin, const uint16_t* dev_x,
                        const uint32_t* dev_lhs, const uint32_t* dev_rhs, int32_t rows,
                        void* dev_y, int32_t out_f32);
/* Up to four matrices of one format and row length over the same M rows in ONE launch (the
 * projections of a layer that share their input, e.g. q/k/v or the shared expert's gate and up):
 * dev_ys[j] [M, O_j].  Same arithmetic contract as orn_gemm. */
int32_t orn_gemm_multi(orn_ctx* ctx, const orn_linear* const* lins, int32_t n, const uint16_t* dev_x,
                       int32_t M, void* const* dev_ys, int32_t out_f32);
/* ops::embedding (src/ops/embedding.rs:18-47) for the affine-8 table */
int32_t orn_embedding(orn_ctx* ctx, const orn_linear* table, const uint32_t* dev_ids, int32_t T,
                      uint16_t* dev_out);

/* ---- norms and elementwise (src/ops/norm.rs:19-220, elementwise.rs) */
int32_t orn_rms_norm(orn_ctx* ctx, const uint16_t* dev_x, const uint16_t* dev_w /*nullable*/,
                     int32_t rows, int32_t n, float eps, uint16_t* dev_out);
int32_t orn_add_rms_norm(orn_ctx* ctx, const uint16_t* dev_a, const uint16_t* dev_b,
                         const uint16_t* dev_w, int32_t rows, int32_t n, float eps,
                         uint16_t* dev_h, uint16_t* dev_out);
/* The decode layers' fused form of add_rms_norm followed by up to four
 * Linear::matmul over the same normed rows (src/model/qwen3_5.rs:478-565 runs
 * input_layernorm then in_proj_qkv / in_proj_z / in_proj_a / in_proj_b;
 * norm.rs:19-220, linear.rs:23-80): h = bf16(a + b) (b nullable: h = a),
 * x = w * bf16(h * rsqrt(mean(h^2) + eps)), outs[j][M, O_j] = x lins[j]^T.
 * One persistent kernel; results are bit-identical to orn_add_rms_norm +
 * orn_gemv.  M <= 4, K <= 2048, njobs <= 4; dev_h / dev_normed (nullable)
 * receive h and x. */
int32_t orn_add_norm_gemv(orn_ctx* ctx, const uint16_t* dev_a, const uint16_t* dev_b /*nullable*/,
                          const uint16_t* dev_w, int32_t M, int32_t K, float eps,
                          const orn_linear* const* lins, uint16_t* const* dev_outs, int32_t njobs,
                          uint16_t* dev_h /*nullable*/, uint16_t* dev_normed /*nullable*/);
int32_t orn_rms_norm_gated(orn_ctx* ctx, const uint16_t* dev_x, const uint16_t* dev_w,
                           const uint16_t* dev_z, int32_t rows, int32_t n, float eps,
                           uint16_t* dev_out);
int32_t orn_sigmoid_gate(orn_ctx* ctx, const uint16_t* dev_gate, const uint16_t* dev_x, int32_t n,
                         int32_t inner, uint16_t* dev_out);
int32_t orn_swiglu(orn_ctx* ctx, const uint16_t* dev_g, const uint16_t* dev_u, int32_t n,
                   uint16_t* dev_out);

/* ---- MoE (src/ops/moe.rs, kernels/moe.metal) */
int32_t orn_softmax_precise(orn_ctx* ctx, const uint16_t* dev_x, int32_t rows, int32_t n,
                            uint16_t* dev_out);                       /* softmax.rs:18-51 */
int32_t orn_router_topk(orn_ctx* ctx, const uint16_t* dev_gates, int32_t rows, int32_t n,
                        int32_t k, uint32_t* dev_inds, uint16_t* dev_scores); /* moe.rs:113-134 */
int32_t orn_moe_combine(orn_ctx* ctx, const uint16_t* dev_scores, const uint16_t* dev_y,
                        const uint16_t* dev_gate, const uint16_t* dev_shared, int32_t T, int32_t k,
                        int32_t dim, int32_t normalize, uint16_t* dev_out);  /* moe.rs:548-596 */
/* sparse_moe_block (moe.rs:662-741) / sparse_moe_block_dense (:902-937) */
int32_t orn_moe_block(orn_ctx* ctx, const orn_linear* gate, const orn_linear* sw_gate,
                      const orn_linear* sw_up, const orn_linear* sw_down,
                      const orn_linear* sh_gate, const orn_linear* sh_up,
                      const orn_linear* sh_down, const orn_linear* sh_egate,
                      const uint16_t* dev_x, int32_t T, int32_t top_k, int32_t norm_topk,
                      uint16_t* dev_out, uint32_t* dev_inds_out /*nullable*/);

/* ---- expert parallelism over the GPUs of one node (no counterpart in the reference, which is
 * single-GPU, README.md:217-221; the block it distributes is sparse_moe_block, moe.rs:662-741,
 * and the owner's work is the sorted expert path, moe.rs:283-314,463-508).  Experts are split
 * evenly: expert e lives on rank e / (E / world).  One process per GPU; the two exchanges of a layer are
 * the library's own kernels over peer memory (exchange windows mapped at orn_ep_init, flags with bounded
 * waits) or, where the windows cannot be had, NCCL collectives on the context's stream (libnccl.so.2 is
 * resolved at run time; world == 1 needs none).  All ranks call the block with the same shapes in the
 * same order and destroy their groups together.
 * orn_ep_unique_id: rank 0 makes the 128-byte NCCL id, the caller carries it to the other ranks.
 * orn_ep_init: collective over all ranks.  orn_ep_moe_block: collective; R rows per rank (the same
 * R everywhere); gate, the shared expert and its gate are replicated, sw_* hold this rank's
 * E / world experts.  Nothing is read back to the host inside the block.  Routing, the shared
 * expert and the combine always run the row-invariant arithmetic at the row's home (routing
 * indices equal the single-GPU block's bit for bit).  The routed experts (and, from 16 rows per
 * rank, the shared expert) run as products on
 * the tensor cores (a decode batch of many sequences is a dense contraction per expert; results
 * agree with the single-GPU block to rounding), or, with ORN_EP_EXACT, through the grouped
 * row-invariant mat-vec (every output bit equals the single-GPU block's).  Either way a row's
 * result does not depend on which rows share its tile, so the output bits do not depend on world. */
int32_t orn_ep_unique_id(uint8_t* id_out /*128 bytes*/);
#define ORN_EP_EXACT 1 /* flags: routed experts through the row-invariant grouped mat-vec too */
int32_t orn_ep_init(orn_ctx* ctx, const uint8_t* id /*128 bytes; NULL when world == 1*/, int32_t rank,
                    int32_t world, int32_t flags, orn_ep** out);
int32_t orn_ep_destroy(orn_ep* ep);
int32_t orn_ep_moe_block(orn_ep* ep, const orn_linear* gate, const orn_linear* sw_gate,
                         const orn_linear* sw_up, const orn_linear* sw_down,
                         const orn_linear* sh_gate, const orn_linear* sh_up,
                         const orn_linear* sh_down, const orn_linear* sh_egate,
                         const uint16_t* dev_x, int32_t R, int32_t top_k, int32_t norm_topk,
                         uint16_t* dev_out, uint32_t* dev_inds_out /*nullable*/);

/* ---- gated delta net (src/ops/gdn.rs:191-413) */
int32_t orn_gdn_front(orn_ctx* ctx, const uint16_t* dev_conv_state, const uint16_t* dev_qkv,
                      const uint16_t* dev_conv_w, const uint16_t* dev_a, const uint16_t* dev_b,
                      const uint16_t* dev_a_log, const uint16_t* dev_dt_bias, int32_t T,
                      int32_t Hk, int32_t Hv, int32_t Dh, int32_t Kc, float eps,
                      uint16_t* dev_conv_next, uint16_t* dev_q, uint16_t* dev_k, uint16_t* dev_v,
                      uint16_t* dev_beta, float* dev_g);
/* gated_delta_kernel(_into): state [Hv,128,128] f32 updated in place; if
 * dev_snaps != NULL the state after token t is also written to snaps[t]. */
int32_t orn_gated_delta(orn_ctx* ctx, const uint16_t* dev_q, const uint16_t* dev_k,
                        const uint16_t* dev_v, const float* dev_g, const uint16_t* dev_beta,
                        float* dev_state, int32_t T, int32_t Hk, int32_t Hv, uint16_t* dev_y,
                        float* dev_snaps /*nullable*/);
/* The same recurrence over a prompt chunk in chunkwise form on the warp-level tensor cores (64-token
 * chunks: the triangular system inside a chunk solved once, the state carried from chunk to chunk by
 * bf16 products with f32 accumulation).  Same contract as orn_gated_delta without snapshots; agrees
 * with it to rounding, not bit for bit (the prompt path, src/generate.rs:99). */
int32_t orn_gated_delta_prefill(orn_ctx* ctx, const uint16_t* dev_q, const uint16_t* dev_k,
                                const uint16_t* dev_v, const float* dev_g, const uint16_t* dev_beta,
                                float* dev_state, int32_t T, int32_t Hk, int32_t Hv, uint16_t* dev_y);

/* ---- attention (src/ops/rope.rs:23-89, src/ops/sdpa.rs:122-229) */
int32_t orn_rope(orn_ctx* ctx, uint16_t* dev_x, int32_t T, int32_t H, int32_t hd, int32_t dims,
                 float theta, int32_t offset);
int32_t orn_sdpa_decode(orn_ctx* ctx, const uint16_t* dev_q, const uint16_t* dev_kc,
                        const uint16_t* dev_vc, int32_t T, int32_t Hq, int32_t Hkv, int32_t hd,
                        int32_t cap, int32_t offset, float scale, uint16_t* dev_out);
/* The prompt path's attention (the causal scaled_dot_product_attention of a chunk,
 * src/model/qwen3_5.rs:430-470): the same contract as orn_sdpa_decode for any T, computed on the
 * warp-level tensor cores with an online softmax (head_dim 256).  Agrees with orn_sdpa_decode to
 * rounding, not bit for bit (the reference exempts the prompt path from row invariance,
 * src/generate.rs:99). */
int32_t orn_sdpa_prefill(orn_ctx* ctx, const uint16_t* dev_q, const uint16_t* dev_kc,
                         const uint16_t* dev_vc, int32_t T, int32_t Hq, int32_t Hkv, int32_t hd,
                         int32_t cap, int32_t offset, float scale, uint16_t* dev_out);

/* ---- greedy sampling (src/ops/sample.rs:134-147,186-191) */
int32_t orn_greedy(orn_ctx* ctx, const uint16_t* dev_logits, int32_t T, int32_t V,
                   int32_t normalize, uint32_t* dev_tokens);
/* The same result as orn_greedy without allocating anything.  No counterpart in
 * the reference (its Metal buffers come from a pool, src/metal/mod.rs:137-143):
 * this is for callers that must not call the device allocator.  The kernels'
 * scratch is a fixed 8 KB array in the library's device memory, so T <= 4 and
 * V <= 262144; anything larger returns ORN_ERR_ARG (use orn_greedy).  The work
 * is queued on the context's stream and the call returns without waiting
 * (orn_sync or a download waits).  The first call on each device looks the
 * array's address up once; make that first call before any stream capture
 * begins.  All calls on a device share the one array: calls that may overlap in
 * time race on it, so keep them on one stream or serialise them. */
int32_t orn_greedy_static(orn_ctx* ctx, const uint16_t* dev_logits, int32_t T, int32_t V,
                          int32_t normalize, uint32_t* dev_tokens);

/* ---- model (src/model/qwen3_5.rs, mtp.rs, cache.rs; src/weights.rs) */
int32_t orn_model_create(orn_ctx* ctx, const orn_config* cfg, orn_model** out);
int32_t orn_model_destroy(orn_model* m);
/* attach a weight under its artifact name (qwen3_5.rs:102-158, mtp.rs:96-143);
 * the model takes ownership of lin */
int32_t orn_model_set_linear(orn_model* m, const char* name, orn_linear* lin);
/* plain bf16 tensor (norm weights, conv1d, A_log, dt_bias), copied from host */
int32_t orn_model_set_tensor(orn_model* m, const char* name, const uint16_t* host, size_t n);
/* random-init every weight of the config-4 mix (expert gate/up Q4_K, expert
 * down Q6_K, everything else affine-8, MTP head bf16) from one seed */
int32_t orn_model_init_random(orn_model* m, uint64_t seed);
/* TextModel::load + MtpHead::load (src/weights.rs:41-279): safetensors shards
 * + config.json in `dir`; mtp sidecar if present */
int32_t orn_model_load(orn_ctx* ctx, const char* dir, int32_t max_ctx, orn_model** out);
/* look a weight up again (checkers export it for the CPU oracle) */
int32_t orn_model_get_linear(orn_model* m, const char* name, const orn_linear** out);
int32_t orn_model_get_tensor(orn_model* m, const char* name, const uint16_t** dev_out, size_t* n);
int32_t orn_model_config(const orn_model* m, orn_config* out);
size_t orn_model_weight_bytes(const orn_model* m);
/* FrSpec::load (src/frspec.rs:67-113): ids file = u32 n + n x u32 LE */
int32_t orn_frspec_load(orn_model* m, const char* ids_path);
int32_t orn_frspec_set(orn_model* m, const uint32_t* host_ids, int32_t n);

int32_t orn_cache_create(orn_model* m, orn_cache** out);     /* make_cache + make_mtp_cache */
int32_t orn_cache_destroy(orn_cache* c);
int32_t orn_cache_reset(orn_cache* c);
int32_t orn_cache_offset(const orn_cache* c);
/* TextModel::forward_hidden: T <= 4 rows per call; dev_normed [T,H] */
int32_t orn_forward(orn_model* m, orn_cache* c, const uint32_t* host_ids, int32_t T,
                    uint16_t* dev_normed, uint16_t* dev_pre_norm /*nullable*/);
/* generate::prefill (src/generate.rs:90-136) over all n tokens: chunks of prefill_step rows
 * (the reference's default is 2048; up to 8192 rows per chunk are taken whole).  A chunk of 64 rows or more runs every projection as one wide
 * product on the tensor cores (orn_gemm / orn_gather_gemm), experts grouped by a counting sort;
 * shorter chunks run as row-invariant windows of up to 4 rows.  The caches advance by n.
 * dev_normed (nullable) receives the n hidden rows after the final norm, [n, hidden]. */
int32_t orn_prefill(orn_model* m, orn_cache* c, const uint32_t* host_ids, int32_t n,
                    int32_t prefill_step, uint16_t* dev_normed /*nullable*/);
/* forward_capture + TrunkCapture::rewind(keep) (qwen3_5.rs:190-229,324-348) */
int32_t orn_forward_capture(orn_model* m, orn_cache* c, const uint32_t* host_ids, int32_t T,
                            uint16_t* dev_normed);
int32_t orn_cache_rewind(orn_cache* c, int32_t keep);
/* MtpHead::forward (src/model/mtp.rs:150-262) for T <= 4 rows: dev_hidden [T, hidden] are the
 * trunk's post-norm rows the tokens pair with; the head's own KV cache advances by T.  kv_only:
 * only the cache rows are wanted (the Committed re-encode, src/mtp_generate.rs:292-301); otherwise
 * host_draft (nullable) receives the raw-logit argmax of the last row. */
int32_t orn_mtp_forward(orn_model* m, orn_cache* c, const uint16_t* dev_hidden, const uint32_t* host_ids,
                        int32_t T, int32_t kv_only, uint32_t* host_draft /*nullable*/);
int32_t orn_cache_mtp_offset(const orn_cache* c);
int32_t orn_cache_set_mtp_offset(orn_cache* c, int32_t offset);
/* lm_head + greedy_token for T hidden rows (generate.rs:139-150) */
int32_t orn_head_greedy(orn_model* m, const uint16_t* dev_hidden, int32_t T,
                        uint32_t* host_tokens, uint16_t* dev_logits_out /*nullable*/);

typedef int32_t (*orn_token_cb)(uint32_t token, void* user); /* return 0 to stop */

/* generate::generate_step with the Greedy sampler (src/generate.rs:162-206).
 * Caches end holding the prompt plus every token shown to on_token. */
int32_t orn_generate_step(orn_model* m, orn_cache* c, const uint32_t* host_prompt,
                          int32_t n_prompt, int32_t max_tokens, int32_t prefill_step,
                          orn_token_cb on_token, void* user);

typedef struct {
  int32_t cycles, drafted, accepted;
  int32_t reached_by_depth[8], accepted_by_depth[8];
} orn_mtp_stats; /* MtpStats, src/mtp_generate.rs:66-84 */

/* harness device for controlled acceptance (no reference counterpart): with
 * probability p the draft for generated position i is replaced by stream[i] */
typedef struct {
  const uint32_t* stream;
  int32_t len;
  float p;
  uint64_t seed;
} orn_force_draft;

#define ORN_POLICY_CYCLE 0
#define ORN_POLICY_COMMITTED 1
/* mtp_generate::generate_step_mtp with the Greedy sampler
 * (src/mtp_generate.rs:150-317); use_frspec drafts through the pruned head */
int32_t orn_generate_step_mtp(orn_model* m, orn_cache* c, const uint32_t* host_prompt,
                              int32_t n_prompt, int32_t depth, int32_t max_tokens,
                              int32_t prefill_step, int32_t policy, int32_t use_frspec,
                              const orn_force_draft* force /*nullable*/, orn_token_cb on_token,
                              void* user, orn_mtp_stats* stats);

/* per-phase device time of the last generate call, milliseconds (the
 * reference's ORNITH_PROF report, src/main.rs:256-422, reduced to phases) */
typedef struct {
  float prefill_ms, draft_ms, verify_ms, head_ms, total_ms;
  int64_t kernel_launches;
  int64_t verify_steps, draft_steps, ar_steps;
} orn_prof;
int32_t orn_get_prof(orn_model* m, orn_prof* out);

/* ---- batched decode: B concurrent sequences, a verify window of T rows each (T = 2 for MTP
 * depth 1), one pass over the weights per step.  No counterpart in the reference, which decodes one
 * sequence (README.md:217-221); the layer sequence is TextModel::forward_capture
 * (src/model/qwen3_5.rs:578-695) and the per-sequence acceptance is TrunkCapture::rewind
 * (qwen3_5.rs:324-348).  Per sequence: a KV cache of `cap` positions per attention layer, a conv
 * window and a ring of T_max + 1 recurrent states per gated-delta layer, a position.  Rows are
 * sequence-major: row b * T + t is window row t of sequence b.  The MoE blocks run through
 * orn_ep_moe_block on `ep` (NULL: this GPU alone); with a group of several ranks every rank steps
 * its own B sequences and serves its E / world experts of every layer (views into the model's
 * matrices, nothing is copied), so the call is collective.  From 16 rows the projections run on the
 * tensor cores and attention as a split-KV pass over the caches; with ORN_BATCH_EXACT (or fewer
 * rows) every product is the row-invariant mat-vec and the batched pass equals the single-sequence
 * engine bit for bit.
 * orn_batch_fill_random: benchmark set-up, every sequence as if ctx_len tokens had been decoded.
 * orn_batch_forward: host_ids [B*T]; dev_normed (nullable) [B*T, hidden]; host_targets (nullable)
 * receives the greedy token of every row (syncs).  orn_batch_commit: keep[b] in 1..T. */
typedef struct orn_batch orn_batch;
#define ORN_BATCH_EXACT 1 /* flags: row-invariant products at every row count */
#define ORN_BATCH_SPLIT_ATTN 2 /* flags: split-KV attention at every row count (isolates it for a checker) */
int32_t orn_batch_create(orn_model* m, int32_t B, int32_t T_max, int32_t cap, int32_t flags, orn_batch** out);
int32_t orn_batch_destroy(orn_batch* bt);
int32_t orn_batch_reset(orn_batch* bt);
int32_t orn_batch_fill_random(orn_batch* bt, int32_t ctx_len, uint64_t seed);
int32_t orn_batch_positions(orn_batch* bt, int32_t* host_pos /*[B]*/);
int32_t orn_batch_forward(orn_batch* bt, orn_ep* ep /*nullable*/, const uint32_t* host_ids, int32_t T,
                          uint16_t* dev_normed /*nullable*/, uint32_t* host_targets /*nullable*/);
int32_t orn_batch_commit(orn_batch* bt, const int32_t* host_keep /*[B]*/);
/* MtpHead::forward at depth 1 for every sequence (src/model/mtp.rs:150-262): host_primary [B] is the
 * token each sequence feeds next, the hidden row it pairs with is the one the last commit kept;
 * host_drafts [B] receives the raw-logit argmax.  The head has its own per-sequence KV cache; a
 * commit of the 2-row window that follows re-encodes the accepted draft into it
 * (HistoryPolicy::Committed, src/mtp_generate.rs:292-301).  One cycle = draft, forward of
 * [primary, draft], commit(1 + accepted). */
int32_t orn_batch_mtp_draft(orn_batch* bt, orn_ep* ep /*nullable*/, const uint32_t* host_primary,
                            uint32_t* host_drafts);
int32_t orn_ep_world(const orn_ep* ep);
int32_t orn_ep_rank(const orn_ep* ep);
/* 1 when the group's per-layer exchanges run as the library's own kernels over peer memory (every rank
 * mapped the exchange windows of all the others at orn_ep_init), 0 when they are NCCL collectives (one
 * rank, more than 8 ranks, windows that could not be mapped, or ORN_EP_NCCL=1 in the environment). */
int32_t orn_ep_peer_windows(const orn_ep* ep);

/* host copies of the shared elementary functions, so that a checker can
 * compare them with its own restatement without a GPU */
float orn_host_expf(float x);
float orn_host_logf(float x);
float orn_host_log1pf(float x);
void orn_host_sincosf(float a, float* s, float* c);
float orn_host_sigmoid_bf(float x);
float orn_host_softplus_bf(float x);

#ifdef __cplusplus
}
#endif
#endif
