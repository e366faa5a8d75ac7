/* TEST INFRASTRUCTURE, NOT PRODUCT CODE.  CPU restatement of ornith-rs's decode
 * hot path; see orn_oracle_math.h for what is and is not pinned. */
#ifndef ORN_ORACLE_H
#define ORN_ORACLE_H

#include "orn_oracle_math.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_Q4K = 0, ORC_Q6K = 1, ORC_A8 = 2, ORC_BF16 = 3, ORC_A4 = 4 };

/* One (optionally expert-stacked) weight matrix [E, O, K] in host memory, in
 * the reference's artifact layout (src/ops/kquant.rs:13-29, weights.rs:132-227):
 *   Q4_K : w = qs bytes [E,O,K/2], s = scales u8 [E,O,K/256,12], b = dm f16 [E,O,K/256,2]
 *   Q6_K : w = ql|qh bytes [E,O,K/256*192], s = scales i8 [E,O,K/256,16], b = d f16 [E,O,K/256]
 *   A8   : w = codes u8 [E,O,K], s = scales bf16 [E,O,K/64], b = biases bf16 [E,O,K/64]
 *   BF16 : w = bf16 [E,O,K] */
typedef struct {
  int32_t kind, E, O, K;
  const void* w;
  const void* s;
  const void* b;
} orc_lin;

typedef struct {
  int32_t hidden, n_layers, full_attn_interval;
  int32_t n_heads, n_kv_heads, head_dim, rope_dims;
  float rope_theta;
  int32_t gdn_k_heads, gdn_v_heads, gdn_head_dim, gdn_conv_kernel;
  int32_t n_experts, top_k, expert_inter, shared_inter, norm_topk_prob;
  int32_t vocab;
  float rms_eps;
  int32_t max_ctx;
} orc_config;

/* ops (orn_oracle_ops.c) */
void orc_q4k_scale_min(int j, const uint8_t* q, uint8_t* sc, uint8_t* mn);
void orc_q4k_dequantize(const uint8_t* qs, const uint8_t* scales, const uint16_t* dm,
                        int64_t nblocks, float* out);
void orc_q4k_fields(const uint8_t* qs, const uint8_t* scales, int64_t nblocks, uint8_t* sc_out,
                    uint8_t* mn_out, uint8_t* q_out);
void orc_q6k_dequantize(const uint8_t* w, const int8_t* scales, const uint16_t* dm,
                        int64_t nblocks, float* out);
float orc_row_dot(const orc_lin* L, int e, int o, const float* x);
void orc_gemv(const orc_lin* L, const bf16* x, int M, float* y_f32, bf16* y_bf);
void orc_gather_gemv(const orc_lin* L, const bf16* x, const uint32_t* lhs, const uint32_t* rhs,
                     int rows, bf16* y);
void orc_embedding_a8(const orc_lin* L, const uint32_t* ids, int T, bf16* out);
float orc_sumsq(const float* x, int n);
void orc_rms_norm(const bf16* x, const bf16* w, int rows, int n, float eps, bf16* out);
void orc_add_rms_norm(const bf16* a, const bf16* b, const bf16* w, int rows, int n, float eps,
                      bf16* h, bf16* out);
void orc_rms_norm_gated(const bf16* x, const bf16* w, const bf16* z, int rows, int n, float eps,
                        bf16* out);
void orc_sigmoid_gate(const bf16* gate, const bf16* x, int n, int inner, bf16* out);
void orc_swiglu(const bf16* g, const bf16* u, int n, bf16* out);
void orc_softmax_precise(const bf16* x, int rows, int n, bf16* out);
void orc_router_topk(const bf16* gates, int rows, int n, int k, uint32_t* inds, bf16* scores);
void orc_moe_combine(const bf16* scores, const bf16* y, const bf16* gate, const bf16* shared,
                     int T, int k, int dim, int normalize, bf16* out);
void orc_gdn_front(const bf16* conv_state, const bf16* qkv, const bf16* cw, const bf16* a_in,
                   const bf16* b_in, const bf16* a_log, const bf16* dt_bias, int T, int Hk,
                   int Hv, int Dh, int Kc, float eps, bf16* conv_next, bf16* q_out, bf16* k_out,
                   bf16* v_out, bf16* beta_out, float* g_out);
void orc_gated_delta(const bf16* q, const bf16* k, const bf16* v, const float* g, const bf16* beta,
                     float* state, int T, int Hk, int Hv, bf16* y, float* snaps);
void orc_rope(bf16* x, int T, int H, int hd, int dims, float ln_base_over_half, int offset);
void orc_sdpa_decode(const bf16* q, const bf16* kc, const bf16* vc, int T, int Hq, int Hkv,
                     int hd, int cap, int offset, float scale, bf16* out);
void orc_lse_chunk(const bf16* x, int n, float* m_out, float* s_out);
bf16 orc_logsumexp(const bf16* x, int V);
uint32_t orc_greedy_token(const bf16* logits, int V, int normalize);

/* MoE block (src/ops/moe.rs:662-741).  inds_out may be NULL. */
typedef struct {
  orc_lin gate, sw_gate, sw_up, sw_down, sh_gate, sh_up, sh_down, sh_egate;
} orc_moe;
void orc_moe_block(const orc_moe* m, const bf16* x, int T, int top_k, int norm_topk,
                   bf16* out, uint32_t* inds_out);

/* model (orn_oracle_model.c) */
typedef struct orc_model orc_model;
typedef struct orc_cache orc_cache;

orc_model* orc_model_new(const orc_config* cfg);
void orc_model_free(orc_model* m);
/* Register a tensor under its artifact name (Appendix: src/model/qwen3_5.rs:
 * 102-158, src/model/mtp.rs:96-143), with or without the
 * "language_model.model." / "language_model." prefix.  Quantised modules are
 * registered once under the module name (no ".weight"); plain tensors under
 * their full name with kind BF16.  Returns 0, or -1 for an unknown name. */
int orc_model_set(orc_model* m, const char* name, int kind, int E, int O, int K, const void* w,
                  const void* s, const void* b);
/* FR-Spec (src/frspec.rs:38-148): pruned head (row gather done by the caller)
 * and the id each pruned row stands for. */
void orc_model_set_frspec(orc_model* m, const orc_lin* pruned_head, const uint32_t* ids, int n);

orc_cache* orc_cache_new(const orc_model* m);
void orc_cache_free(orc_cache* c);
int orc_cache_offset(const orc_cache* c);

/* TextModel::forward_hidden (qwen3_5.rs:255-279): returns post-final-norm
 * hidden [T,H]; pre_norm may be NULL. */
void orc_forward(const orc_model* m, orc_cache* c, const uint32_t* ids, int T, bf16* normed,
                 bf16* pre_norm);
/* lm_head + greedy for each of T hidden rows */
void orc_head_greedy(const orc_model* m, const bf16* hidden, int T, uint32_t* tokens,
                     bf16* logits_out /* [T,V] or NULL */);

/* generate::generate_step (src/generate.rs:162-206) with the Greedy sampler.
 * Returns the number of tokens written to out. */
int orc_generate(const orc_model* m, orc_cache* c, const uint32_t* prompt, int n_prompt,
                 int max_tokens, uint32_t* out);

typedef struct {
  int32_t cycles, drafted, accepted;
  int32_t reached_by_depth[8], accepted_by_depth[8];
} orc_mtp_stats;

/* Harness device for controlled acceptance: with probability p the draft for
 * generated position i is replaced by stream[i]. */
typedef struct {
  const uint32_t* stream;
  int32_t len;
  float p;
  uint64_t seed;
} orc_force;

/* mtp_generate::generate_step_mtp (src/mtp_generate.rs:150-317), Greedy
 * sampler; policy 0 = Cycle, 1 = Committed; use_frspec drafts through the
 * pruned head.  force may be NULL. */
int orc_generate_mtp(const orc_model* m, orc_cache* c, const uint32_t* prompt, int n_prompt,
                     int depth, int max_tokens, int policy, int use_frspec,
                     const orc_force* force, uint32_t* out, orc_mtp_stats* stats);

/* OpenMP threads used by the row loops */
void orc_set_threads(int n);
int orc_get_threads(void);

#ifdef __cplusplus
}
#endif
#endif
