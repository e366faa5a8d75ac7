// Model level of the C ABI: the Qwen3.5-MoE trunk, the MTP head, the caches
// and the two greedy generation loops.
//
// Follows src/model/qwen3_5.rs (TextModel::forward_hidden / forward_capture,
// TrunkCapture::rewind), src/model/mtp.rs (MtpHead::hidden / forward),
// src/model/cache.rs, src/generate.rs (prefill, step, generate_step) and
// src/mtp_generate.rs (draft, generate_step_mtp).  Host code only sequences
// kernels; positions and the state-ring selector live in device memory so
// that nothing the kernels read changes address from step to step.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <type_traits>

#include "fused.h"
#include "model_types.h"
#include "orn_internal.h"

#define CK(call)                     \
  do {                               \
    int rc__ = (call);               \
    if (rc__ != ORN_OK) return rc__; \
  } while (0)

namespace {

__global__ void iota_div_kernel(uint32_t* lhs, uint32_t* ident, int n, int k) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { lhs[i] = (uint32_t)(i / k); ident[i] = (uint32_t)i; }
}
__global__ void set_u32_kernel(uint32_t* p, uint32_t v) { *p = v; }
__global__ void set_int_kernel(int* p, int v) { *p = v; }
// mailbox = {primary, force flag[3], force token[3]} written by the host before each cycle;
// slot < 0 places the primary at the head of the window, slot i applies draft i's override
__global__ void mailbox_apply_kernel(const uint32_t* mb, uint32_t* window, int slot) {
  if (slot < 0) window[0] = mb[0];
  else if (mb[1 + slot] != 0) window[slot + 1] = mb[4 + slot];
}
__global__ void add_int_kernel(int* p, int v) { *p += v; }
// FrSpec::map_id (src/frspec.rs:137-148, kernels/moe.metal:68-74 gather_u32)
__global__ void gather_u32_kernel(const uint32_t* table, const uint32_t* idx, uint32_t* out) {
  *out = table[*idx];
}
// rows keep..keep+S-1 of every layer's conv window move to rows 0..S-1
// (TrunkCapture::rewind, qwen3_5.rs:324-348: conv = slice of conv_input)
__global__ void conv_shift_kernel(bf16_t* const* bufs, int S, int D, int keep) {
  bf16_t* b = bufs[blockIdx.y];
  int c = blockIdx.x * blockDim.x + threadIdx.x;  // over D/8 16-byte pieces
  if (c >= D / 8) return;
  uint4* p = reinterpret_cast<uint4*>(b);
  for (int j = 0; j < S; ++j) p[(size_t)j * (D / 8) + c] = p[(size_t)(j + keep) * (D / 8) + c];
}
__global__ void copy_bf16_kernel(const bf16_t* src, bf16_t* dst, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[i];
}

std::string canon(const char* name) {
  std::string n(name);
  const char* p1 = "language_model.model.";
  const char* p2 = "language_model.";
  if (n.rfind(p1, 0) == 0) n = n.substr(strlen(p1));
  else if (n.rfind(p2, 0) == 0) n = n.substr(strlen(p2));
  return n;
}

}  // namespace

namespace {

int conv_dim(const orn_config& c) {
  return 2 * c.gdn_k_heads * c.gdn_head_dim + c.gdn_v_heads * c.gdn_head_dim;
}
bool is_linear_layer(const orn_config& c, int i) { return ((i + 1) % c.full_attn_interval) != 0; }

template <typename T>
int ws_alloc(orn_model* m, T** p, size_t count) {
  void* d = nullptr;
  CK(orn_alloc(m->ctx, sizeof(T) * (count ? count : 1), &d));
  m->ws_allocs.push_back(d);
  *p = (T*)d;
  return ORN_OK;
}

int build_workspace(orn_model* m) {
  const orn_config& c = m->cfg;
  Workspace& w = m->ws;
  const size_t R = kMaxRows, H = c.hidden;
  const size_t D = conv_dim(c), VD = (size_t)c.gdn_v_heads * c.gdn_head_dim;
  const size_t KD = (size_t)c.gdn_k_heads * c.gdn_head_dim;
  const size_t QD = (size_t)c.n_heads * c.head_dim, KVD = (size_t)c.n_kv_heads * c.head_dim;
  const size_t E = c.n_experts, I = c.expert_inter, SI = c.shared_inter, k = c.top_k;
  (void)D;
  CK(ws_alloc(m, &w.x, R * H)); CK(ws_alloc(m, &w.normed, R * H)); CK(ws_alloc(m, &w.r, R * H));
  CK(ws_alloc(m, &w.h, R * H)); CK(ws_alloc(m, &w.normed2, R * H)); CK(ws_alloc(m, &w.mo, R * H));
  CK(ws_alloc(m, &w.z, R * VD)); CK(ws_alloc(m, &w.aa, R * c.gdn_v_heads)); CK(ws_alloc(m, &w.bb, R * c.gdn_v_heads));
  CK(ws_alloc(m, &w.gq, R * KD)); CK(ws_alloc(m, &w.gk, R * KD)); CK(ws_alloc(m, &w.gv, R * VD));
  CK(ws_alloc(m, &w.beta, R * c.gdn_v_heads)); CK(ws_alloc(m, &w.gg, R * c.gdn_v_heads));
  CK(ws_alloc(m, &w.gy, R * VD)); CK(ws_alloc(m, &w.ggated, R * VD));
  CK(ws_alloc(m, &w.qg, R * 2 * QD)); CK(ws_alloc(m, &w.aq, R * QD)); CK(ws_alloc(m, &w.agate, R * QD));
  CK(ws_alloc(m, &w.ak, R * KVD)); CK(ws_alloc(m, &w.av, R * KVD)); CK(ws_alloc(m, &w.att, R * QD));
  CK(ws_alloc(m, &w.agated, R * QD));
  CK(ws_alloc(m, &w.gates, R * E)); CK(ws_alloc(m, &w.probs, R * E)); CK(ws_alloc(m, &w.scores, R * k));
  CK(ws_alloc(m, &w.eg, R * k * I)); CK(ws_alloc(m, &w.eu, R * k * I)); CK(ws_alloc(m, &w.eact, R * k * I));
  CK(ws_alloc(m, &w.ey, R * k * H)); CK(ws_alloc(m, &w.sg, R * SI)); CK(ws_alloc(m, &w.su, R * SI));
  CK(ws_alloc(m, &w.sact, R * SI)); CK(ws_alloc(m, &w.sy, R * H)); CK(ws_alloc(m, &w.gs, R));
  CK(ws_alloc(m, &w.inds, R * k)); CK(ws_alloc(m, &w.lhs, R * k)); CK(ws_alloc(m, &w.ident, R * k));
  CK(ws_alloc(m, &w.logits, R * (size_t)c.vocab)); CK(ws_alloc(m, &w.dlogits, (size_t)c.vocab));
  CK(ws_alloc(m, &w.greedy_scratch, greedy_scratch_floats(kMaxRows, c.vocab)));
  CK(ws_alloc(m, &w.ids, (size_t)8)); CK(ws_alloc(m, &w.window, (size_t)8));
  CK(ws_alloc(m, &w.targets, (size_t)8)); CK(ws_alloc(m, &w.local, (size_t)1)); CK(ws_alloc(m, &w.mailbox, (size_t)16));
  CK(ws_alloc(m, &w.vh, R * H)); CK(ws_alloc(m, &w.hrow, H)); CK(ws_alloc(m, &w.dh, R * H));
  CK(ws_alloc(m, &w.memb, R * H)); CK(ws_alloc(m, &w.me, R * H)); CK(ws_alloc(m, &w.mh, R * H));
  CK(ws_alloc(m, &w.mjoined, R * 2 * H)); CK(ws_alloc(m, &w.mx, R * H));
  int n = kMaxRows * c.top_k;
  iota_div_kernel<<<(n + 63) / 64, 64, 0, m->ctx->stream>>>(w.lhs, w.ident, n, c.top_k);
  return orn_launch_check(m->ctx, "iota_div");
}

orn_linear* find_lin(orn_model* m, const std::string& name) {
  auto it = m->lins.find(name);
  return it == m->lins.end() ? nullptr : it->second;
}
bf16_t* find_tensor(orn_model* m, const std::string& name) {
  auto it = m->tensors.find(name);
  return it == m->tensors.end() ? nullptr : it->second.p;
}

int need_lin(orn_model* m, const std::string& name, int O, int K, int E, orn_linear** out) {
  orn_linear* l = find_lin(m, name);
  if (!l) ORN_FAIL(m->ctx, ORN_ERR_STATE, "model: missing weight " + name);
  if (l->O != O || l->K != K || l->E != E) ORN_FAIL(m->ctx, ORN_ERR_ARG, "model: wrong shape for " + name);
  *out = l;
  return ORN_OK;
}
int need_tensor(orn_model* m, const std::string& name, size_t n, bf16_t** out) {
  auto it = m->tensors.find(name);
  if (it == m->tensors.end()) ORN_FAIL(m->ctx, ORN_ERR_STATE, "model: missing tensor " + name);
  if (it->second.n != n) ORN_FAIL(m->ctx, ORN_ERR_ARG, "model: wrong size for " + name);
  *out = it->second.p;
  return ORN_OK;
}

int load_moe(orn_model* m, const std::string& p, Moe& moe) {
  const orn_config& c = m->cfg;
  CK(need_lin(m, p + "gate", c.n_experts, c.hidden, 1, &moe.gate));
  CK(need_lin(m, p + "switch_mlp.gate_proj", c.expert_inter, c.hidden, c.n_experts, &moe.sw_gate));
  CK(need_lin(m, p + "switch_mlp.up_proj", c.expert_inter, c.hidden, c.n_experts, &moe.sw_up));
  CK(need_lin(m, p + "switch_mlp.down_proj", c.hidden, c.expert_inter, c.n_experts, &moe.sw_down));
  CK(need_lin(m, p + "shared_expert.gate_proj", c.shared_inter, c.hidden, 1, &moe.sh_gate));
  CK(need_lin(m, p + "shared_expert.up_proj", c.shared_inter, c.hidden, 1, &moe.sh_up));
  CK(need_lin(m, p + "shared_expert.down_proj", c.hidden, c.shared_inter, 1, &moe.sh_down));
  CK(need_lin(m, p + "shared_expert_gate", 1, c.hidden, 1, &moe.sh_egate));
  return ORN_OK;
}

// resolve every name the forward pass needs (TextModel::load, qwen3_5.rs:102-158;
// MtpHead::load, mtp.rs:96-143)
int finalize(orn_model* m) {
  if (m->finalized) return ORN_OK;
  const orn_config& c = m->cfg;
  const int H = c.hidden, D = conv_dim(c), VD = c.gdn_v_heads * c.gdn_head_dim;
  const int QD = c.n_heads * c.head_dim, KVD = c.n_kv_heads * c.head_dim;
  CK(need_lin(m, "embed_tokens", c.vocab, H, 1, &m->embed));
  if (m->embed->kind != ORN_A8) ORN_FAIL(m->ctx, ORN_ERR_ARG, "model: embed_tokens must be affine-8");
  CK(need_lin(m, "lm_head", c.vocab, H, 1, &m->lm_head));
  CK(need_tensor(m, "norm.weight", H, &m->norm));
  m->layers.assign(c.n_layers, Layer());
  for (int i = 0; i < c.n_layers; ++i) {
    Layer& ly = m->layers[i];
    std::string lp = "layers." + std::to_string(i) + ".";
    ly.linear = is_linear_layer(c, i);
    CK(need_tensor(m, lp + "input_layernorm.weight", H, &ly.input_ln));
    CK(need_tensor(m, lp + "post_attention_layernorm.weight", H, &ly.post_ln));
    if (ly.linear) {
      std::string a = lp + "linear_attn.";
      CK(need_lin(m, a + "in_proj_qkv", D, H, 1, &ly.in_qkv));
      CK(need_lin(m, a + "in_proj_z", VD, H, 1, &ly.in_z));
      CK(need_lin(m, a + "in_proj_a.weight", c.gdn_v_heads, H, 1, &ly.in_a));
      CK(need_lin(m, a + "in_proj_b.weight", c.gdn_v_heads, H, 1, &ly.in_b));
      CK(need_lin(m, a + "out_proj", H, VD, 1, &ly.out_proj));
      CK(need_tensor(m, a + "conv1d.weight", (size_t)D * c.gdn_conv_kernel, &ly.conv_w));
      CK(need_tensor(m, a + "dt_bias", c.gdn_v_heads, &ly.dt_bias));
      CK(need_tensor(m, a + "A_log", c.gdn_v_heads, &ly.a_log));
      CK(need_tensor(m, a + "norm.weight", c.gdn_head_dim, &ly.gdn_norm));
    } else {
      std::string a = lp + "self_attn.";
      CK(need_lin(m, a + "q_proj", 2 * QD, H, 1, &ly.q_proj));
      CK(need_lin(m, a + "k_proj", KVD, H, 1, &ly.k_proj));
      CK(need_lin(m, a + "v_proj", KVD, H, 1, &ly.v_proj));
      CK(need_lin(m, a + "o_proj", H, QD, 1, &ly.o_proj));
      CK(need_tensor(m, a + "q_norm.weight", c.head_dim, &ly.q_norm));
      CK(need_tensor(m, a + "k_norm.weight", c.head_dim, &ly.k_norm));
    }
    CK(load_moe(m, lp + "mlp.", ly.moe));
  }
  if (find_lin(m, "mtp.fc.weight")) {
    Mtp& h = m->mtp;
    std::string lp = "mtp.layers.0.";
    CK(need_tensor(m, "mtp.pre_fc_norm_embedding.weight", H, &h.pre_fc_norm_embedding));
    CK(need_tensor(m, "mtp.pre_fc_norm_hidden.weight", H, &h.pre_fc_norm_hidden));
    CK(need_lin(m, "mtp.fc.weight", H, 2 * H, 1, &h.fc));
    CK(need_tensor(m, "mtp.norm.weight", H, &h.norm));
    CK(need_tensor(m, lp + "input_layernorm.weight", H, &h.input_ln));
    CK(need_tensor(m, lp + "post_attention_layernorm.weight", H, &h.post_ln));
    CK(need_lin(m, lp + "self_attn.q_proj.weight", 2 * QD, H, 1, &h.q_proj));
    CK(need_lin(m, lp + "self_attn.k_proj.weight", KVD, H, 1, &h.k_proj));
    CK(need_lin(m, lp + "self_attn.v_proj.weight", KVD, H, 1, &h.v_proj));
    CK(need_lin(m, lp + "self_attn.o_proj.weight", H, QD, 1, &h.o_proj));
    CK(need_tensor(m, lp + "self_attn.q_norm.weight", c.head_dim, &h.q_norm));
    CK(need_tensor(m, lp + "self_attn.k_norm.weight", c.head_dim, &h.k_norm));
    CK(load_moe(m, lp + "mlp.", h.moe));
    h.present = true;
  }
  // formats outside the fused kernels' four: allowed anywhere, but only MoE blocks fall back one by one
  m->fused_ok = m->embed->kind <= ORN_BF16 && m->lm_head->kind <= ORN_BF16;
  for (const Layer& ly : m->layers) {
    const orn_linear* mix[9] = {ly.in_qkv, ly.in_z, ly.in_a, ly.in_b, ly.out_proj, ly.q_proj, ly.k_proj, ly.v_proj, ly.o_proj};
    for (const orn_linear* l : mix)
      if (l != nullptr && l->kind > ORN_BF16) m->fused_ok = false;
  }
  if (m->mtp.present) {
    const orn_linear* mix[5] = {m->mtp.fc, m->mtp.q_proj, m->mtp.k_proj, m->mtp.v_proj, m->mtp.o_proj};
    for (const orn_linear* l : mix)
      if (l->kind > ORN_BF16) m->fused_ok = false;
  }
  m->lnb = (float)(std::log((double)c.rope_theta) / (double)(c.rope_dims / 2));
  CK(build_workspace(m));
  for (int i = 0; i < 4; ++i) ORN_CHECK_CUDA(m->ctx, cudaEventCreate(&m->ev[i]));
  m->finalized = true;
  return ORN_OK;
}

// ------------------------------------------------------------------ blocks
// sparse_moe_block (src/ops/moe.rs:662-741); with bf16 weights it is
// sparse_moe_block_dense (:902-937): the same sequence of ops.
int moe_block(orn_model* m, const Moe& moe, const bf16_t* x, int T, bf16_t* out, uint32_t* inds_out) {
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  Workspace& w = m->ws;
  const orn_config& c = m->cfg;
  const int rows = T * c.top_k;
  CK(k_gemv(ctx, s, moe.gate, x, T, w.gates, 0));
  CK(k_gemv(ctx, s, moe.sh_gate, x, T, w.sg, 0));
  CK(k_gemv(ctx, s, moe.sh_up, x, T, w.su, 0));
  CK(k_gemv(ctx, s, moe.sh_egate, x, T, w.gs, 0));
  CK(k_softmax_precise(ctx, s, w.gates, T, c.n_experts, w.probs));
  CK(k_swiglu(ctx, s, w.sg, w.su, T * c.shared_inter, w.sact));
  uint32_t* inds = inds_out ? inds_out : w.inds;
  CK(k_router_topk(ctx, s, w.probs, T, c.n_experts, c.top_k, inds, w.scores));
  CK(k_gemv(ctx, s, moe.sh_down, w.sact, T, w.sy, 0));
  CK(k_gather_gemv(ctx, s, moe.sw_gate, x, w.lhs, inds, rows, w.eg));
  CK(k_gather_gemv(ctx, s, moe.sw_up, x, w.lhs, inds, rows, w.eu));
  CK(k_swiglu(ctx, s, w.eg, w.eu, rows * c.expert_inter, w.eact));
  CK(k_gather_gemv(ctx, s, moe.sw_down, w.eact, w.ident, inds, rows, w.ey));
  CK(k_moe_combine(ctx, s, w.scores, w.ey, w.gs, w.sy, T, c.top_k, c.hidden, c.norm_topk_prob, out));
  return ORN_OK;
}

// Attention::forward (qwen3_5.rs:430-474) / MtpHead::attention (mtp.rs:219-262)
int attention(orn_model* m, orn_linear* qp, orn_linear* kp, orn_linear* vp, orn_linear* op,
              const bf16_t* q_norm, const bf16_t* k_norm, const bf16_t* x, int T, bf16_t* kc,
              bf16_t* vc, const int* pos, bf16_t* out) {
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  Workspace& w = m->ws;
  const orn_config& c = m->cfg;
  const int Hq = c.n_heads, Hkv = c.n_kv_heads, hd = c.head_dim;
  CK(k_gemv(ctx, s, qp, x, T, w.qg, 0));
  CK(k_gemv(ctx, s, kp, x, T, w.ak, 0));
  CK(k_gemv(ctx, s, vp, x, T, w.av, 0));
  CK(k_split_qgate(ctx, s, w.qg, T, Hq, hd, w.aq, w.agate));
  CK(k_rms_norm(ctx, s, w.aq, q_norm, T * Hq, hd, c.rms_eps, w.aq));
  CK(k_rms_norm(ctx, s, w.ak, k_norm, T * Hkv, hd, c.rms_eps, w.ak));
  CK(k_rope(ctx, s, w.aq, T, Hq, hd, c.rope_dims, m->lnb, pos, 0));
  CK(k_rope(ctx, s, w.ak, T, Hkv, hd, c.rope_dims, m->lnb, pos, 0));
  CK(k_kv_append(ctx, s, w.ak, w.av, T, Hkv, hd, c.max_ctx, pos, 0, kc, vc));
  const float scale = 1.0f / sqrtf((float)hd);
  CK(k_sdpa_decode(ctx, s, w.aq, kc, vc, T, Hq, Hkv, hd, c.max_ctx, pos, 0, scale, w.att));
  CK(k_sigmoid_gate(ctx, s, w.agate, w.att, T * Hq * hd, 1, w.agated));
  CK(k_gemv(ctx, s, op, w.agated, T, out, 0));
  return ORN_OK;
}

// GatedDeltaNet::forward / forward_capture (qwen3_5.rs:478-695).  The layer's
// conv window buffer holds [cached rows 0..S-1 | this call's qkv rows]; the
// qkv projection writes straight into it.
int gdn_layer(orn_model* m, const Layer& ly, const bf16_t* x, int T, bf16_t* conv, float* ring,
              const int* cur, bool capture, bf16_t* out) {
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  Workspace& w = m->ws;
  const orn_config& c = m->cfg;
  const int S = c.gdn_conv_kernel - 1, D = conv_dim(c);
  bf16_t* qkv = conv + (size_t)S * D;
  CK(k_gemv(ctx, s, ly.in_qkv, x, T, qkv, 0));
  CK(k_gemv(ctx, s, ly.in_z, x, T, w.z, 0));
  CK(k_gemv(ctx, s, ly.in_b, x, T, w.bb, 0));
  CK(k_gemv(ctx, s, ly.in_a, x, T, w.aa, 0));
  CK(k_gdn_front(ctx, s, conv, qkv, ly.conv_w, w.aa, w.bb, ly.a_log, ly.dt_bias, T, c.gdn_k_heads,
                 c.gdn_v_heads, c.gdn_head_dim, c.gdn_conv_kernel, 1e-6f, nullptr, w.gq, w.gk, w.gv,
                 w.beta, w.gg, nullptr));
  CK(k_gated_delta_ring(ctx, s, w.gq, w.gk, w.gv, w.gg, w.beta, ring, kRing, cur, capture ? 0 : 1, T,
                        c.gdn_k_heads, c.gdn_v_heads, w.gy));
  CK(k_rms_norm_gated(ctx, s, w.gy, ly.gdn_norm, w.z, T * c.gdn_v_heads, c.gdn_head_dim, c.rms_eps,
                      w.ggated));
  CK(k_gemv(ctx, s, ly.out_proj, w.ggated, T, out, 0));
  return ORN_OK;
}

// commit `keep` of the window's tokens: KV offset, conv windows, and the state
// ring, which moves by one slot per kept snapshot (`ring_step` = keep after a
// capture window, 1 after a call that kept only its final state)
int commit(orn_cache* c, int keep, int ring_step) {
  orn_model* m = c->m;
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  add_int_kernel<<<1, 1, 0, s>>>(c->pos, keep);
  CK(orn_launch_check(ctx, "add_int"));
  add_int_kernel<<<1, 1, 0, s>>>(c->cur, ring_step);
  CK(orn_launch_check(ctx, "add_int"));
  if (c->n_gdn > 0) {
    const int S = m->cfg.gdn_conv_kernel - 1, D = conv_dim(m->cfg);
    dim3 grid((D / 8 + 127) / 128, c->n_gdn);
    conv_shift_kernel<<<grid, 128, 0, s>>>(c->conv_table, S, D, keep);
    CK(orn_launch_check(ctx, "conv_shift"));
  }
  c->h_pos += keep;
  c->h_cur += ring_step;
  return ORN_OK;
}

bool use_fused_env() {
  // ORN_UNFUSED=1 runs the one-kernel-per-op control path (same arithmetic)
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ORN_UNFUSED");
    v = (e && e[0] == '1') ? 0 : 1;
  }
  return v == 1;
}
bool use_fused(const orn_model* m) { return use_fused_env() && m->fused_ok; }
// the fused expert kernels read the four decode formats; gate/up share one, routed and shared down share one
bool moe_fusable(const Moe& e) {
  const orn_linear* all[8] = {e.gate, e.sw_gate, e.sw_up, e.sw_down, e.sh_gate, e.sh_up, e.sh_down, e.sh_egate};
  for (const orn_linear* l : all)
    if (l->kind > ORN_BF16) return false;
  return e.sw_gate->kind == e.sw_up->kind && e.sh_gate->kind == e.sh_up->kind && e.sw_down->kind == e.sh_down->kind;
}

// MoE block from the pre-norm pair (a, b): h = bf(a+b) -> w.h, norm with `nw`,
// router + shared expert + routed experts + combine -> w.mo   (three kernels)
int moe_fused(orn_model* m, const Moe& moe, const bf16_t* a, const bf16_t* b, const bf16_t* nw, int T) {
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  Workspace& w = m->ws;
  const orn_config& c = m->cfg;
  if (!moe_fusable(moe)) {
    // a block with a format outside the fused kernels (affine-4 shared experts of the published
    // q6k-full mix, or routed and shared down projections in different formats): one kernel per op
    if (b != nullptr) CK(k_add_rms_norm(ctx, s, a, b, nw, T, c.hidden, c.rms_eps, w.h, w.normed2));
    else {
      ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(w.h, a, sizeof(bf16_t) * (size_t)T * c.hidden, cudaMemcpyDeviceToDevice, s));
      CK(k_rms_norm(ctx, s, a, nw, T, c.hidden, c.rms_eps, w.normed2));
    }
    return moe_block(m, moe, w.normed2, T, w.mo, nullptr);
  }
  FusedPrologue fp;
  fp.mode = PRO_ADDNORM; fp.K = c.hidden; fp.a = a; fp.b = b; fp.w = nw; fp.sum_out = w.h; fp.norm_out = w.normed2;
  fp.eps = c.rms_eps;
  FusedJob jobs[3];
  jobs[0].lin = moe.gate; jobs[0].out = w.gates;
  jobs[1].lin = moe.sh_gate; jobs[1].lin2 = moe.sh_up; jobs[1].out = w.sact; jobs[1].epi = EPI_SWIGLU;
  jobs[2].lin = moe.sh_egate; jobs[2].out = w.gs;
  CK(f_norm_gemv(ctx, s, T, fp, jobs, 3));
  CK(f_moe_up(ctx, s, T, w.gates, w.normed2, moe.sw_gate, moe.sw_up, c.top_k, w.inds, w.scores, w.eact));
  CK(f_moe_down(ctx, s, T, w.eact, w.sact, w.inds, w.scores, w.gs, moe.sw_down, moe.sh_down, c.top_k,
                c.norm_topk_prob, w.mo));
  return ORN_OK;
}

// The 40 layers.  On return the residual stream is bf(w.h + w.mo), not yet
// added: the add belongs to whatever norm comes next (the final norm here, the
// next layer's input norm inside the loop), as in add_rms_norm (norm.rs).
// the reference switches its attention to a two-pass form from 1024 keys (src/ops/sdpa.rs:166-170); here the
// fused kernel spreads a head's key groups over four CTAs (same bits) from 512 keys, where that form
// starts to win on this part (23.9 -> 22.4 us per launch at 600 keys, 155 -> 74 us at 6600)
// (ORN_LONG_CONTEXT_KEYS moves the threshold, for measurements: 0 = never)
constexpr int kLongContext = 512;
int long_context(int keys) {
  static const int thr = [] {  // set once, thread-safe
    const char* e = getenv("ORN_LONG_CONTEXT_KEYS");
    const int t = e ? atoi(e) : kLongContext;
    return t <= 0 ? 1 << 30 : t;
  }();
  return keys > thr ? 1 : 0;
}

int trunk_layers(orn_model* m, orn_cache* cc, const uint32_t* dev_ids, int T, bool capture) {
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  Workspace& w = m->ws;
  const orn_config& c = m->cfg;
  const int H = c.hidden;
  if (T < 1 || T > kMaxRows) ORN_FAIL(ctx, ORN_ERR_ARG, "forward: 1..4 rows per call");
  if (cc->h_pos + T > c.max_ctx) ORN_FAIL(ctx, ORN_ERR_STATE, "forward: context exceeds max_ctx");
  if (!use_fused(m)) {
    CK(k_embedding(ctx, s, m->embed, dev_ids, T, w.x));
    CK(k_rms_norm(ctx, s, w.x, m->layers[0].input_ln, T, H, c.rms_eps, w.normed));
    for (int i = 0; i < c.n_layers; ++i) {
      const Layer& ly = m->layers[i];
      if (ly.linear) CK(gdn_layer(m, ly, w.normed, T, cc->conv[i], cc->ring[i], cc->cur, capture, w.r));
      else
        CK(attention(m, ly.q_proj, ly.k_proj, ly.v_proj, ly.o_proj, ly.q_norm, ly.k_norm, w.normed, T,
                     cc->kc[i], cc->vc[i], cc->pos, w.r));
      CK(k_add_rms_norm(ctx, s, w.x, w.r, ly.post_ln, T, H, c.rms_eps, w.h, w.normed2));
      CK(moe_block(m, ly.moe, w.normed2, T, w.mo, nullptr));
      if (i + 1 < c.n_layers)
        CK(k_add_rms_norm(ctx, s, w.h, w.mo, m->layers[i + 1].input_ln, T, H, c.rms_eps, w.x, w.normed));
    }
    return ORN_OK;
  }
  const int S = c.gdn_conv_kernel - 1, D = conv_dim(c);
  const int VD = c.gdn_v_heads * c.gdn_head_dim, QD = c.n_heads * c.head_dim;
  CK(k_embedding(ctx, s, m->embed, dev_ids, T, w.memb));
  const bf16_t* pa = w.memb;
  const bf16_t* pb = nullptr;
  for (int i = 0; i < c.n_layers; ++i) {
    const Layer& ly = m->layers[i];
    FusedPrologue fp;
    fp.mode = PRO_ADDNORM; fp.K = H; fp.a = pa; fp.b = pb; fp.w = ly.input_ln; fp.sum_out = w.x; fp.eps = c.rms_eps;
    if (ly.linear) {
      bf16_t* conv = cc->conv[i];
      FusedJob jobs[4];
      jobs[0].lin = ly.in_qkv; jobs[0].out = conv + (size_t)S * D;
      jobs[1].lin = ly.in_z; jobs[1].out = w.z;
      jobs[2].lin = ly.in_b; jobs[2].out = w.bb;
      jobs[3].lin = ly.in_a; jobs[3].out = w.aa;
      CK(f_norm_gemv(ctx, s, T, fp, jobs, 4));
      CK(f_gdn(ctx, s, conv, ly.conv_w, w.aa, w.bb, ly.a_log, ly.dt_bias, cc->ring[i], kRing, cc->cur,
               capture ? 0 : 1, T, c.gdn_k_heads, c.gdn_v_heads, c.gdn_conv_kernel, 1e-6f, w.gy, w.z, ly.gdn_norm,
               c.rms_eps, w.ggated));
      FusedPrologue gp;  // the gated norm is already applied: the projection only loads its rows
      gp.mode = PRO_PLAIN; gp.K = VD; gp.a = w.ggated;
      FusedJob oj;
      oj.lin = ly.out_proj; oj.out = w.r;
      CK(f_norm_gemv(ctx, s, T, gp, &oj, 1));
    } else {
      FusedJob jobs[3];
      jobs[0].lin = ly.q_proj; jobs[0].out = w.qg;
      jobs[1].lin = ly.k_proj; jobs[1].out = w.ak;
      jobs[2].lin = ly.v_proj; jobs[2].out = w.av;
      CK(f_norm_gemv(ctx, s, T, fp, jobs, 3));
      CK(f_attn(ctx, s, w.qg, w.ak, w.av, ly.q_norm, ly.k_norm, cc->kc[i], cc->vc[i], cc->pos, T, c.n_heads,
                c.n_kv_heads, c.head_dim, c.max_ctx, c.rope_dims, m->lnb, c.rms_eps, w.agated, long_context(cc->h_pos + T)));
      FusedPrologue gp;
      gp.mode = PRO_PLAIN; gp.K = QD; gp.a = w.agated;
      FusedJob oj;
      oj.lin = ly.o_proj; oj.out = w.r;
      CK(f_norm_gemv(ctx, s, T, gp, &oj, 1));
    }
    CK(moe_fused(m, ly.moe, w.x, w.r, ly.post_ln, T));
    pa = w.h;
    pb = w.mo;
  }
  return ORN_OK;
}

// The final add + norm, alone or as the prologue of the lm_head mat-vec
// (generate.rs:139-150: `lm_head.matmul(h)`), then the bookkeeping of the call.
int trunk_finish(orn_model* m, orn_cache* cc, int T, bool capture, bf16_t* normed_out, bf16_t* pre_norm_out,
                 const orn_linear* head, bf16_t* logits) {
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  Workspace& w = m->ws;
  const orn_config& c = m->cfg;
  const int H = c.hidden;
  if (head != nullptr && use_fused(m)) {
    FusedPrologue fp;
    fp.mode = PRO_ADDNORM; fp.K = H; fp.a = w.h; fp.b = w.mo; fp.w = m->norm; fp.sum_out = pre_norm_out;
    fp.norm_out = normed_out; fp.eps = c.rms_eps;
    FusedJob j;
    j.lin = head; j.out = logits;
    CK(f_norm_gemv(ctx, s, T, fp, &j, 1));
  } else {
    CK(k_add_rms_norm(ctx, s, w.h, w.mo, m->norm, T, H, c.rms_eps, w.x, w.normed));
    if (normed_out) ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(normed_out, w.normed, sizeof(bf16_t) * (size_t)T * H, cudaMemcpyDeviceToDevice, s));
    if (pre_norm_out) ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(pre_norm_out, w.x, sizeof(bf16_t) * (size_t)T * H, cudaMemcpyDeviceToDevice, s));
    if (head != nullptr) CK(k_gemv(ctx, s, head, w.normed, T, logits, 0));
  }
  if (capture) cc->cap_T = T;
  else CK(commit(cc, T, 1));
  return ORN_OK;
}

// the trunk over T <= kMaxRows rows whose ids are already on the device
int forward_dev(orn_model* m, orn_cache* cc, const uint32_t* dev_ids, int T, bool capture,
                bf16_t* normed_out, bf16_t* pre_norm_out) {
  CK(trunk_layers(m, cc, dev_ids, T, capture));
  return trunk_finish(m, cc, T, capture, normed_out, pre_norm_out, nullptr, nullptr);
}

// trunk + lm_head + greedy for every row: tokens land in dev_tokens, the
// post-norm hidden rows in normed_out
int forward_greedy_dev(orn_model* m, orn_cache* cc, const uint32_t* dev_ids, int T, bool capture,
                       bf16_t* normed_out, uint32_t* dev_tokens) {
  Workspace& w = m->ws;
  CK(trunk_layers(m, cc, dev_ids, T, capture));
  CK(trunk_finish(m, cc, T, capture, normed_out, nullptr, m->lm_head, w.logits));
  return k_greedy(m->ctx, m->ctx->stream, w.logits, T, m->lm_head->O, 1, dev_tokens, w.greedy_scratch);
}

int upload_ids(orn_model* m, const uint32_t* host_ids, int T) {
  ORN_CHECK_CUDA(m->ctx, cudaMemcpyAsync(m->ws.ids, host_ids, sizeof(uint32_t) * (size_t)T,
                                         cudaMemcpyHostToDevice, m->ctx->stream));
  // A copy from pageable memory is staged before the call returns and a pinned buffer of the
  // caller outlives the generate call, which drains the stream before it returns: no wait here.
  return ORN_OK;
}

// MtpHead::hidden / forward (mtp.rs:150-217) for T rows; ids on the device.
// head != null: logits of `head` over the post-norm hidden (the draft chain);
// kv_only: only the head's KV rows are wanted (the Committed re-encode discards
// the hidden, mtp_generate.rs:292-301).
int mtp_step(orn_model* m, orn_cache* cc, const bf16_t* trunk_hidden, const uint32_t* dev_ids, int T,
             const orn_linear* head, bf16_t* hidden_out, bf16_t* logits, bool kv_only) {
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  Workspace& w = m->ws;
  const orn_config& c = m->cfg;
  const Mtp& h = m->mtp;
  const int H = c.hidden;
  if (!h.present) ORN_FAIL(ctx, ORN_ERR_STATE, "mtp: the model has no MTP head");
  if (cc->h_mtp_pos + T > c.max_ctx) ORN_FAIL(ctx, ORN_ERR_STATE, "mtp: context exceeds max_ctx");
  if (!use_fused(m)) {
    CK(k_embedding(ctx, s, m->embed, dev_ids, T, w.memb));
    CK(k_rms_norm(ctx, s, w.memb, h.pre_fc_norm_embedding, T, H, c.rms_eps, w.me));
    CK(k_rms_norm(ctx, s, trunk_hidden, h.pre_fc_norm_hidden, T, H, c.rms_eps, w.mh));
    CK(k_concat2(ctx, s, w.me, w.mh, T, H, w.mjoined));
    CK(k_gemv(ctx, s, h.fc, w.mjoined, T, w.mx, 0));
    CK(k_rms_norm(ctx, s, w.mx, h.input_ln, T, H, c.rms_eps, w.normed));
    CK(attention(m, h.q_proj, h.k_proj, h.v_proj, h.o_proj, h.q_norm, h.k_norm, w.normed, T, cc->mtp_kc,
                 cc->mtp_vc, cc->mtp_pos, w.r));
    CK(k_add(ctx, s, w.mx, w.r, T * H, w.h));
    CK(k_rms_norm(ctx, s, w.h, h.post_ln, T, H, c.rms_eps, w.normed2));
    CK(moe_block(m, h.moe, w.normed2, T, w.mo, nullptr));
    CK(k_add(ctx, s, w.h, w.mo, T * H, w.h));
    CK(k_rms_norm(ctx, s, w.h, h.norm, T, H, c.rms_eps, hidden_out));
    if (head != nullptr) CK(k_gemv(ctx, s, head, hidden_out, T, logits, 0));
  } else {
    const int QD = c.n_heads * c.head_dim;
    FusedPrologue jp;
    jp.mode = PRO_MTPJOIN; jp.K = 2 * H; jp.a = trunk_hidden; jp.w = h.pre_fc_norm_embedding;
    jp.w2 = h.pre_fc_norm_hidden; jp.emb = m->embed; jp.ids = dev_ids; jp.eps = c.rms_eps;
    FusedJob fj;
    fj.lin = h.fc; fj.out = w.mx;
    CK(f_norm_gemv(ctx, s, T, jp, &fj, 1));
    FusedPrologue fp;
    fp.mode = PRO_ADDNORM; fp.K = H; fp.a = w.mx; fp.w = h.input_ln; fp.eps = c.rms_eps;
    FusedJob jobs[3];
    jobs[0].lin = h.q_proj; jobs[0].out = w.qg;
    jobs[1].lin = h.k_proj; jobs[1].out = w.ak;
    jobs[2].lin = h.v_proj; jobs[2].out = w.av;
    CK(f_norm_gemv(ctx, s, T, fp, jobs, 3));
    CK(f_attn(ctx, s, w.qg, w.ak, w.av, h.q_norm, h.k_norm, cc->mtp_kc, cc->mtp_vc, cc->mtp_pos, T, c.n_heads,
              c.n_kv_heads, c.head_dim, c.max_ctx, c.rope_dims, m->lnb, c.rms_eps, w.agated, long_context(cc->h_mtp_pos + T)));
    if (!kv_only) {
      FusedPrologue gp;
      gp.mode = PRO_PLAIN; gp.K = QD; gp.a = w.agated;
      FusedJob oj;
      oj.lin = h.o_proj; oj.out = w.r;
      CK(f_norm_gemv(ctx, s, T, gp, &oj, 1));
      CK(moe_fused(m, h.moe, w.mx, w.r, h.post_ln, T));
      if (head != nullptr) {
        FusedPrologue hp;
        hp.mode = PRO_ADDNORM; hp.K = H; hp.a = w.h; hp.b = w.mo; hp.w = h.norm; hp.norm_out = hidden_out;
        hp.eps = c.rms_eps;
        FusedJob hj;
        hj.lin = head; hj.out = logits;
        CK(f_norm_gemv(ctx, s, T, hp, &hj, 1));
      } else {
        CK(k_add_rms_norm(ctx, s, w.h, w.mo, h.norm, T, H, c.rms_eps, w.x, hidden_out));
      }
    }
  }
  add_int_kernel<<<1, 1, 0, s>>>(cc->mtp_pos, T);
  CK(orn_launch_check(ctx, "add_int"));
  cc->h_mtp_pos += T;
  return ORN_OK;
}

int set_mtp_pos(orn_cache* cc, int v) {
  set_int_kernel<<<1, 1, 0, cc->m->ctx->stream>>>(cc->mtp_pos, v);
  CK(orn_launch_check(cc->m->ctx, "set_int"));
  cc->h_mtp_pos = v;
  return ORN_OK;
}

// lm_head + greedy for T rows; tokens land in dev_tokens
int head_greedy_dev(orn_model* m, const orn_linear* head, const bf16_t* hidden, int T, int normalize,
                    bf16_t* logits, uint32_t* dev_tokens) {
  CK(k_gemv(m->ctx, m->ctx->stream, head, hidden, T, logits, 0));
  return k_greedy(m->ctx, m->ctx->stream, logits, T, head->O, normalize, dev_tokens, m->ws.greedy_scratch);
}

// One speculative cycle on the device: window[0] = primary, `want` draft levels
// (mtp_generate.rs:99-135) with the harness's forced-draft overrides read from the
// mailbox, then the verify forward with every row's greedy target.
int cycle_body(orn_model* m, orn_cache* c, int want, bool use_frspec) {
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  Workspace& w = m->ws;
  const int H = m->cfg.hidden;
  const orn_linear* dlm = use_frspec ? m->fr_head : m->lm_head;
  mailbox_apply_kernel<<<1, 1, 0, s>>>(w.mailbox, w.window, -1);
  CK(orn_launch_check(ctx, "mailbox_apply"));
  const bf16_t* dh_in = w.hrow;
  for (int i = 0; i < want; ++i) {
    bf16_t* dh_out = w.dh + (size_t)(i & 1) * H;
    CK(mtp_step(m, c, dh_in, w.window + i, 1, dlm, dh_out, w.dlogits, false));
    if (use_frspec) {
      CK(k_greedy(ctx, s, w.dlogits, 1, dlm->O, 0, w.local, w.greedy_scratch));
      gather_u32_kernel<<<1, 1, 0, s>>>(m->fr_ids, w.local, w.window + i + 1);
      CK(orn_launch_check(ctx, "gather_u32"));
    } else {
      CK(k_greedy(ctx, s, w.dlogits, 1, dlm->O, 0, w.window + i + 1, w.greedy_scratch));
    }
    mailbox_apply_kernel<<<1, 1, 0, s>>>(w.mailbox, w.window, i);
    CK(orn_launch_check(ctx, "mailbox_apply"));
    dh_in = dh_out;
  }
  return forward_greedy_dev(m, c, w.window, want + 1, true, w.vh, w.targets);
}

// one autoregressive step: the token in targets[0] goes in, its successor comes out
int ar_body(orn_model* m, orn_cache* c) {
  Workspace& w = m->ws;
  return forward_greedy_dev(m, c, w.targets, 1, false, w.vh, w.targets);
}

// Run a step body eagerly the first time a shape is seen, capture it into a CUDA
// graph the second time and replay it afterwards.  The host-side bookkeeping the
// body does (positions, counters) is repeated by hand on a replay.
int run_step(orn_model* m, orn_cache* c, int kind /*0 cycle, 1 ar, 2 prefill rows*/, int want, bool use_frspec) {
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  const int n_rows = want + 1;
  // the launch shape of the fused attention changes once a cache passes kLongContext keys (the key
  // groups of a head spread over four CTAs): such steps are graphs of their own
  const int key = kind * 64 + want * 2 + (use_frspec ? 1 : 0) + 4096 * long_context(c->h_pos + n_rows) +
                  8192 * (kind == 0 ? long_context(c->h_mtp_pos + want) : 0);
  orn_cache::StepGraph& g = c->graphs[key];
  if (c->h_pos + n_rows > m->cfg.max_ctx) ORN_FAIL(ctx, ORN_ERR_STATE, "forward: context exceeds max_ctx");
  if (kind == 0 && c->h_mtp_pos + want > m->cfg.max_ctx) ORN_FAIL(ctx, ORN_ERR_STATE, "mtp: context exceeds max_ctx");
  static int no_graph = -1;
  if (no_graph < 0) { const char* e = getenv("ORN_NO_GRAPH"); no_graph = (e && e[0] == '1') ? 1 : 0; }
  const bool eager = no_graph || ctx->kt != nullptr;  // per-kernel times need eager launches
  if (g.exec != nullptr && use_frspec && g.fr_gen != m->fr_gen) {
    // the pruned head was replaced since this graph was captured: its kernel arguments point at
    // freed memory.  Drop it; the shape is run eagerly once and captured again.
    ORN_CHECK_CUDA(ctx, cudaStreamSynchronize(s));
    cudaGraphExecDestroy(g.exec);
    g = orn_cache::StepGraph();
  }
  if (g.exec != nullptr && !eager) {
    ORN_CHECK_CUDA(ctx, cudaGraphLaunch(g.exec, s));
    ctx->launches += g.launches;
    if (kind == 0) { c->h_mtp_pos += want; c->cap_T = n_rows; }
    else if (kind == 1) { c->h_pos += 1; c->h_cur += 1; }
    else { c->h_pos += n_rows; c->h_cur += 1; }
    return ORN_OK;
  }
  auto body = [&]() {
    if (kind == 0) return cycle_body(m, c, want, use_frspec);
    if (kind == 1) return ar_body(m, c);
    return forward_dev(m, c, m->ws.ids, n_rows, false, nullptr, nullptr);  // a window of prompt rows
  };
  if (g.seen == 0 || eager || !use_fused(m) || g.exec != nullptr) {
    g.seen += 1;
    return body();
  }
  const int64_t l0 = ctx->launches;
  ORN_CHECK_CUDA(ctx, cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
  int rc = body();
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(s, &graph);
  if (rc != ORN_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
  if (e != cudaSuccess) ORN_FAIL(ctx, ORN_ERR_CUDA, std::string("cudaStreamEndCapture: ") + cudaGetErrorString(e));
  e = cudaGraphInstantiate(&g.exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) { g.exec = nullptr; ORN_FAIL(ctx, ORN_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e)); }
  g.launches = ctx->launches - l0;
  g.fr_gen = m->fr_gen;
  // the capture recorded the work without running it; the host bookkeeping it did stands
  ORN_CHECK_CUDA(ctx, cudaGraphLaunch(g.exec, s));
  return ORN_OK;
}

// ------------------------------------------------------------------ prompt chunks on the tensor cores
bool use_wide_prefill() {
  // ORN_NO_WIDE_PREFILL=1 sends every prompt through the row-invariant 4-row windows
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ORN_NO_WIDE_PREFILL");
    v = (e && e[0] == '1') ? 0 : 1;
  }
  return v == 1;
}
// ORN_WIDE_EXACT=1 keeps the chunked prompt path but computes every product with the row-invariant
// mat-vec kernels (groups of four rows; routed rows one by one): the chunk plumbing (conv windows,
// KV append, causal attention over the chunk, the T-step recurrence, the expert sort) then has to
// reproduce the 4-row windows bit for bit, which is how the tests check it
bool wide_exact() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ORN_WIDE_EXACT");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}
// y[T, O] = x[T, K] W^T for a prompt chunk
int wide_mm(orn_model* m, const orn_linear* L, const bf16_t* x, int T, bf16_t* y) {
  orn_ctx* ctx = m->ctx;
  if (!wide_exact()) return f_qgemm(ctx, ctx->stream, L, x, T, y, L->O, nullptr, nullptr);
  for (int r = 0; r < T; r += kMaxRows) {
    const int n = std::min(kMaxRows, T - r);
    CK(k_gemv(ctx, ctx->stream, L, x + (size_t)r * L->K, n, y + (size_t)r * L->O, 0));
  }
  return ORN_OK;
}
constexpr int kWideMinRows = 64;    // measured: below about 60 rows the 4-row mat-vec windows are faster (the
                                    // reference's own crossover, kquant.rs MM_ROW_LIMIT, is 16 on its hardware)
constexpr int kWideMaxRows = 8192;  // widest chunk of the wide path (the reference's default chunk is 2048, generate.rs:25)

int wide_reserve(orn_model* m, int rows) {
  WideWs& w = m->wide;
  if (w.cap >= rows) return ORN_OK;
  for (void* p : w.allocs) cudaFree(p);
  w.allocs.clear();
  w.cap = 0;
  const orn_config& c = m->cfg;
  const size_t R = rows, H = c.hidden, D = conv_dim(c), VD = (size_t)c.gdn_v_heads * c.gdn_head_dim;
  const size_t KD = (size_t)c.gdn_k_heads * c.gdn_head_dim, QD = (size_t)c.n_heads * c.head_dim;
  const size_t KVD = (size_t)c.n_kv_heads * c.head_dim, E = c.n_experts, I = c.expert_inter, SI = c.shared_inter, k = c.top_k;
  const size_t S = c.gdn_conv_kernel - 1;
  int rc = ORN_OK;
  auto A = [&](auto** p, size_t n) {
    if (rc != ORN_OK) return;
    void* d = nullptr;
    rc = orn_alloc(m->ctx, sizeof(**p) * (n ? n : 1), &d);
    if (rc == ORN_OK) { w.allocs.push_back(d); *p = (std::remove_reference_t<decltype(**p)>*)d; }
  };
  A(&w.ids, R); A(&w.lhs, R * k); A(&w.perm, R * k); A(&w.inds, R * k); A(&w.seg, 2 * E + 4);
  A(&w.ident, R * k); A(&w.sorted_e, R * k); A(&w.perm_inv, R * k);
  A(&w.x, R * H); A(&w.n, R * H); A(&w.r, R * H); A(&w.h, R * H); A(&w.n2, R * H); A(&w.mo, R * H);
  A(&w.cb, (S + R) * D); A(&w.z, R * VD); A(&w.a, R * c.gdn_v_heads); A(&w.b, R * c.gdn_v_heads);
  A(&w.gq, R * KD); A(&w.gk, R * KD); A(&w.gv, R * VD); A(&w.beta, R * c.gdn_v_heads); A(&w.gg, R * c.gdn_v_heads);
  A(&w.gy, R * VD); A(&w.gated, R * VD);
  A(&w.qg, R * 2 * QD); A(&w.aq, R * QD); A(&w.agate, R * QD); A(&w.ak, R * KVD); A(&w.av, R * KVD);
  A(&w.att, R * QD); A(&w.agated, R * QD);
  A(&w.gates, R * E); A(&w.probs, R * E); A(&w.scores, R * k); A(&w.sg, R * SI); A(&w.su, R * SI); A(&w.sact, R * SI);
  A(&w.sy, R * H); A(&w.gs, R);
  A(&w.xs, R * k * H); A(&w.eg, R * k * I); A(&w.eu, R * k * I); A(&w.eact, R * k * I); A(&w.ey, R * k * H);
  if (rc == ORN_OK) {
    const size_t big = std::max(qgemm_scratch_bytes((int)(R * k), (int)E, (int)H), qgemm_scratch_bytes((int)(R * k), (int)E, (int)I));
    rc = orn_alloc(m->ctx, big, &w.gemm_scratch);
    if (rc == ORN_OK) w.allocs.push_back(w.gemm_scratch);
    if (rc == ORN_OK) rc = orn_alloc(m->ctx, gdn_chunk_scratch_bytes(rows, c.gdn_v_heads), &w.gdn_scratch);
    if (rc == ORN_OK) w.allocs.push_back(w.gdn_scratch);
  }
  if (rc != ORN_OK) {
    for (void* p : w.allocs) cudaFree(p);
    w.allocs.clear();
    return rc;
  }
  const int n = rows * c.top_k;
  iota_div_kernel<<<(n + 255) / 256, 256, 0, m->ctx->stream>>>(w.lhs, w.ident, n, c.top_k);
  CK(orn_launch_check(m->ctx, "iota_div"));
  w.cap = rows;
  return ORN_OK;
}

// sorted_e[p] = expert of sorted row p; perm_inv[original row] = its sorted position
__global__ void perm_tables_kernel(const uint32_t* perm, const uint32_t* inds, int rows, uint32_t* sorted_e, uint32_t* perm_inv) {
  int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p < rows) {
    const uint32_t o = perm[p];
    sorted_e[p] = inds[o];
    perm_inv[o] = (uint32_t)p;
  }
}
__global__ void copy_u4_kernel(const uint4* src, uint4* dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[i];
}

// sparse_moe_block on a chunk (moe.rs:662-741 with the sorted expert path of :283-314,463-508):
// rows are counting-sorted by expert, an expert's matrices are read once for all its rows
int moe_block_wide(orn_model* m, const Moe& moe, const bf16_t* x, int T, bf16_t* out) {
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  WideWs& w = m->wide;
  const orn_config& c = m->cfg;
  const int rows = T * c.top_k, H = c.hidden, I = c.expert_inter, SI = c.shared_inter, E = c.n_experts;
  CK(wide_mm(m, moe.gate, x, T, w.gates));
  CK(wide_mm(m, moe.sh_gate, x, T, w.sg));
  CK(wide_mm(m, moe.sh_up, x, T, w.su));
  CK(wide_mm(m, moe.sh_egate, x, T, w.gs));
  CK(k_softmax_precise(ctx, s, w.gates, T, E, w.probs));
  CK(k_swiglu(ctx, s, w.sg, w.su, T * SI, w.sact));
  CK(k_router_topk(ctx, s, w.probs, T, E, c.top_k, w.inds, w.scores));
  CK(wide_mm(m, moe.sh_down, w.sact, T, w.sy));
  CK(f_route_sort(ctx, s, w.inds, rows, E, w.seg, w.seg + E + 1, w.perm));
  CK(f_gather_rows(ctx, s, x, w.lhs, w.perm, rows, H, w.xs));
  if (wide_exact()) {
    perm_tables_kernel<<<(rows + 255) / 256, 256, 0, s>>>(w.perm, w.inds, rows, w.sorted_e, w.perm_inv);
    CK(orn_launch_check(ctx, "perm_tables"));
  }
  if (wide_exact()) {
    // the routed rows through the row-invariant gather mat-vec, in sorted order like the products below
    CK(k_gather_gemv(ctx, s, moe.sw_gate, w.xs, w.ident, w.sorted_e, rows, w.eg));
    CK(k_gather_gemv(ctx, s, moe.sw_up, w.xs, w.ident, w.sorted_e, rows, w.eu));
    CK(k_swiglu(ctx, s, w.eg, w.eu, rows * I, w.eact));
    CK(k_gather_gemv(ctx, s, moe.sw_down, w.eact, w.perm_inv, w.inds, rows, w.ey));
  } else {
    QGemmGroup sorted{w.seg, nullptr, 0}, back{w.seg, w.perm, 0};
    CK(f_qgemm(ctx, s, moe.sw_gate, w.xs, rows, w.eg, I, &sorted, w.gemm_scratch));
    CK(f_qgemm(ctx, s, moe.sw_up, w.xs, rows, w.eu, I, &sorted, w.gemm_scratch));
    CK(k_swiglu(ctx, s, w.eg, w.eu, rows * I, w.eact));
    CK(f_qgemm(ctx, s, moe.sw_down, w.eact, rows, w.ey, H, &back, w.gemm_scratch));  // rows back in (token, slot) order
  }
  CK(k_moe_combine(ctx, s, w.scores, w.ey, w.gs, w.sy, T, c.top_k, H, c.norm_topk_prob, out));
  return ORN_OK;
}

// One prompt chunk of T rows (ids on the device in wide.ids) through the trunk: the layer
// sequence of TextModel::forward_hidden (qwen3_5.rs:578-695) with every projection as one wide
// product.  Only the caches matter (generate::prefill discards the hidden rows, generate.rs:90-136).
int prefill_wide(orn_model* m, orn_cache* cc, int T, bf16_t* normed_out /*nullable: [T, H] rows after the final norm*/) {
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  WideWs& w = m->wide;
  const orn_config& c = m->cfg;
  const int H = c.hidden, S = c.gdn_conv_kernel - 1, D = conv_dim(c);
  const int VD = c.gdn_v_heads * c.gdn_head_dim, QD = c.n_heads * c.head_dim, KVD = c.n_kv_heads * c.head_dim;
  const int Hq = c.n_heads, Hkv = c.n_kv_heads, hd = c.head_dim;
  if (cc->h_pos + T > c.max_ctx) ORN_FAIL(ctx, ORN_ERR_STATE, "forward: context exceeds max_ctx");
  CK(k_embedding(ctx, s, m->embed, w.ids, T, w.x));
  CK(k_rms_norm(ctx, s, w.x, m->layers[0].input_ln, T, H, c.rms_eps, w.n));
  for (int i = 0; i < c.n_layers; ++i) {
    const Layer& ly = m->layers[i];
    if (ly.linear) {
      // conv window of the chunk: the cached rows, then this chunk's qkv rows (written by the product)
      const size_t n16 = (size_t)S * D / 8;
      copy_u4_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, s>>>(reinterpret_cast<const uint4*>(cc->conv[i]),
                                                                 reinterpret_cast<uint4*>(w.cb), n16);
      CK(orn_launch_check(ctx, "copy_u4"));
      bf16_t* qkv = w.cb + (size_t)S * D;
      CK(wide_mm(m, ly.in_qkv, w.n, T, qkv));
      CK(wide_mm(m, ly.in_z, w.n, T, w.z));
      CK(wide_mm(m, ly.in_b, w.n, T, w.b));
      CK(wide_mm(m, ly.in_a, w.n, T, w.a));
      CK(k_gdn_front(ctx, s, w.cb, qkv, ly.conv_w, w.a, w.b, ly.a_log, ly.dt_bias, T, c.gdn_k_heads, c.gdn_v_heads,
                     c.gdn_head_dim, c.gdn_conv_kernel, 1e-6f, cc->conv[i], w.gq, w.gk, w.gv, w.beta, w.gg, nullptr));
      if (wide_exact())  // token by token, the decode path's arithmetic
        CK(k_gated_delta_ring(ctx, s, w.gq, w.gk, w.gv, w.gg, w.beta, cc->ring[i], kRing, cc->cur, 1, T, c.gdn_k_heads,
                              c.gdn_v_heads, w.gy));
      else  // chunkwise on the tensor cores; the state after the chunk's last token goes to ring slot cur + 1
        CK(k_gated_delta_chunked(ctx, s, w.gq, w.gk, w.gv, w.gg, w.beta, nullptr, cc->ring[i], kRing, cc->cur, T, c.gdn_k_heads,
                                 c.gdn_v_heads, w.gy, w.gdn_scratch));
      CK(k_rms_norm_gated(ctx, s, w.gy, ly.gdn_norm, w.z, T * c.gdn_v_heads, c.gdn_head_dim, c.rms_eps, w.gated));
      CK(wide_mm(m, ly.out_proj, w.gated, T, w.r));
    } else {
      CK(wide_mm(m, ly.q_proj, w.n, T, w.qg));
      CK(wide_mm(m, ly.k_proj, w.n, T, w.ak));
      CK(wide_mm(m, ly.v_proj, w.n, T, w.av));
      CK(k_split_qgate(ctx, s, w.qg, T, Hq, hd, w.aq, w.agate));
      CK(k_rms_norm(ctx, s, w.aq, ly.q_norm, T * Hq, hd, c.rms_eps, w.aq));
      CK(k_rms_norm(ctx, s, w.ak, ly.k_norm, T * Hkv, hd, c.rms_eps, w.ak));
      CK(k_rope(ctx, s, w.aq, T, Hq, hd, c.rope_dims, m->lnb, cc->pos, 0));
      CK(k_rope(ctx, s, w.ak, T, Hkv, hd, c.rope_dims, m->lnb, cc->pos, 0));
      CK(k_kv_append(ctx, s, w.ak, w.av, T, Hkv, hd, c.max_ctx, cc->pos, 0, cc->kc[i], cc->vc[i]));
      if (wide_exact() || hd != 256)  // the row-invariant kernel: one pass over the cache per (head, row)
        CK(k_sdpa_decode(ctx, s, w.aq, cc->kc[i], cc->vc[i], T, Hq, Hkv, hd, c.max_ctx, cc->pos, 0, 1.0f / sqrtf((float)hd),
                         w.att));
      else
        CK(k_flash_prefill(ctx, s, w.aq, cc->kc[i], cc->vc[i], T, Hq, Hkv, hd, c.max_ctx, cc->pos, 1.0f / sqrtf((float)hd), w.att));
      CK(k_sigmoid_gate(ctx, s, w.agate, w.att, T * Hq * hd, 1, w.agated));
      CK(wide_mm(m, ly.o_proj, w.agated, T, w.r));
    }
    CK(k_add_rms_norm(ctx, s, w.x, w.r, ly.post_ln, T, H, c.rms_eps, w.h, w.n2));
    CK(moe_block_wide(m, ly.moe, w.n2, T, w.mo));
    if (i + 1 < c.n_layers) CK(k_add_rms_norm(ctx, s, w.h, w.mo, m->layers[i + 1].input_ln, T, H, c.rms_eps, w.x, w.n));
  }
  if (normed_out != nullptr) CK(k_add_rms_norm(ctx, s, w.h, w.mo, m->norm, T, H, c.rms_eps, w.x, normed_out));
  // bookkeeping of a call that keeps only its final state: the conv windows were written in place
  add_int_kernel<<<1, 1, 0, s>>>(cc->pos, T);
  CK(orn_launch_check(ctx, "add_int"));
  add_int_kernel<<<1, 1, 0, s>>>(cc->cur, 1);
  CK(orn_launch_check(ctx, "add_int"));
  cc->h_pos += T;
  cc->h_cur += 1;
  return ORN_OK;
}

// generate::prefill (src/generate.rs:90-136): everything but the last prompt
// token.  Rows are computed with one-row arithmetic, so the chunk width (the
// reference's prefill_step) cannot change the result; chunks are cut to the
// widest window a forward call takes.
int prefill(orn_model* m, orn_cache* cc, const uint32_t* prompt, int n, int prefill_step, int* done_out,
            bf16_t* normed_out = nullptr, int keep_last = 1) {
  int done = 0;
  int step = prefill_step < 1 ? 1 : prefill_step;
  while (n - done > keep_last) {
    int chunk = std::min(step, n - done - keep_last);
    int off = 0;
    if (chunk >= kWideMinRows && use_wide_prefill() && use_fused_env()) {
      // a chunk wide enough for the tensor cores (the reference's tile path, kquant.rs:783-812)
      chunk = std::min(chunk, kWideMaxRows);
      CK(wide_reserve(m, chunk));
      ORN_CHECK_CUDA(m->ctx, cudaMemcpyAsync(m->wide.ids, prompt + done, sizeof(uint32_t) * (size_t)chunk,
                                             cudaMemcpyHostToDevice, m->ctx->stream));
      CK(prefill_wide(m, cc, chunk, normed_out ? normed_out + (size_t)done * m->cfg.hidden : nullptr));
      off = chunk;
    }
    while (off < chunk) {
      int t = std::min(kMaxRows, chunk - off);
      CK(upload_ids(m, prompt + done + off, t));
      if (normed_out != nullptr)
        CK(forward_dev(m, cc, m->ws.ids, t, false, normed_out + (size_t)(done + off) * m->cfg.hidden, nullptr));
      else
        CK(run_step(m, cc, 2, t - 1, false));  // the same rows as forward_dev, replayed as a graph
      off += t;
    }
    CK(orn_sync(m->ctx));  // the reference drains the queue after each chunk (generate.rs:128-131)
    done += chunk;
  }
  *done_out = done;
  return ORN_OK;
}

uint64_t splitmix64(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

}  // namespace

int orn_model_finalize(orn_model* m) { return finalize(m); }
bool orn_wide_exact() { return wide_exact(); }
int orn_conv_dim(const orn_config& c) { return conv_dim(c); }

extern "C" {

int32_t orn_model_create(orn_ctx* ctx, const orn_config* cfg, orn_model** out) {
  if (!ctx || !cfg || !out) return ORN_ERR_ARG;
  *out = nullptr;
  if (cfg->hidden % 256 || cfg->gdn_head_dim != 128 || cfg->head_dim != 256 || cfg->n_layers < 1 ||
      cfg->full_attn_interval < 1 || cfg->top_k < 1 || cfg->top_k > cfg->n_experts ||
      cfg->n_experts > 512 || cfg->n_heads % cfg->n_kv_heads || cfg->gdn_v_heads % cfg->gdn_k_heads ||
      cfg->expert_inter % 256 || cfg->shared_inter % 256 || cfg->max_ctx < 8 || cfg->vocab < 1 ||
      cfg->rope_dims > cfg->head_dim || cfg->rope_dims % 2 || cfg->gdn_conv_kernel < 2)
    ORN_FAIL(ctx, ORN_ERR_ARG, "model_create: unsupported dimensions");
  orn_model* m = new orn_model();
  m->ctx = ctx;
  m->cfg = *cfg;
  *out = m;
  return ORN_OK;
}

int32_t orn_model_destroy(orn_model* m) {
  if (!m) return ORN_OK;
  cudaStreamSynchronize(m->ctx->stream);
  for (auto& kv : m->lins) orn_linear_destroy(m->ctx, kv.second);
  for (auto& kv : m->tensors) cudaFree(kv.second.p);
  for (void* p : m->ws_allocs) cudaFree(p);
  for (void* p : m->wide.allocs) cudaFree(p);
  if (m->fr_head) orn_linear_destroy(m->ctx, m->fr_head);
  cudaFree(m->fr_ids);
  for (int i = 0; i < 4; ++i)
    if (m->ev[i]) cudaEventDestroy(m->ev[i]);
  delete m;
  return ORN_OK;
}

int32_t orn_model_set_linear(orn_model* m, const char* name, orn_linear* lin) {
  if (!m || !name || !lin) return ORN_ERR_ARG;
  if (m->finalized) ORN_FAIL(m->ctx, ORN_ERR_STATE, "model_set_linear: model already in use");
  std::string n = canon(name);
  auto it = m->lins.find(n);
  if (it != m->lins.end()) orn_linear_destroy(m->ctx, it->second);
  m->lins[n] = lin;
  return ORN_OK;
}

int32_t orn_model_set_tensor(orn_model* m, const char* name, const uint16_t* host, size_t n) {
  if (!m || !name || !host || n == 0) return ORN_ERR_ARG;
  if (m->finalized) ORN_FAIL(m->ctx, ORN_ERR_STATE, "model_set_tensor: model already in use");
  void* d = nullptr;
  CK(orn_alloc(m->ctx, n * sizeof(uint16_t), &d));
  int rc = orn_upload(m->ctx, d, host, n * sizeof(uint16_t));
  if (rc != ORN_OK) { cudaFree(d); return rc; }
  std::string cn = canon(name);
  auto it = m->tensors.find(cn);
  if (it != m->tensors.end()) cudaFree(it->second.p);
  m->tensors[cn] = Tensor{(bf16_t*)d, n};
  return ORN_OK;
}

int32_t orn_model_get_linear(orn_model* m, const char* name, const orn_linear** out) {
  if (!m || !name || !out) return ORN_ERR_ARG;
  orn_linear* l = find_lin(m, canon(name));
  if (!l) ORN_FAIL(m->ctx, ORN_ERR_ARG, std::string("model_get_linear: no weight ") + name);
  *out = l;
  return ORN_OK;
}

int32_t orn_model_get_tensor(orn_model* m, const char* name, const uint16_t** dev_out, size_t* n) {
  if (!m || !name || !dev_out || !n) return ORN_ERR_ARG;
  auto it = m->tensors.find(canon(name));
  if (it == m->tensors.end()) ORN_FAIL(m->ctx, ORN_ERR_ARG, std::string("model_get_tensor: no tensor ") + name);
  *dev_out = it->second.p;
  *n = it->second.n;
  return ORN_OK;
}

int32_t orn_model_config(const orn_model* m, orn_config* out) {
  if (!m || !out) return ORN_ERR_ARG;
  *out = m->cfg;
  return ORN_OK;
}

size_t orn_model_weight_bytes(const orn_model* m) {
  size_t total = 0;
  if (!m) return 0;
  for (auto& kv : m->lins) total += kv.second->w_bytes;
  for (auto& kv : m->tensors) total += kv.second.n * 2;
  return total;
}

// Random-init in the mix the benchmark names: expert gate/up Q4_K, expert down
// Q6_K (shared expert: the same formats), every other matrix 8-bit affine, the
// small gated-delta projections and the whole MTP head bf16.
int32_t orn_model_init_random(orn_model* m, uint64_t seed) {
  if (!m) return ORN_ERR_ARG;
  if (m->finalized) ORN_FAIL(m->ctx, ORN_ERR_STATE, "model_init_random: model already in use");
  orn_ctx* ctx = m->ctx;
  const orn_config& c = m->cfg;
  const int H = c.hidden, D = conv_dim(c), VD = c.gdn_v_heads * c.gdn_head_dim;
  const int QD = c.n_heads * c.head_dim, KVD = c.n_kv_heads * c.head_dim;
  uint64_t counter = 0;
  auto lin = [&](const std::string& name, int kind, int E, int O, int K) -> int {
    orn_linear* L = nullptr;
    CK(orn_linear_create_random(ctx, kind, E, O, K, splitmix64(seed + (++counter)), 0.02f, &L));
    return orn_model_set_linear(m, name.c_str(), L);
  };
  auto ten = [&](const std::string& name, size_t n, float mean, float std) -> int {
    void* d = nullptr;
    CK(orn_alloc(ctx, n * 2, &d));
    int rc = k_fill_bf16(ctx, ctx->stream, (bf16_t*)d, n, splitmix64(seed + (++counter)), mean, std);
    if (rc != ORN_OK) { cudaFree(d); return rc; }
    std::string cn = canon(name.c_str());
    auto it = m->tensors.find(cn);
    if (it != m->tensors.end()) cudaFree(it->second.p);
    m->tensors[cn] = Tensor{(bf16_t*)d, n};
    return ORN_OK;
  };
  auto moe = [&](const std::string& p, bool dense) -> int {
    CK(lin(p + "gate", dense ? ORN_BF16 : ORN_A8, 1, c.n_experts, H));
    CK(lin(p + "switch_mlp.gate_proj", dense ? ORN_BF16 : ORN_Q4K, c.n_experts, c.expert_inter, H));
    CK(lin(p + "switch_mlp.up_proj", dense ? ORN_BF16 : ORN_Q4K, c.n_experts, c.expert_inter, H));
    CK(lin(p + "switch_mlp.down_proj", dense ? ORN_BF16 : ORN_Q6K, c.n_experts, H, c.expert_inter));
    CK(lin(p + "shared_expert.gate_proj", dense ? ORN_BF16 : ORN_Q4K, 1, c.shared_inter, H));
    CK(lin(p + "shared_expert.up_proj", dense ? ORN_BF16 : ORN_Q4K, 1, c.shared_inter, H));
    CK(lin(p + "shared_expert.down_proj", dense ? ORN_BF16 : ORN_Q6K, 1, H, c.shared_inter));
    CK(lin(p + "shared_expert_gate", dense ? ORN_BF16 : ORN_A8, 1, 1, H));
    return ORN_OK;
  };
  CK(lin("embed_tokens", ORN_A8, 1, c.vocab, H));
  CK(lin("lm_head", ORN_A8, 1, c.vocab, H));
  CK(ten("norm.weight", H, 1.0f, 0.05f));
  for (int i = 0; i < c.n_layers; ++i) {
    std::string lp = "layers." + std::to_string(i) + ".";
    CK(ten(lp + "input_layernorm.weight", H, 1.0f, 0.05f));
    CK(ten(lp + "post_attention_layernorm.weight", H, 1.0f, 0.05f));
    if (is_linear_layer(c, i)) {
      std::string a = lp + "linear_attn.";
      CK(lin(a + "in_proj_qkv", ORN_A8, 1, D, H));
      CK(lin(a + "in_proj_z", ORN_A8, 1, VD, H));
      CK(lin(a + "in_proj_a.weight", ORN_BF16, 1, c.gdn_v_heads, H));
      CK(lin(a + "in_proj_b.weight", ORN_BF16, 1, c.gdn_v_heads, H));
      CK(lin(a + "out_proj", ORN_A8, 1, H, VD));
      CK(ten(a + "conv1d.weight", (size_t)D * c.gdn_conv_kernel, 0.0f, 0.2f));
      CK(ten(a + "dt_bias", c.gdn_v_heads, 0.0f, 0.3f));
      CK(ten(a + "A_log", c.gdn_v_heads, 0.0f, 0.3f));
      CK(ten(a + "norm.weight", c.gdn_head_dim, 1.0f, 0.05f));
    } else {
      std::string a = lp + "self_attn.";
      CK(lin(a + "q_proj", ORN_A8, 1, 2 * QD, H));
      CK(lin(a + "k_proj", ORN_A8, 1, KVD, H));
      CK(lin(a + "v_proj", ORN_A8, 1, KVD, H));
      CK(lin(a + "o_proj", ORN_A8, 1, H, QD));
      CK(ten(a + "q_norm.weight", c.head_dim, 1.0f, 0.05f));
      CK(ten(a + "k_norm.weight", c.head_dim, 1.0f, 0.05f));
    }
    CK(moe(lp + "mlp.", false));
  }
  {
    std::string lp = "mtp.layers.0.";
    CK(ten("mtp.pre_fc_norm_embedding.weight", H, 1.0f, 0.05f));
    CK(ten("mtp.pre_fc_norm_hidden.weight", H, 1.0f, 0.05f));
    CK(lin("mtp.fc.weight", ORN_BF16, 1, H, 2 * H));
    CK(ten("mtp.norm.weight", H, 1.0f, 0.05f));
    CK(ten(lp + "input_layernorm.weight", H, 1.0f, 0.05f));
    CK(ten(lp + "post_attention_layernorm.weight", H, 1.0f, 0.05f));
    CK(lin(lp + "self_attn.q_proj.weight", ORN_BF16, 1, 2 * QD, H));
    CK(lin(lp + "self_attn.k_proj.weight", ORN_BF16, 1, KVD, H));
    CK(lin(lp + "self_attn.v_proj.weight", ORN_BF16, 1, KVD, H));
    CK(lin(lp + "self_attn.o_proj.weight", ORN_BF16, 1, H, QD));
    CK(ten(lp + "self_attn.q_norm.weight", c.head_dim, 1.0f, 0.05f));
    CK(ten(lp + "self_attn.k_norm.weight", c.head_dim, 1.0f, 0.05f));
    CK(moe(lp + "mlp.", true));
  }
  return orn_sync(ctx);
}

int32_t orn_frspec_set(orn_model* m, const uint32_t* host_ids, int32_t n) {
  if (!m || !host_ids || n < 1) return ORN_ERR_ARG;
  CK(finalize(m));
  // FrSpec::load validation (src/frspec.rs:78-100): in range and unique
  std::vector<uint8_t> seen((size_t)m->cfg.vocab, 0);
  for (int i = 0; i < n; ++i) {
    if (host_ids[i] >= (uint32_t)m->cfg.vocab) ORN_FAIL(m->ctx, ORN_ERR_ARG, "frspec: id out of range");
    if (seen[host_ids[i]]) ORN_FAIL(m->ctx, ORN_ERR_ARG, "frspec: duplicate id");
    seen[host_ids[i]] = 1;
  }
  ORN_CHECK_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));  // nothing may still read the old head
  m->fr_gen += 1;
  if (m->fr_head) { orn_linear_destroy(m->ctx, m->fr_head); m->fr_head = nullptr; }
  cudaFree(m->fr_ids); m->fr_ids = nullptr;
  CK(orn_linear_gather_rows(m->ctx, m->lm_head, host_ids, n, &m->fr_head));
  CK(orn_alloc(m->ctx, sizeof(uint32_t) * (size_t)n, (void**)&m->fr_ids));
  CK(orn_upload(m->ctx, m->fr_ids, host_ids, sizeof(uint32_t) * (size_t)n));
  m->fr_n = n;
  return ORN_OK;
}

int32_t orn_frspec_load(orn_model* m, const char* ids_path) {
  if (!m || !ids_path) return ORN_ERR_ARG;
  FILE* f = fopen(ids_path, "rb");
  if (!f) ORN_FAIL(m->ctx, ORN_ERR_IO, std::string("frspec: cannot open ") + ids_path);
  uint32_t n = 0;
  std::vector<uint32_t> ids;
  bool ok = fread(&n, 4, 1, f) == 1 && n >= 1 && n <= (uint32_t)m->cfg.vocab;
  if (ok) {
    ids.resize(n);
    ok = fread(ids.data(), 4, n, f) == n;
  }
  fclose(f);
  if (!ok) ORN_FAIL(m->ctx, ORN_ERR_IO, std::string("frspec: malformed id file ") + ids_path);
  return orn_frspec_set(m, ids.data(), (int)n);
}

// ------------------------------------------------------------------ caches
int32_t orn_cache_create(orn_model* m, orn_cache** out) {
  if (!m || !out) return ORN_ERR_ARG;
  *out = nullptr;
  CK(finalize(m));
  const orn_config& c = m->cfg;
  orn_cache* k = new orn_cache();
  k->m = m;
  k->kc.assign(c.n_layers, nullptr); k->vc.assign(c.n_layers, nullptr);
  k->conv.assign(c.n_layers, nullptr); k->ring.assign(c.n_layers, nullptr);
  const size_t kvsz = sizeof(bf16_t) * (size_t)c.n_kv_heads * c.max_ctx * c.head_dim;
  const size_t ssz = sizeof(float) * (size_t)c.gdn_v_heads * 128 * 128;
  const size_t csz = sizeof(bf16_t) * (size_t)(c.gdn_conv_kernel - 1 + kMaxRows) * conv_dim(c);
  int rc = ORN_OK;
  std::vector<bf16_t*> table;
  for (int i = 0; i < c.n_layers && rc == ORN_OK; ++i) {
    if (m->layers[i].linear) {
      rc = orn_alloc(m->ctx, csz, (void**)&k->conv[i]);
      if (rc == ORN_OK) rc = orn_alloc(m->ctx, ssz * kRing, (void**)&k->ring[i]);
      table.push_back(k->conv[i]);
    } else {
      rc = orn_alloc(m->ctx, kvsz, (void**)&k->kc[i]);
      if (rc == ORN_OK) rc = orn_alloc(m->ctx, kvsz, (void**)&k->vc[i]);
    }
  }
  if (rc == ORN_OK) rc = orn_alloc(m->ctx, kvsz, (void**)&k->mtp_kc);
  if (rc == ORN_OK) rc = orn_alloc(m->ctx, kvsz, (void**)&k->mtp_vc);
  if (rc == ORN_OK) rc = orn_alloc(m->ctx, 3 * sizeof(int), (void**)&k->pos);
  k->n_gdn = (int)table.size();
  if (rc == ORN_OK && k->n_gdn) {
    rc = orn_alloc(m->ctx, sizeof(bf16_t*) * table.size(), (void**)&k->conv_table);
    if (rc == ORN_OK) rc = orn_upload(m->ctx, k->conv_table, table.data(), sizeof(bf16_t*) * table.size());
  }
  if (rc != ORN_OK) { orn_cache_destroy(k); return rc; }
  if (cudaMallocHost((void**)&k->mailbox_h, 16 * sizeof(uint32_t)) != cudaSuccess) {
    orn_cache_destroy(k);
    ORN_FAIL(m->ctx, ORN_ERR_ALLOC, "cache_create: pinned mailbox");
  }
  k->cur = k->pos + 1;
  k->mtp_pos = k->pos + 2;
  *out = k;
  return orn_cache_reset(k);
}

int32_t orn_cache_destroy(orn_cache* k) {
  if (!k) return ORN_OK;
  cudaStreamSynchronize(k->m->ctx->stream);
  for (auto p : k->kc) cudaFree(p);
  for (auto p : k->vc) cudaFree(p);
  for (auto p : k->conv) cudaFree(p);
  for (auto p : k->ring) cudaFree(p);
  cudaFree(k->mtp_kc); cudaFree(k->mtp_vc); cudaFree(k->pos); cudaFree(k->conv_table);
  for (auto& g : k->graphs)
    if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
  if (k->mailbox_h) cudaFreeHost(k->mailbox_h);
  delete k;
  return ORN_OK;
}

// make_cache (cache.rs:160-181): zero conv windows and states, empty KV
int32_t orn_cache_reset(orn_cache* k) {
  if (!k) return ORN_ERR_ARG;
  orn_model* m = k->m;
  const orn_config& c = m->cfg;
  const size_t ssz = sizeof(float) * (size_t)c.gdn_v_heads * 128 * 128;
  const size_t csz = sizeof(bf16_t) * (size_t)(c.gdn_conv_kernel - 1 + kMaxRows) * conv_dim(c);
  for (int i = 0; i < c.n_layers; ++i)
    if (m->layers[i].linear) {
      CK(orn_memset(m->ctx, k->conv[i], 0, csz));
      CK(orn_memset(m->ctx, k->ring[i], 0, ssz * kRing));
    }
  CK(orn_memset(m->ctx, k->pos, 0, 3 * sizeof(int)));
  k->h_pos = k->h_cur = k->h_mtp_pos = 0;
  k->cap_T = 0;
  return orn_sync(m->ctx);
}

int32_t orn_cache_offset(const orn_cache* c) { return c ? c->h_pos : ORN_ERR_ARG; }

int32_t orn_forward(orn_model* m, orn_cache* c, const uint32_t* host_ids, int32_t T,
                    uint16_t* dev_normed, uint16_t* dev_pre_norm) {
  if (!m || !c || !host_ids) return ORN_ERR_ARG;
  CK(finalize(m));
  if (T < 1 || T > kMaxRows) ORN_FAIL(m->ctx, ORN_ERR_ARG, "forward: 1..4 rows per call");
  CK(upload_ids(m, host_ids, T));
  return forward_dev(m, c, m->ws.ids, T, false, dev_normed, dev_pre_norm);
}

int32_t orn_forward_capture(orn_model* m, orn_cache* c, const uint32_t* host_ids, int32_t T,
                            uint16_t* dev_normed) {
  if (!m || !c || !host_ids) return ORN_ERR_ARG;
  CK(finalize(m));
  if (T < 1 || T > kMaxRows) ORN_FAIL(m->ctx, ORN_ERR_ARG, "forward_capture: 1..4 rows per call");
  CK(upload_ids(m, host_ids, T));
  return forward_dev(m, c, m->ws.ids, T, true, dev_normed, nullptr);
}

int32_t orn_prefill(orn_model* m, orn_cache* c, const uint32_t* host_ids, int32_t n, int32_t prefill_step,
                    uint16_t* dev_normed) {
  if (!m || !c || !host_ids || n < 1) return ORN_ERR_ARG;
  CK(finalize(m));
  int done = 0;
  CK(prefill(m, c, host_ids, n, prefill_step, &done, dev_normed, 0));
  return orn_sync(m->ctx);
}

int32_t orn_cache_rewind(orn_cache* c, int32_t keep) {
  if (!c) return ORN_ERR_ARG;
  if (c->cap_T == 0) ORN_FAIL(c->m->ctx, ORN_ERR_STATE, "cache_rewind: no captured window");
  if (keep < 1 || keep > c->cap_T) ORN_FAIL(c->m->ctx, ORN_ERR_ARG, "cache_rewind: keep out of range");
  c->cap_T = 0;
  return commit(c, keep, keep);
}

int32_t orn_head_greedy(orn_model* m, const uint16_t* dev_hidden, int32_t T, uint32_t* host_tokens,
                        uint16_t* dev_logits_out) {
  if (!m || !dev_hidden || !host_tokens) return ORN_ERR_ARG;
  CK(finalize(m));
  if (T < 1 || T > kMaxRows) ORN_FAIL(m->ctx, ORN_ERR_ARG, "head_greedy: 1..4 rows per call");
  bf16_t* logits = dev_logits_out ? dev_logits_out : m->ws.logits;
  CK(head_greedy_dev(m, m->lm_head, dev_hidden, T, 1, logits, m->ws.targets));
  return orn_download(m->ctx, host_tokens, m->ws.targets, sizeof(uint32_t) * (size_t)T);
}

int32_t orn_generate_step(orn_model* m, orn_cache* c, const uint32_t* prompt, int32_t n_prompt,
                          int32_t max_tokens, int32_t prefill_step, orn_token_cb on_token, void* user) {
  if (!m || !c || !prompt || !on_token) return ORN_ERR_ARG;
  CK(finalize(m));
  if (n_prompt < 1) ORN_FAIL(m->ctx, ORN_ERR_ARG, "generate_step needs a prompt");
  orn_ctx* ctx = m->ctx;
  Workspace& w = m->ws;
  m->prof = orn_prof{};
  const int64_t launches0 = ctx->launches;
  cudaEventRecord(m->ev[2], ctx->stream);
  int done = 0;
  CK(prefill(m, c, prompt, n_prompt, prefill_step, &done));
  cudaEventRecord(m->ev[3], ctx->stream);
  uint32_t y = 0;
  // step (generate.rs:139-150) on the last prompt token
  CK(upload_ids(m, prompt + done, 1));
  CK(forward_greedy_dev(m, c, w.ids, 1, false, w.vh, w.targets));
  CK(orn_download(ctx, &y, w.targets, 4));
  {
    float ms = 0.f;
    cudaEventElapsedTime(&ms, m->ev[2], m->ev[3]);
    m->prof.prefill_ms = ms;
  }
  cudaEventRecord(m->ev[2], ctx->stream);
  int n = 0;
  while (n != max_tokens) {
    // the next step is taken before the token is handed out (generate.rs:195-205);
    // the sampled token stays on the device and feeds the next forward directly
    CK(run_step(m, c, 1, 0, false));
    uint32_t next = 0;
    CK(orn_download(ctx, &next, w.targets, 4));
    m->prof.ar_steps += 1;
    n += 1;
    if (!on_token(y, user)) break;
    y = next;
  }
  cudaEventRecord(m->ev[3], ctx->stream);
  CK(orn_sync(ctx));
  {
    float ms = 0.f;
    cudaEventElapsedTime(&ms, m->ev[2], m->ev[3]);
    m->prof.total_ms = ms;
    m->prof.verify_ms = ms;
  }
  m->prof.kernel_launches = ctx->launches - launches0;
  return ORN_OK;
}

int32_t orn_generate_step_mtp(orn_model* m, orn_cache* c, const uint32_t* prompt, int32_t n_prompt,
                              int32_t depth, int32_t max_tokens, int32_t prefill_step, int32_t policy,
                              int32_t use_frspec, const orn_force_draft* force, orn_token_cb on_token,
                              void* user, orn_mtp_stats* stats) {
  if (!m || !c || !prompt || !on_token || !stats) return ORN_ERR_ARG;
  CK(finalize(m));
  orn_ctx* ctx = m->ctx;
  cudaStream_t s = ctx->stream;
  Workspace& w = m->ws;
  const int H = m->cfg.hidden;
  memset(stats, 0, sizeof(*stats));
  if (depth < 1) ORN_FAIL(ctx, ORN_ERR_ARG, "MTP depth must be at least 1");
  if (depth > kMaxRows - 1) ORN_FAIL(ctx, ORN_ERR_ARG, "MTP depth must be at most 3");
  if (n_prompt < 1) ORN_FAIL(ctx, ORN_ERR_ARG, "generate_step_mtp needs a prompt");
  if (!m->mtp.present) ORN_FAIL(ctx, ORN_ERR_STATE, "generate_step_mtp: the model has no MTP head");
  if (use_frspec && !m->fr_head) ORN_FAIL(ctx, ORN_ERR_STATE, "generate_step_mtp: no FR-Spec head loaded");
  if (policy != ORN_POLICY_CYCLE && policy != ORN_POLICY_COMMITTED) ORN_FAIL(ctx, ORN_ERR_ARG, "unknown history policy");
  m->prof = orn_prof{};
  const int64_t launches0 = ctx->launches;
  cudaEventRecord(m->ev[2], s);
  int done = 0;
  CK(prefill(m, c, prompt, n_prompt, prefill_step, &done));
  cudaEventRecord(m->ev[3], s);
  CK(upload_ids(m, prompt + done, 1));
  CK(forward_greedy_dev(m, c, w.ids, 1, false, w.hrow, w.targets));
  uint32_t primary = 0;
  CK(orn_download(ctx, &primary, w.targets, 4));
  {
    float ms = 0.f;
    cudaEventElapsedTime(&ms, m->ev[2], m->ev[3]);
    m->prof.prefill_ms = ms;
  }
  cudaEventRecord(m->ev[2], s);
  const orn_linear* dlm = use_frspec ? m->fr_head : m->lm_head;
  int emitted = 0;
  uint64_t cycle_idx = 0;
  CK(set_mtp_pos(c, 0));
  uint32_t hbuf[16];
  bool stop = false;
  while (!stop) {
    if (policy == ORN_POLICY_CYCLE) CK(set_mtp_pos(c, 0));  // a fresh cache each cycle
    const int cycle_off = c->h_mtp_pos;
    int want = max_tokens - (emitted + 1);
    if (want < 0) want = 0;
    if (want > depth) want = depth;
    // ---- draft + verify on the device; the host only fills the mailbox
    uint32_t* mb = c->mailbox_h;
    for (int i = 0; i < 16; ++i) mb[i] = 0;
    mb[0] = primary;
    for (int i = 0; i < want; ++i) {
      if (force && force->p > 0.f && emitted + 1 + i < force->len) {
        uint64_t rnd = splitmix64(force->seed + cycle_idx * 8 + (uint64_t)i);
        float uni = (float)(rnd >> 40) * (1.0f / 16777216.0f);
        if (uni < force->p) { mb[1 + i] = 1; mb[4 + i] = force->stream[emitted + 1 + i]; }
      }
    }
    ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(w.mailbox, mb, 16 * sizeof(uint32_t), cudaMemcpyHostToDevice, s));
    CK(run_step(m, c, 0, want, use_frspec != 0));
    m->prof.draft_steps += want;
    if (want > 0) { stats->cycles += 1; stats->drafted += want; }
    cycle_idx += 1;
    const int n_rows = want + 1;
    m->prof.verify_steps += 1;
    // the one host round trip of the cycle (mtp_generate.rs:250-254)
    ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(hbuf, w.targets, 4 * (size_t)n_rows, cudaMemcpyDeviceToHost, s));
    ORN_CHECK_CUDA(ctx, cudaMemcpyAsync(hbuf + 8, w.window, 4 * (size_t)n_rows, cudaMemcpyDeviceToHost, s));
    ORN_CHECK_CUDA(ctx, cudaStreamSynchronize(s));
    const uint32_t* targets = hbuf;
    const uint32_t* window = hbuf + 8;
    int k = 0;
    while (k < want) {
      stats->reached_by_depth[k] += 1;
      if (targets[k] != window[k + 1]) break;
      stats->accepted_by_depth[k] += 1;
      stats->accepted += 1;
      k += 1;
    }
    const uint32_t next_primary = targets[k];
    CK(orn_cache_rewind(c, k + 1));
    if (policy == ORN_POLICY_COMMITTED) {
      CK(set_mtp_pos(c, cycle_off + 1));
      if (k > 0) CK(mtp_step(m, c, w.vh, w.window + 1, k, nullptr, w.dh, nullptr, true));
    }
    copy_bf16_kernel<<<(H + 255) / 256, 256, 0, s>>>(w.vh + (size_t)k * H, w.hrow, H);
    CK(orn_launch_check(ctx, "copy_bf16"));
    for (int i = 0; i <= k; ++i) {
      emitted += 1;
      if (!on_token(window[i], user)) { stop = true; break; }
      if (emitted == max_tokens) { stop = true; break; }
    }
    primary = next_primary;
  }
  cudaEventRecord(m->ev[3], s);
  CK(orn_sync(ctx));
  {
    float ms = 0.f;
    cudaEventElapsedTime(&ms, m->ev[2], m->ev[3]);
    m->prof.total_ms = ms;
  }
  m->prof.kernel_launches = ctx->launches - launches0;
  return ORN_OK;
}

// MtpHead::forward for T rows (mtp.rs:150-262): the head's cache advances by T; the draft is the
// raw-logit argmax of the last row
int32_t orn_mtp_forward(orn_model* m, orn_cache* c, const uint16_t* dev_hidden, const uint32_t* host_ids, int32_t T,
                        int32_t kv_only, uint32_t* host_draft) {
  if (!m || !c || !dev_hidden || !host_ids || T < 1 || T > kMaxRows) return ORN_ERR_ARG;
  CK(orn_model_finalize(m));
  orn_ctx* ctx = m->ctx;
  Workspace& w = m->ws;
  CK(upload_ids(m, host_ids, T));
  CK(mtp_step(m, c, dev_hidden, w.ids, T, kv_only ? nullptr : m->lm_head, w.dh, kv_only ? nullptr : w.dlogits, kv_only != 0));
  if (!kv_only && host_draft) {
    CK(k_greedy(ctx, ctx->stream, w.dlogits + (size_t)(T - 1) * m->lm_head->O, 1, m->lm_head->O, 0, w.local, w.greedy_scratch));
    return orn_download(ctx, host_draft, w.local, sizeof(uint32_t));
  }
  return orn_sync(ctx);
}
int32_t orn_cache_mtp_offset(const orn_cache* c) { return c ? c->h_mtp_pos : -1; }
int32_t orn_cache_set_mtp_offset(orn_cache* c, int32_t v) {
  if (!c || v < 0) return ORN_ERR_ARG;
  return set_mtp_pos(c, v);
}

int32_t orn_get_prof(orn_model* m, orn_prof* out) {
  if (!m || !out) return ORN_ERR_ARG;
  *out = m->prof;
  return ORN_OK;
}

int32_t orn_moe_block(orn_ctx* ctx, const orn_linear* gate, const orn_linear* sw_gate,
                      const orn_linear* sw_up, const orn_linear* sw_down, const orn_linear* sh_gate,
                      const orn_linear* sh_up, const orn_linear* sh_down, const orn_linear* sh_egate,
                      const uint16_t* dev_x, int32_t T, int32_t top_k, int32_t norm_topk,
                      uint16_t* dev_out, uint32_t* dev_inds_out) {
  if (!ctx || !gate || !sw_gate || !sw_up || !sw_down || !sh_gate || !sh_up || !sh_down || !sh_egate ||
      !dev_x || !dev_out)
    return ORN_ERR_ARG;
  if (T < 1 || T > kMaxRows) ORN_FAIL(ctx, ORN_ERR_ARG, "moe_block: 1..4 rows per call");
  // a throw-away model shell gives the block its scratch
  orn_config cfg{};
  cfg.hidden = gate->K; cfg.n_experts = gate->O; cfg.top_k = top_k; cfg.expert_inter = sw_gate->O;
  cfg.shared_inter = sh_gate->O; cfg.norm_topk_prob = norm_topk;
  if (sw_gate->E != cfg.n_experts || sw_up->E != cfg.n_experts || sw_down->E != cfg.n_experts ||
      sw_gate->K != cfg.hidden || sw_down->O != cfg.hidden || sw_down->K != cfg.expert_inter ||
      sh_down->K != cfg.shared_inter || sh_egate->O != 1 || top_k < 1 || top_k > cfg.n_experts)
    ORN_FAIL(ctx, ORN_ERR_ARG, "moe_block: inconsistent weight shapes");
  orn_model shell;
  shell.ctx = ctx;
  shell.cfg = cfg;
  Workspace& w = shell.ws;
  const size_t R = kMaxRows, H = cfg.hidden, E = cfg.n_experts, I = cfg.expert_inter, SI = cfg.shared_inter, k = top_k;
  int rc = ORN_OK;
  auto A = [&](auto** p, size_t n) { if (rc == ORN_OK) rc = ws_alloc(&shell, p, n); };
  A(&w.gates, R * E); A(&w.probs, R * E); A(&w.scores, R * k); A(&w.eg, R * k * I); A(&w.eu, R * k * I);
  A(&w.eact, R * k * I); A(&w.ey, R * k * H); A(&w.sg, R * SI); A(&w.su, R * SI); A(&w.sact, R * SI);
  A(&w.sy, R * H); A(&w.gs, R); A(&w.inds, R * k); A(&w.lhs, R * k); A(&w.ident, R * k);
  if (rc == ORN_OK) {
    int n = kMaxRows * top_k;
    iota_div_kernel<<<(n + 63) / 64, 64, 0, ctx->stream>>>(w.lhs, w.ident, n, top_k);
    rc = orn_launch_check(ctx, "iota_div");
  }
  Moe moe;
  moe.gate = (orn_linear*)gate; moe.sw_gate = (orn_linear*)sw_gate; moe.sw_up = (orn_linear*)sw_up;
  moe.sw_down = (orn_linear*)sw_down; moe.sh_gate = (orn_linear*)sh_gate; moe.sh_up = (orn_linear*)sh_up;
  moe.sh_down = (orn_linear*)sh_down; moe.sh_egate = (orn_linear*)sh_egate;
  // the route the model takes (three persistent kernels) whenever the shapes allow it; the
  // one-kernel-per-op sequence under ORN_UNFUSED=1 and for shapes outside the fused kernels' limits
  const bool fused = use_fused_env() && cfg.hidden % 256 == 0 && cfg.hidden <= 4096 && cfg.n_experts <= 512 && top_k <= 8 &&
                     cfg.expert_inter % 256 == 0 && cfg.shared_inter % 256 == 0 && cfg.expert_inter <= 2048 &&
                     cfg.shared_inter <= 2048 && sw_gate->kind == sw_up->kind && sw_down->kind == sh_down->kind &&
                     sh_gate->kind == sh_up->kind && gate->kind <= ORN_BF16 && sw_gate->kind <= ORN_BF16 &&
                     sw_down->kind <= ORN_BF16 && sh_gate->kind <= ORN_BF16 && sh_egate->kind <= ORN_BF16 &&
                     sh_gate->K == cfg.hidden && sh_up->O == cfg.shared_inter &&
                     sh_up->K == cfg.hidden;
  if (rc == ORN_OK && fused) {
    FusedPrologue fp;
    fp.mode = PRO_PLAIN; fp.K = cfg.hidden; fp.a = dev_x;
    FusedJob jobs[3];
    jobs[0].lin = gate; jobs[0].out = w.gates;
    jobs[1].lin = sh_gate; jobs[1].lin2 = sh_up; jobs[1].out = w.sact; jobs[1].epi = EPI_SWIGLU;
    jobs[2].lin = sh_egate; jobs[2].out = w.gs;
    uint32_t* inds = dev_inds_out ? dev_inds_out : w.inds;
    rc = f_norm_gemv(ctx, ctx->stream, T, fp, jobs, 3);
    if (rc == ORN_OK) rc = f_moe_up(ctx, ctx->stream, T, w.gates, dev_x, sw_gate, sw_up, top_k, inds, w.scores, w.eact);
    if (rc == ORN_OK)
      rc = f_moe_down(ctx, ctx->stream, T, w.eact, w.sact, inds, w.scores, w.gs, sw_down, sh_down, top_k, norm_topk, dev_out);
  } else if (rc == ORN_OK) {
    rc = moe_block(&shell, moe, dev_x, T, dev_out, dev_inds_out);
  }
  if (rc == ORN_OK) rc = orn_sync(ctx);
  else cudaStreamSynchronize(ctx->stream);
  for (void* p : shell.ws_allocs) cudaFree(p);
  return rc;
}

}  // extern "C"
