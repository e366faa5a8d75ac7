/* TEST INFRASTRUCTURE, NOT PRODUCT CODE.  See orn_oracle_math.h.
 *
 * Model-level CPU restatement: the Qwen3.5-MoE trunk, the MTP head and the two
 * generation loops of ornith-rs, composed from the ops in orn_oracle_ops.c.
 */
#include "orn_oracle.h"

#include <stdio.h>
#include <stdlib.h>

typedef struct {
  int is_linear;
  const bf16 *input_ln, *post_ln;
  orc_lin in_qkv, in_z, in_a, in_b, out_proj;
  const bf16 *conv_w, *dt_bias, *a_log, *gdn_norm;
  orc_lin q_proj, k_proj, v_proj, o_proj;
  const bf16 *q_norm, *k_norm;
  orc_moe moe;
} orc_layer;

typedef struct {
  const bf16 *pre_fc_norm_embedding, *pre_fc_norm_hidden, *input_ln, *post_ln, *norm;
  const bf16 *q_norm, *k_norm;
  orc_lin fc, q_proj, k_proj, v_proj, o_proj;
  orc_moe moe;
} orc_mtp;

struct orc_model {
  orc_config cfg;
  orc_lin embed, lm_head;
  const bf16* norm;
  orc_layer* layers;
  orc_mtp mtp;
  orc_lin fr_head;
  const uint32_t* fr_ids;
  int fr_n;
};

typedef struct {
  bf16 *k, *v; /* [Hkv, cap, hd] */
  int offset;
} orc_kv;

typedef struct {
  bf16* conv;   /* [Kc-1, D] */
  float* state; /* [Hv, 128, 128] */
} orc_gdn;

struct orc_cache {
  const orc_model* m;
  orc_kv* kv;   /* per layer (unused entries NULL) */
  orc_gdn* gdn; /* per layer */
  orc_kv mtp_kv;
  /* capture of the last forward_capture window (qwen3_5.rs:301-349) */
  int cap_T;
  int cap_base;
  bf16** cap_conv_input; /* per GDN layer: [Kc-1+T, D] */
  float** cap_states;    /* per GDN layer: [T, Hv,128,128] */
};

/* ---------------------------------------------------------------- helpers */
static int conv_dim(const orc_config* c) {
  return 2 * c->gdn_k_heads * c->gdn_head_dim + c->gdn_v_heads * c->gdn_head_dim;
}
static int is_linear_layer(const orc_config* c, int i) {
  return ((i + 1) % c->full_attn_interval) != 0; /* config.rs: full attention at 3,7,... */
}
static bf16* balloc(size_t n) { return (bf16*)calloc(n ? n : 1, sizeof(bf16)); }

orc_model* orc_model_new(const orc_config* cfg) {
  orc_model* m = (orc_model*)calloc(1, sizeof(orc_model));
  m->cfg = *cfg;
  m->layers = (orc_layer*)calloc((size_t)cfg->n_layers, sizeof(orc_layer));
  for (int i = 0; i < cfg->n_layers; ++i) m->layers[i].is_linear = is_linear_layer(cfg, i);
  return m;
}
void orc_model_free(orc_model* m) {
  if (!m) return;
  free(m->layers);
  free(m);
}

static const char* strip(const char* name, const char* prefix) {
  size_t n = strlen(prefix);
  return strncmp(name, prefix, n) == 0 ? name + n : NULL;
}

static int set_moe(orc_moe* moe, const char* s, const orc_lin* L) {
  if (!strcmp(s, "gate")) moe->gate = *L;
  else if (!strcmp(s, "switch_mlp.gate_proj")) moe->sw_gate = *L;
  else if (!strcmp(s, "switch_mlp.up_proj")) moe->sw_up = *L;
  else if (!strcmp(s, "switch_mlp.down_proj")) moe->sw_down = *L;
  else if (!strcmp(s, "shared_expert.gate_proj")) moe->sh_gate = *L;
  else if (!strcmp(s, "shared_expert.up_proj")) moe->sh_up = *L;
  else if (!strcmp(s, "shared_expert.down_proj")) moe->sh_down = *L;
  else if (!strcmp(s, "shared_expert_gate")) moe->sh_egate = *L;
  else return -1;
  return 0;
}

int orc_model_set(orc_model* m, const char* name, int kind, int E, int O, int K, const void* w,
                  const void* s, const void* b) {
  orc_lin L = {kind, E, O, K, w, s, b};
  const char* n = name;
  const char* r;
  if ((r = strip(n, "language_model.model."))) n = r;
  else if ((r = strip(n, "language_model."))) n = r;
  if (!strcmp(n, "embed_tokens")) { m->embed = L; return 0; }
  if (!strcmp(n, "lm_head")) { m->lm_head = L; return 0; }
  if (!strcmp(n, "norm.weight")) { m->norm = (const bf16*)w; return 0; }
  if ((r = strip(n, "layers."))) {
    char* end;
    long i = strtol(r, &end, 10);
    if (i < 0 || i >= m->cfg.n_layers || *end != '.') return -1;
    orc_layer* ly = &m->layers[i];
    const char* t = end + 1;
    const char* q;
    if (!strcmp(t, "input_layernorm.weight")) ly->input_ln = (const bf16*)w;
    else if (!strcmp(t, "post_attention_layernorm.weight")) ly->post_ln = (const bf16*)w;
    else if ((q = strip(t, "linear_attn."))) {
      if (!strcmp(q, "in_proj_qkv")) ly->in_qkv = L;
      else if (!strcmp(q, "in_proj_z")) ly->in_z = L;
      else if (!strcmp(q, "in_proj_a.weight")) ly->in_a = L;
      else if (!strcmp(q, "in_proj_b.weight")) ly->in_b = L;
      else if (!strcmp(q, "out_proj")) ly->out_proj = L;
      else if (!strcmp(q, "conv1d.weight")) ly->conv_w = (const bf16*)w;
      else if (!strcmp(q, "dt_bias")) ly->dt_bias = (const bf16*)w;
      else if (!strcmp(q, "A_log")) ly->a_log = (const bf16*)w;
      else if (!strcmp(q, "norm.weight")) ly->gdn_norm = (const bf16*)w;
      else return -1;
    } else if ((q = strip(t, "self_attn."))) {
      if (!strcmp(q, "q_proj")) ly->q_proj = L;
      else if (!strcmp(q, "k_proj")) ly->k_proj = L;
      else if (!strcmp(q, "v_proj")) ly->v_proj = L;
      else if (!strcmp(q, "o_proj")) ly->o_proj = L;
      else if (!strcmp(q, "q_norm.weight")) ly->q_norm = (const bf16*)w;
      else if (!strcmp(q, "k_norm.weight")) ly->k_norm = (const bf16*)w;
      else return -1;
    } else if ((q = strip(t, "mlp."))) {
      return set_moe(&ly->moe, q, &L);
    } else return -1;
    return 0;
  }
  if ((r = strip(n, "mtp."))) {
    orc_mtp* h = &m->mtp;
    const char* q;
    if (!strcmp(r, "pre_fc_norm_embedding.weight")) h->pre_fc_norm_embedding = (const bf16*)w;
    else if (!strcmp(r, "pre_fc_norm_hidden.weight")) h->pre_fc_norm_hidden = (const bf16*)w;
    else if (!strcmp(r, "fc.weight")) h->fc = L;
    else if (!strcmp(r, "norm.weight")) h->norm = (const bf16*)w;
    else if ((q = strip(r, "layers.0."))) {
      const char* p;
      if (!strcmp(q, "input_layernorm.weight")) h->input_ln = (const bf16*)w;
      else if (!strcmp(q, "post_attention_layernorm.weight")) h->post_ln = (const bf16*)w;
      else if ((p = strip(q, "self_attn."))) {
        if (!strcmp(p, "q_proj.weight")) h->q_proj = L;
        else if (!strcmp(p, "k_proj.weight")) h->k_proj = L;
        else if (!strcmp(p, "v_proj.weight")) h->v_proj = L;
        else if (!strcmp(p, "o_proj.weight")) h->o_proj = L;
        else if (!strcmp(p, "q_norm.weight")) h->q_norm = (const bf16*)w;
        else if (!strcmp(p, "k_norm.weight")) h->k_norm = (const bf16*)w;
        else return -1;
      } else if ((p = strip(q, "mlp."))) {
        /* the harness registers the stacked experts under the switch_mlp names
         * and the dense matrices without the ".weight" suffix */
        return set_moe(&h->moe, p, &L);
      } else return -1;
    } else return -1;
    return 0;
  }
  return -1;
}

void orc_model_set_frspec(orc_model* m, const orc_lin* pruned_head, const uint32_t* ids, int n) {
  m->fr_head = *pruned_head;
  m->fr_ids = ids;
  m->fr_n = n;
}

/* src/model/cache.rs:18-181.  KV capacity is fixed at cfg.max_ctx here (the
 * reference grows in 256-token steps; the contents are the same). */
orc_cache* orc_cache_new(const orc_model* m) {
  const orc_config* c = &m->cfg;
  orc_cache* k = (orc_cache*)calloc(1, sizeof(orc_cache));
  k->m = m;
  k->kv = (orc_kv*)calloc((size_t)c->n_layers, sizeof(orc_kv));
  k->gdn = (orc_gdn*)calloc((size_t)c->n_layers, sizeof(orc_gdn));
  k->cap_conv_input = (bf16**)calloc((size_t)c->n_layers, sizeof(bf16*));
  k->cap_states = (float**)calloc((size_t)c->n_layers, sizeof(float*));
  size_t kvsz = (size_t)c->n_kv_heads * c->max_ctx * c->head_dim;
  size_t ssz = (size_t)c->gdn_v_heads * c->gdn_head_dim * c->gdn_head_dim;
  for (int i = 0; i < c->n_layers; ++i) {
    if (m->layers[i].is_linear) {
      k->gdn[i].conv = balloc((size_t)(c->gdn_conv_kernel - 1) * conv_dim(c));
      k->gdn[i].state = (float*)calloc(ssz, sizeof(float));
    } else {
      k->kv[i].k = balloc(kvsz);
      k->kv[i].v = balloc(kvsz);
    }
  }
  k->mtp_kv.k = balloc(kvsz);
  k->mtp_kv.v = balloc(kvsz);
  return k;
}
void orc_cache_free(orc_cache* k) {
  if (!k) return;
  int L = k->m->cfg.n_layers;
  for (int i = 0; i < L; ++i) {
    free(k->kv[i].k); free(k->kv[i].v); free(k->gdn[i].conv); free(k->gdn[i].state);
    free(k->cap_conv_input[i]); free(k->cap_states[i]);
  }
  free(k->mtp_kv.k); free(k->mtp_kv.v);
  free(k->kv); free(k->gdn); free(k->cap_conv_input); free(k->cap_states);
  free(k);
}
int orc_cache_offset(const orc_cache* c) {
  for (int i = 0; i < c->m->cfg.n_layers; ++i)
    if (!c->m->layers[i].is_linear) return c->kv[i].offset;
  return 0;
}

/* ------------------------------------------------------------------ blocks */
/* src/ops/moe.rs:662-741 (sparse_moe_block) / :902-937 (dense) */
void orc_moe_block(const orc_moe* m, const bf16* x, int T, int top_k, int norm_topk, bf16* out,
                   uint32_t* inds_out) {
  int H = m->gate.K, E = m->gate.O, I = m->sw_gate.O, SI = m->sh_gate.O;
  bf16* gates = balloc((size_t)T * E);
  bf16* probs = balloc((size_t)T * E);
  orc_gemv(&m->gate, x, T, NULL, gates);
  orc_softmax_precise(gates, T, E, probs);
  uint32_t* inds = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)T * top_k);
  bf16* scores = balloc((size_t)T * top_k);
  orc_router_topk(probs, T, E, top_k, inds, scores);
  int rows = T * top_k;
  uint32_t* lhs = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)rows);
  uint32_t* ident = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)rows);
  for (int r = 0; r < rows; ++r) { lhs[r] = (uint32_t)(r / top_k); ident[r] = (uint32_t)r; }
  bf16* g = balloc((size_t)rows * I);
  bf16* u = balloc((size_t)rows * I);
  bf16* act = balloc((size_t)rows * I);
  bf16* y = balloc((size_t)rows * H);
  orc_gather_gemv(&m->sw_gate, x, lhs, inds, rows, g);
  orc_gather_gemv(&m->sw_up, x, lhs, inds, rows, u);
  orc_swiglu(g, u, rows * I, act);
  orc_gather_gemv(&m->sw_down, act, ident, inds, rows, y);
  bf16* sg = balloc((size_t)T * SI);
  bf16* su = balloc((size_t)T * SI);
  bf16* sact = balloc((size_t)T * SI);
  bf16* sy = balloc((size_t)T * H);
  bf16* gs = balloc((size_t)T);
  orc_gemv(&m->sh_gate, x, T, NULL, sg);
  orc_gemv(&m->sh_up, x, T, NULL, su);
  orc_swiglu(sg, su, T * SI, sact);
  orc_gemv(&m->sh_down, sact, T, NULL, sy);
  orc_gemv(&m->sh_egate, x, T, NULL, gs);
  orc_moe_combine(scores, y, gs, sy, T, top_k, H, norm_topk, out);
  if (inds_out) memcpy(inds_out, inds, sizeof(uint32_t) * (size_t)rows);
  free(gates); free(probs); free(inds); free(scores); free(lhs); free(ident);
  free(g); free(u); free(act); free(y); free(sg); free(su); free(sact); free(sy); free(gs);
}

/* Attention::forward (qwen3_5.rs:430-474); the MTP head's attention
 * (mtp.rs:219-262) is the same with dense projections. */
static void attention(const orc_config* c, const orc_lin* qp, const orc_lin* kp, const orc_lin* vp,
                      const orc_lin* op, const bf16* q_norm, const bf16* k_norm, const bf16* x,
                      int T, orc_kv* kv, bf16* out) {
  int Hq = c->n_heads, Hkv = c->n_kv_heads, hd = c->head_dim, cap = c->max_ctx;
  bf16* qg = balloc((size_t)T * Hq * 2 * hd);
  bf16* q = balloc((size_t)T * Hq * hd);
  bf16* gate = balloc((size_t)T * Hq * hd);
  bf16* k = balloc((size_t)T * Hkv * hd);
  bf16* v = balloc((size_t)T * Hkv * hd);
  orc_gemv(qp, x, T, NULL, qg);
  orc_gemv(kp, x, T, NULL, k);
  orc_gemv(vp, x, T, NULL, v);
  for (int t = 0; t < T; ++t)
    for (int h = 0; h < Hq; ++h) {
      memcpy(q + ((size_t)t * Hq + h) * hd, qg + ((size_t)t * Hq + h) * 2 * hd, sizeof(bf16) * hd);
      memcpy(gate + ((size_t)t * Hq + h) * hd, qg + ((size_t)t * Hq + h) * 2 * hd + hd,
             sizeof(bf16) * hd);
    }
  orc_rms_norm(q, q_norm, T * Hq, hd, c->rms_eps, q);
  orc_rms_norm(k, k_norm, T * Hkv, hd, c->rms_eps, k);
  float lnb = (float)(log((double)c->rope_theta) / (double)(c->rope_dims / 2));
  orc_rope(q, T, Hq, hd, c->rope_dims, lnb, kv->offset);
  orc_rope(k, T, Hkv, hd, c->rope_dims, lnb, kv->offset);
  for (int t = 0; t < T; ++t)
    for (int h = 0; h < Hkv; ++h) {
      memcpy(kv->k + ((size_t)h * cap + kv->offset + t) * hd, k + ((size_t)t * Hkv + h) * hd,
             sizeof(bf16) * hd);
      memcpy(kv->v + ((size_t)h * cap + kv->offset + t) * hd, v + ((size_t)t * Hkv + h) * hd,
             sizeof(bf16) * hd);
    }
  bf16* att = balloc((size_t)T * Hq * hd);
  float scale = 1.0f / sqrtf((float)hd);
  orc_sdpa_decode(q, kv->k, kv->v, T, Hq, Hkv, hd, cap, kv->offset, scale, att);
  kv->offset += T;
  bf16* gated = balloc((size_t)T * Hq * hd);
  orc_sigmoid_gate(gate, att, T * Hq * hd, 1, gated);
  orc_gemv(op, gated, T, NULL, out);
  free(qg); free(q); free(gate); free(k); free(v); free(att); free(gated);
}

/* GatedDeltaNet::forward / forward_capture (qwen3_5.rs:478-695) */
static void gdn_layer(const orc_config* c, const orc_layer* ly, const bf16* x, int T, orc_gdn* st,
                      bf16* conv_input_keep, float* states_keep, bf16* out) {
  int Hk = c->gdn_k_heads, Hv = c->gdn_v_heads, Dh = c->gdn_head_dim, Kc = c->gdn_conv_kernel;
  int D = conv_dim(c), VD = Hv * Dh, S = Kc - 1;
  bf16* qkv = balloc((size_t)T * D);
  bf16* z = balloc((size_t)T * VD);
  bf16* aa = balloc((size_t)T * Hv);
  bf16* bb = balloc((size_t)T * Hv);
  orc_gemv(&ly->in_qkv, x, T, NULL, qkv);
  orc_gemv(&ly->in_z, x, T, NULL, z);
  orc_gemv(&ly->in_b, x, T, NULL, bb);
  orc_gemv(&ly->in_a, x, T, NULL, aa);
  if (conv_input_keep) {
    memcpy(conv_input_keep, st->conv, sizeof(bf16) * (size_t)S * D);
    memcpy(conv_input_keep + (size_t)S * D, qkv, sizeof(bf16) * (size_t)T * D);
  }
  bf16* q = balloc((size_t)T * Hk * Dh);
  bf16* k = balloc((size_t)T * Hk * Dh);
  bf16* v = balloc((size_t)T * VD);
  bf16* beta = balloc((size_t)T * Hv);
  float* g = (float*)malloc(sizeof(float) * (size_t)T * Hv);
  bf16* conv_next = balloc((size_t)S * D);
  orc_gdn_front(st->conv, qkv, ly->conv_w, aa, bb, ly->a_log, ly->dt_bias, T, Hk, Hv, Dh, Kc,
                1e-6f, conv_next, q, k, v, beta, g);
  memcpy(st->conv, conv_next, sizeof(bf16) * (size_t)S * D);
  bf16* y = balloc((size_t)T * VD);
  orc_gated_delta(q, k, v, g, beta, st->state, T, Hk, Hv, y, states_keep);
  bf16* gated = balloc((size_t)T * VD);
  orc_rms_norm_gated(y, ly->gdn_norm, z, T * Hv, Dh, c->rms_eps, gated);
  orc_gemv(&ly->out_proj, gated, T, NULL, out);
  free(qkv); free(z); free(aa); free(bb); free(q); free(k); free(v); free(beta); free(g);
  free(conv_next); free(y); free(gated);
}

/* TextModel::forward_hidden / forward_capture (qwen3_5.rs:190-279) */
static void forward_impl(const orc_model* m, orc_cache* cc, const uint32_t* ids, int T,
                         int capture, bf16* normed_out, bf16* pre_norm_out) {
  const orc_config* c = &m->cfg;
  int H = c->hidden;
  bf16* x = balloc((size_t)T * H);
  bf16* normed = balloc((size_t)T * H);
  bf16* r = balloc((size_t)T * H);
  bf16* h = balloc((size_t)T * H);
  bf16* normed2 = balloc((size_t)T * H);
  bf16* mo = balloc((size_t)T * H);
  orc_embedding_a8(&m->embed, ids, T, x);
  orc_rms_norm(x, m->layers[0].input_ln, T, H, c->rms_eps, normed);
  if (capture) {
    cc->cap_T = T;
    cc->cap_base = orc_cache_offset(cc);
  }
  size_t ssz = (size_t)c->gdn_v_heads * c->gdn_head_dim * c->gdn_head_dim;
  for (int i = 0; i < c->n_layers; ++i) {
    const orc_layer* ly = &m->layers[i];
    if (ly->is_linear) {
      bf16* ci = NULL;
      float* sk = NULL;
      if (capture) {
        free(cc->cap_conv_input[i]);
        free(cc->cap_states[i]);
        ci = cc->cap_conv_input[i] = balloc((size_t)(c->gdn_conv_kernel - 1 + T) * conv_dim(c));
        sk = cc->cap_states[i] = (float*)malloc(sizeof(float) * ssz * (size_t)T);
      }
      gdn_layer(c, ly, normed, T, &cc->gdn[i], ci, sk, r);
    } else {
      attention(c, &ly->q_proj, &ly->k_proj, &ly->v_proj, &ly->o_proj, ly->q_norm, ly->k_norm,
                normed, T, &cc->kv[i], r);
    }
    orc_add_rms_norm(x, r, ly->post_ln, T, H, c->rms_eps, h, normed2);
    orc_moe_block(&ly->moe, normed2, T, c->top_k, c->norm_topk_prob, mo, NULL);
    const bf16* nw = (i + 1 < c->n_layers) ? m->layers[i + 1].input_ln : m->norm;
    orc_add_rms_norm(h, mo, nw, T, H, c->rms_eps, x, normed);
  }
  memcpy(normed_out, normed, sizeof(bf16) * (size_t)T * H);
  if (pre_norm_out) memcpy(pre_norm_out, x, sizeof(bf16) * (size_t)T * H);
  free(x); free(normed); free(r); free(h); free(normed2); free(mo);
}

void orc_forward(const orc_model* m, orc_cache* c, const uint32_t* ids, int T, bf16* normed,
                 bf16* pre_norm) {
  forward_impl(m, c, ids, T, 0, normed, pre_norm);
}

/* TrunkCapture::rewind (qwen3_5.rs:324-348) */
static void rewind_capture(orc_cache* cc, int keep) {
  const orc_model* m = cc->m;
  const orc_config* c = &m->cfg;
  int S = c->gdn_conv_kernel - 1, D = conv_dim(c);
  size_t ssz = (size_t)c->gdn_v_heads * c->gdn_head_dim * c->gdn_head_dim;
  for (int i = 0; i < c->n_layers; ++i) {
    if (m->layers[i].is_linear) {
      memcpy(cc->gdn[i].conv, cc->cap_conv_input[i] + (size_t)keep * D, sizeof(bf16) * (size_t)S * D);
      memcpy(cc->gdn[i].state, cc->cap_states[i] + (size_t)(keep - 1) * ssz, sizeof(float) * ssz);
    } else {
      cc->kv[i].offset = cc->cap_base + keep;
    }
  }
}

void orc_head_greedy(const orc_model* m, const bf16* hidden, int T, uint32_t* tokens,
                     bf16* logits_out) {
  int V = m->cfg.vocab;
  bf16* logits = logits_out ? logits_out : balloc((size_t)T * V);
  orc_gemv(&m->lm_head, hidden, T, NULL, logits);
  for (int t = 0; t < T; ++t) tokens[t] = orc_greedy_token(logits + (size_t)t * V, V, 1);
  if (!logits_out) free(logits);
}

/* MtpHead::hidden (mtp.rs:166-217) */
static void mtp_hidden(const orc_model* m, orc_cache* cc, const bf16* trunk_hidden,
                       const uint32_t* next_ids, int T, bf16* out) {
  const orc_config* c = &m->cfg;
  const orc_mtp* hd = &m->mtp;
  int H = c->hidden;
  bf16* emb = balloc((size_t)T * H);
  bf16* joined = balloc((size_t)T * 2 * H);
  bf16* e = balloc((size_t)T * H);
  bf16* hh = balloc((size_t)T * H);
  orc_embedding_a8(&m->embed, next_ids, T, emb);
  orc_rms_norm(emb, hd->pre_fc_norm_embedding, T, H, c->rms_eps, e);
  orc_rms_norm(trunk_hidden, hd->pre_fc_norm_hidden, T, H, c->rms_eps, hh);
  for (int t = 0; t < T; ++t) { /* concat_order "embedding_hidden" */
    memcpy(joined + (size_t)t * 2 * H, e + (size_t)t * H, sizeof(bf16) * H);
    memcpy(joined + (size_t)t * 2 * H + H, hh + (size_t)t * H, sizeof(bf16) * H);
  }
  bf16* x = balloc((size_t)T * H);
  orc_gemv(&hd->fc, joined, T, NULL, x);
  bf16* normed = balloc((size_t)T * H);
  bf16* r = balloc((size_t)T * H);
  bf16* h2 = balloc((size_t)T * H);
  bf16* normed2 = balloc((size_t)T * H);
  bf16* mo = balloc((size_t)T * H);
  orc_rms_norm(x, hd->input_ln, T, H, c->rms_eps, normed);
  attention(c, &hd->q_proj, &hd->k_proj, &hd->v_proj, &hd->o_proj, hd->q_norm, hd->k_norm, normed,
            T, &cc->mtp_kv, r);
  for (int i = 0; i < T * H; ++i) h2[i] = o_f2bf(o_bf2f(x[i]) + o_bf2f(r[i]));
  orc_rms_norm(h2, hd->post_ln, T, H, c->rms_eps, normed2);
  orc_moe_block(&hd->moe, normed2, T, c->top_k, c->norm_topk_prob, mo, NULL);
  for (int i = 0; i < T * H; ++i) h2[i] = o_f2bf(o_bf2f(h2[i]) + o_bf2f(mo[i]));
  orc_rms_norm(h2, hd->norm, T, H, c->rms_eps, out);
  free(emb); free(joined); free(e); free(hh); free(x); free(normed); free(r); free(h2);
  free(normed2); free(mo);
}

/* generate::prefill (generate.rs:90-136): everything but the last prompt token.
 * Every row is computed with single-row arithmetic, so the chunk width cannot
 * change a bit of the result; chunks of 4 keep the scratch small. */
static int prefill(const orc_model* m, orc_cache* c, const uint32_t* prompt, int n) {
  int H = m->cfg.hidden, done = 0;
  bf16* tmp = balloc((size_t)4 * H);
  while (n - done > 1) {
    int t = n - done - 1 < 4 ? n - done - 1 : 4;
    forward_impl(m, c, prompt + done, t, 0, tmp, NULL);
    done += t;
  }
  free(tmp);
  return done;
}

int orc_generate(const orc_model* m, orc_cache* c, const uint32_t* prompt, int n_prompt,
                 int max_tokens, uint32_t* out) {
  int H = m->cfg.hidden;
  bf16* hid = balloc((size_t)H);
  int done = prefill(m, c, prompt, n_prompt);
  uint32_t y;
  forward_impl(m, c, prompt + done, 1, 0, hid, NULL);
  orc_head_greedy(m, hid, 1, &y, NULL);
  int n = 0;
  while (n != max_tokens) {
    uint32_t next;
    forward_impl(m, c, &y, 1, 0, hid, NULL);
    orc_head_greedy(m, hid, 1, &next, NULL);
    out[n++] = y;
    y = next;
  }
  free(hid);
  return n;
}

static uint64_t splitmix64(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

int orc_generate_mtp(const orc_model* m, orc_cache* cc, const uint32_t* prompt, int n_prompt,
                     int depth, int max_tokens, int policy, int use_frspec,
                     const orc_force* force, uint32_t* out, orc_mtp_stats* stats) {
  const orc_config* c = &m->cfg;
  int H = c->hidden, V = c->vocab;
  memset(stats, 0, sizeof(*stats));
  if (depth < 1 || depth > 7 || n_prompt < 1) return -1;
  bf16* hid = balloc((size_t)H);
  int done = prefill(m, cc, prompt, n_prompt);
  forward_impl(m, cc, prompt + done, 1, 0, hid, NULL);
  uint32_t primary;
  orc_head_greedy(m, hid, 1, &primary, NULL);
  bf16* h = balloc((size_t)H);
  memcpy(h, hid, sizeof(bf16) * (size_t)H);

  int emitted = 0;
  uint64_t cycle_idx = 0;
  uint32_t window[8], targets[8];
  bf16* vh = balloc((size_t)(depth + 1) * H);
  bf16* dh = balloc((size_t)H);
  bf16* dh2 = balloc((size_t)H);
  const orc_lin* dlm = use_frspec ? &m->fr_head : &m->lm_head;
  bf16* dlogits = balloc((size_t)dlm->O);
  cc->mtp_kv.offset = 0;
  for (;;) {
    if (policy == 0) cc->mtp_kv.offset = 0; /* HistoryPolicy::Cycle: a fresh cache */
    int cycle_off = cc->mtp_kv.offset;
    int want = max_tokens - (emitted + 1);
    if (want < 0) want = 0;
    if (want > depth) want = depth;
    /* draft (mtp_generate.rs:99-135) */
    window[0] = primary;
    memcpy(dh, h, sizeof(bf16) * (size_t)H);
    for (int i = 0; i < want; ++i) {
      mtp_hidden(m, cc, dh, &window[i], 1, dh2);
      orc_gemv(dlm, dh2, 1, NULL, dlogits);
      uint32_t tok = orc_greedy_token(dlogits, dlm->O, 0);
      if (use_frspec) tok = m->fr_ids[tok];
      if (force && force->p > 0.f && emitted + 1 + i < force->len) {
        uint64_t rnd = splitmix64(force->seed + cycle_idx * 8 + (uint64_t)i);
        float uni = (float)(rnd >> 40) * (1.0f / 16777216.0f);
        if (uni < force->p) tok = force->stream[emitted + 1 + i];
      }
      window[i + 1] = tok;
      memcpy(dh, dh2, sizeof(bf16) * (size_t)H);
    }
    if (want > 0) { stats->cycles += 1; stats->drafted += want; }
    cycle_idx += 1;
    /* verify */
    int n_rows = want + 1;
    forward_impl(m, cc, window, n_rows, 1, vh, NULL);
    orc_head_greedy(m, vh, n_rows, targets, NULL);
    int k = 0;
    while (k < want) {
      stats->reached_by_depth[k] += 1;
      if (targets[k] != window[k + 1]) break;
      stats->accepted_by_depth[k] += 1;
      stats->accepted += 1;
      k += 1;
    }
    uint32_t next_primary = targets[k];
    rewind_capture(cc, k + 1);
    if (policy == 1) {
      cc->mtp_kv.offset = cycle_off + 1;
      if (k > 0) {
        bf16* scratch = balloc((size_t)k * H);
        mtp_hidden(m, cc, vh, &window[1], k, scratch);
        free(scratch);
      }
    }
    memcpy(h, vh + (size_t)k * H, sizeof(bf16) * (size_t)H);
    int stop = 0;
    for (int i = 0; i <= k; ++i) {
      out[emitted++] = window[i];
      if (emitted == max_tokens) { stop = 1; break; }
    }
    if (stop) break;
    primary = next_primary;
  }
  (void)V;
  free(hid); free(h); free(vh); free(dh); free(dh2); free(dlogits);
  return emitted;
}
