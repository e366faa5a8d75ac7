// Model-level types shared by the translation units that walk the layers (model.cu: the
// single-sequence engine; batch.cu: the batched decode engine).
#pragma once

#include <map>
#include <string>
#include <vector>

#include "fused.h"
#include "orn_internal.h"

namespace ornm {


constexpr int kMaxRows = 4;   // widest window a forward call takes
constexpr int kRing = 5;      // state buffers per gated-delta layer (window <= 4)

struct Moe {
  orn_linear *gate = nullptr, *sw_gate = nullptr, *sw_up = nullptr, *sw_down = nullptr;
  orn_linear *sh_gate = nullptr, *sh_up = nullptr, *sh_down = nullptr, *sh_egate = nullptr;
};
struct Layer {
  bool linear = false;
  bf16_t *input_ln = nullptr, *post_ln = nullptr;
  orn_linear *in_qkv = nullptr, *in_z = nullptr, *in_a = nullptr, *in_b = nullptr, *out_proj = nullptr;
  bf16_t *conv_w = nullptr, *dt_bias = nullptr, *a_log = nullptr, *gdn_norm = nullptr;
  orn_linear *q_proj = nullptr, *k_proj = nullptr, *v_proj = nullptr, *o_proj = nullptr;
  bf16_t *q_norm = nullptr, *k_norm = nullptr;
  Moe moe;
};
struct Mtp {
  bool present = false;
  bf16_t *pre_fc_norm_embedding = nullptr, *pre_fc_norm_hidden = nullptr, *input_ln = nullptr,
         *post_ln = nullptr, *norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
  orn_linear *fc = nullptr, *q_proj = nullptr, *k_proj = nullptr, *v_proj = nullptr, *o_proj = nullptr;
  Moe moe;
};

struct Tensor {
  bf16_t* p = nullptr;
  size_t n = 0;
};

// activation scratch for up to kMaxRows rows
struct Workspace {
  bf16_t *x, *normed, *r, *h, *normed2, *mo;
  bf16_t *z, *aa, *bb, *gq, *gk, *gv, *beta, *gy, *ggated;
  float* gg;
  bf16_t *qg, *aq, *agate, *ak, *av, *att, *agated;
  bf16_t *gates, *probs, *scores, *eg, *eu, *eact, *ey, *sg, *su, *sact, *sy, *gs;
  uint32_t *inds, *lhs, *ident;
  bf16_t *logits, *dlogits;
  float* greedy_scratch;
  uint32_t *ids, *window, *targets, *local, *mailbox;
  bf16_t *vh, *hrow, *dh, *memb, *me, *mh, *mjoined, *mx;
};

// activation scratch of the prompt path: one chunk of up to `cap` rows through the layers
struct WideWs {
  int cap = 0;
  std::vector<void*> allocs;
  uint32_t *ids = nullptr, *lhs = nullptr, *perm = nullptr, *inds = nullptr;
  uint32_t *ident = nullptr, *sorted_e = nullptr, *perm_inv = nullptr;  // ORN_WIDE_EXACT only
  int* seg = nullptr;
  void* gemm_scratch = nullptr;
  void* gdn_scratch = nullptr;  // per-chunk operands of the chunkwise gated-delta recurrence
  bf16_t *x, *n, *r, *h, *n2, *mo;
  bf16_t *cb, *z, *a, *b, *gq, *gk, *gv, *beta, *gy, *gated;
  float* gg;
  bf16_t *qg, *aq, *agate, *ak, *av, *att, *agated;
  bf16_t *gates, *probs, *scores, *sg, *su, *sact, *sy, *gs;
  bf16_t *xs, *eg, *eu, *eact, *ey;
};

}  // namespace ornm

using namespace ornm;

struct orn_model {
  orn_ctx* ctx = nullptr;
  orn_config cfg{};
  std::map<std::string, orn_linear*> lins;
  std::map<std::string, Tensor> tensors;
  orn_linear *embed = nullptr, *lm_head = nullptr;
  bf16_t* norm = nullptr;
  std::vector<Layer> layers;
  Mtp mtp;
  orn_linear* fr_head = nullptr;
  uint32_t* fr_ids = nullptr;  // device
  int fr_n = 0;
  bool fused_ok = true;  // false when a matrix outside the MoE blocks is in a format the fused kernels do not read
  int fr_gen = 0;  // bumped whenever the FR-Spec head is replaced: graphs that drafted through the old one are stale
  bool finalized = false;
  Workspace ws{};
  std::vector<void*> ws_allocs;
  orn_prof prof{};
  cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
  float lnb = 0.f;  // ln(theta) / (rope_dims/2)
  WideWs wide{};    // prompt-chunk scratch, allocated on first use
};

struct orn_cache {
  orn_model* m = nullptr;
  std::vector<bf16_t*> kc, vc;       // per layer (attention layers)
  std::vector<bf16_t*> conv;         // per layer (gdn): [S + kMaxRows, D]
  std::vector<float*> ring;          // per layer (gdn): [kRing][Hv,128,128]
  bf16_t** conv_table = nullptr;     // device array of the conv buffers
  int n_gdn = 0;
  bf16_t *mtp_kc = nullptr, *mtp_vc = nullptr;
  int *pos = nullptr, *cur = nullptr, *mtp_pos = nullptr;  // device scalars
  int h_pos = 0, h_cur = 0, h_mtp_pos = 0;                 // host mirrors
  int cap_T = 0;                                           // rows of the last capture window
  // CUDA graphs of one decode cycle / one autoregressive step, keyed by shape;
  // every kernel argument in them is a fixed address, positions live on the device
  struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    int seen = 0;
    int64_t launches = 0;
    int fr_gen = 0;  // orn_model::fr_gen at capture time (FR-Spec graphs hold the pruned head's addresses)
  };
  std::map<int, StepGraph> graphs;
  uint32_t* mailbox_h = nullptr;  // pinned
};

// resolves every weight name the forward pass needs and builds the scratch (idempotent)
int orn_model_finalize(orn_model* m);
// ORN_WIDE_EXACT=1: wide paths compute their products with the row-invariant mat-vec kernels
bool orn_wide_exact();
int orn_conv_dim(const orn_config& c);
