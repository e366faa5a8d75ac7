// Launchers of the persistent fused kernels (fused.cu).
#pragma once

#include "orn_internal.h"

enum { PRO_ADDNORM = 0, PRO_PLAIN = 1, PRO_GATED = 2, PRO_MTPJOIN = 3 };
enum { EPI_STORE = 0, EPI_SWIGLU = 1 };

// How a kernel rebuilds its input row(s) in shared memory.
struct FusedPrologue {
  int mode = PRO_PLAIN;
  int K = 0;                      // length of the staged row
  const bf16_t* a = nullptr;      // ADDNORM/PLAIN: [M][K]; GATED: y [M][K]; MTPJOIN: trunk hidden [M][K/2]
  const bf16_t* b = nullptr;      // ADDNORM: second addend (nullable); GATED: z [M][K]
  const bf16_t* w = nullptr;      // norm weight (GATED: [128]; MTPJOIN: embedding-side norm)
  const bf16_t* w2 = nullptr;     // MTPJOIN: hidden-side norm
  bf16_t* sum_out = nullptr;      // ADDNORM: bf(a+b) written by CTA 0
  bf16_t* norm_out = nullptr;     // staged row written by CTA 0
  const orn_linear* emb = nullptr;  // MTPJOIN: embedding table
  const uint32_t* ids = nullptr;    // MTPJOIN: token ids (device)
  float eps = 1e-6f;
};

struct FusedJob {
  const orn_linear* lin = nullptr;
  const orn_linear* lin2 = nullptr;  // EPI_SWIGLU: the "up" matrix
  bf16_t* out = nullptr;             // [M][O]
  int epi = EPI_STORE;
};

int f_norm_gemv(orn_ctx* ctx, cudaStream_t s, int M, const FusedPrologue& fp, const FusedJob* jobs, int njobs);
int f_moe_up(orn_ctx* ctx, cudaStream_t s, int M, const bf16_t* logits, const bf16_t* x, const orn_linear* gate,
             const orn_linear* up, int k, uint32_t* inds, bf16_t* scores, bf16_t* act);
int f_moe_down(orn_ctx* ctx, cudaStream_t s, int M, const bf16_t* act, const bf16_t* sact, const uint32_t* inds,
               const bf16_t* scores, const bf16_t* gs, const orn_linear* down, const orn_linear* sh_down, int k,
               int normalize, bf16_t* out);
int f_gdn(orn_ctx* ctx, cudaStream_t s, const bf16_t* conv, const bf16_t* cw, const bf16_t* a, const bf16_t* b,
          const bf16_t* a_log, const bf16_t* dt_bias, float* ring, int nring, const int* cur, int final_only, int T,
          int Hk, int Hv, int Kc, float eps, bf16_t* y, const bf16_t* z, const bf16_t* norm_w, float norm_eps,
          bf16_t* gated_out /* nullable: rms_norm_gated(y, z) per head, by the last CTA of the head */);
int f_attn(orn_ctx* ctx, cudaStream_t s, const bf16_t* qg, const bf16_t* k, const bf16_t* v, const bf16_t* q_norm,
           const bf16_t* k_norm, bf16_t* kc, bf16_t* vc, const int* pos, int T, int Hq, int Hkv, int hd, int cap,
           int rope_dims, float lnb, float eps, bf16_t* out,
           int long_context = 0 /* the key groups of a (head, row) over four CTAs: same bits, for long caches */);
// one warp waits, with a limit of `rounds` tries, for a copy that was never requested: sets the
// context's device error flag; *dev_waited receives 0
int f_wait_probe(orn_ctx* ctx, cudaStream_t s, uint32_t rounds, int* dev_waited);

// ---- gemm.cu: the wide (>= 16 rows) mat-mul on the tensor cores
struct QGemmGroup {
  const int* seg;           // device [E + 1]: expert e owns sorted rows seg[e] .. seg[e+1]-1
  const uint32_t* row_map;  // device [rows] or null: output row of sorted row p
  int bn_hint;              // > 0: expected rows per expert (picks the token-tile width)
};
size_t qgemm_scratch_bytes(int rows, int E, int O);
int f_qgemm(orn_ctx* ctx, cudaStream_t s, const orn_linear* L, const bf16_t* x, int rows, void* y, int ldy,
            const QGemmGroup* grp /*nullable: dense*/, void* scratch /*grouped only*/, int out_f32 = 0,
            int bn_force = 0 /*> 0: token-tile width (multiple of 16, <= 256)*/);
// up to four matrices of one format and row length over the same rows in one dense launch
int f_qgemm_multi(orn_ctx* ctx, cudaStream_t s, const orn_linear* const* Ls, void* const* ys, const int* ldys, int n,
                  const bf16_t* x, int rows, const QGemmGroup* grp = nullptr, void* scratch = nullptr, int out_f32 = 0,
                  int bn_force = 0);
int f_route_sort(orn_ctx* ctx, cudaStream_t s, const uint32_t* rhs, int rows, int E, int* seg, int* cursor, uint32_t* perm);
int f_gather_rows(orn_ctx* ctx, cudaStream_t s, const bf16_t* x, const uint32_t* lhs /*nullable*/, const uint32_t* perm,
                  int rows, int K, bf16_t* xs);
