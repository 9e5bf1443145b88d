/* TEST INFRASTRUCTURE — CPU oracle: a plain-C restatement of the reference engine's per-token
 * MoE decode path (arizqi/cpubrrr, src/bin/engine_gpt2.rs).  It is the checker for the CUDA
 * path and the CPU baseline of the benchmark; it is never linked into the shipped library.
 *
 * Parity pin: the reference stores no golden vectors for this path (its verifier binaries read
 * git-ignored files under /tmp) and cannot be compiled here (Rust + aarch64 NEON + macOS), so
 * this oracle is pinned by (a) the gguf Python package's dequantiser for the MXFP4 format,
 * (b) dequantise-then-dot in float64 within the reference's own verifier thresholds, and
 * (c) the reference's invariants and constants.  Float summation orders follow the NEON lane
 * structure of the reference exactly; integer block dots are exact.
 * The MoE FFN step additionally agrees, to int8-activation quantisation error, with the output of the
 * reference's float64 numpy statement (scripts/ffn_reference.py) run on a seeded synthetic layer
 * (tests/golden/ffn_ref, made by tests/golden/make_ffn_ref_golden.py).
 * The K-quant dots of the qwen3moe path (oracle_qwen.c) ARE pinned by reference-produced data: the
 * reference's plain-C versions (metal/engine_metal.m:589-643), compiled from the reference checkout
 * into _ref/ by the Makefile, produced tests/golden/kq_ref_dots.json, which the oracle matches bit
 * for bit (Q6_K directly; Q4_K through its integer accumulators, the C code using the other of the
 * reference's two float associations).  The forward passes above the kernels are unpinned.
 */
#ifndef ORACLE_H
#define ORACLE_H
#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORC_MAXSEQ 4096

typedef struct {
    int32_t d, nh, nkv, hd, nl, ne, topk, nvocab, swa;
    float rope_base, rms_eps;
} orc_cfg;

/* Q8_0-style matrix quantised from bf16 at load (engine_gpt2.rs:464-494) */
typedef struct { int8_t *q; float *s; int rows, cols; } orc_q8mat;
/* quad-interleaved MXFP4 (engine_gpt2.rs:430-461) */
typedef struct { uint8_t *nib; uint8_t *exps; int rows, blocks; } orc_quadmx;

typedef struct orc_model orc_model;

/* ---- kernels ---- */
float orc_expf_c(float x);
void orc_qblock32(const float *src, int8_t *xq, float *xsb, int blk);
void orc_quant_q8(const float *x, int n, int8_t *q, float *s);
float orc_ssq(const float *x, int d);
void orc_rmsnorm(const float *x, const float *w, float eps, int d, float *out);
void orc_q8_from_bf16(const uint16_t *w, int rows, int cols, int8_t *q, float *s);
float orc_dot_q8_i8(const int8_t *wq, const float *ws, const int8_t *xq, const float *xsb, int cols);
void orc_q8_matvec(const int8_t *wq, const float *ws, int rows, int cols, const int8_t *xq, const float *xsb, float *y);
void orc_repack_mx(const uint8_t *raw, int rows, int blocks, uint8_t *nib, uint8_t *exps);
/* dbg (nullable): int32[blocks][4 rows][4 lanes] block-dot accumulators */
void orc_dot4_mx_i8(const uint8_t *nib, const uint8_t *sc, const int8_t *xq, const float *xsb, int blocks, float out[4], int32_t *dbg);
void orc_mx_matvec(const uint8_t *nib, const uint8_t *exps, int rows, int blocks, const int8_t *xq, const float *xsb, float *y, int32_t *dbg);
void orc_mx_dequant_row(const uint8_t *raw_row, int blocks, float *out);
void orc_rope_table(const orc_cfg *c, float *tab /* [MAXSEQ][hd/2][2] */);
void orc_rope_apply(float *v, const float *tab, int pos, int hd);
void orc_router_topk(const float *w, const float *b, const float *xn, int ne, int d, int topk, float *logits, int32_t *top, float *wts);
void orc_swiglu_quant(const float *gu, int topk, int d, int8_t *hq, float *hsb, float *h_out /*nullable*/);
/* one q-head of decode attention over keys start..pos, then Q8 of the 64 outputs */
void orc_attn_head(const float *q, const float *kc, const float *vc, int nkv, int hd, int kvh, int start, int pos, float sink, float *scores_tmp, float *ao);

/* config-1 step: one MoE FFN on a normalised token xn (engine_gpt2.rs:846-923 minus the norm):
 * quantise xn, route, gate/up, SwiGLU, down + weighted combine onto x_io. */
void orc_moe_ffn_step(const orc_cfg *c, const float *xn, const float *ginp, const float *ginp_b,
                      const orc_quadmx *gate, const orc_quadmx *up, const orc_quadmx *down,
                      const float *gate_b, const float *up_b, const float *down_b,
                      float *x_io, int32_t *top_out, float *wts_out);

/* ---- qwen3moe kernels (src/bin/engine_qwen2.rs) ---- */
float orc_half_to_f32(uint16_t h);
void orc_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn);
void orc_qblock_q8k(const float *xn, int8_t *xq, float *ys, int32_t *xsum, int sb);
void orc_quant_q8k(const float *x, int n, int8_t *q, float *s, int32_t *bsum);
float orc_q4k_dot(const uint8_t *row, const int8_t *xq, const float *ys, const int32_t *xsum32, int cols, int32_t *dbg);
float orc_q6k_dot(const uint8_t *row, const int8_t *xq, const float *ys, int cols, int32_t *dbg);
void orc_q4k_matvec(const uint8_t *w, int rows, int cols, const int8_t *xq, const float *ys, const int32_t *xsum, float *y, int32_t *dbg);
void orc_q6k_matvec(const uint8_t *w, int rows, int cols, const int8_t *xq, const float *ys, float *y, int32_t *dbg);

/* ---- qwen3moe model (oracle_qwen_model.c) ---- */
typedef struct {
    int32_t d, nh, nkv, hd, nl, ne, topk, ff, nvocab;
    float rope_base, rms_eps;
} orcq_cfg;
typedef struct orcq_model orcq_model;
orcq_model *orcq_open_dir(const char *dir, const char *blob);
orcq_model *orcq_open_synth(const orcq_cfg *c, uint64_t seed);
void orcq_close(orcq_model *m);
void orcq_get_cfg(const orcq_model *m, orcq_cfg *out);
/* == run(tok, pos) of engine_qwen2.rs:587; the head runs (and the greedy token returns) when want != 0 */
uint32_t orcq_forward(orcq_model *m, uint32_t tok, uint32_t pos, int want);
const float *orcq_logits(const orcq_model *m);
const float *orcq_hidden(const orcq_model *m);
void orcq_set_trace(orcq_model *m, float *buf);   /* [(nl+1)][d] */
const uint8_t *orcq_layer_k(const orcq_model *m, int il, int which, uint32_t *type, int *rows, int *cols);
const float *orcq_layer_f32(const orcq_model *m, int il, int kind);
void orcq_rope_table(const orcq_cfg *c, float *tab /* [MAXSEQ][hd/2][2] */);
void orcq_rmsnorm(const float *x, const float *w, float eps, int d, float *out);
void orcq_head_norm_rope(float *v, const float *w, int hd, int pos, float eps, const float *tab);
void orcq_attn_head(const float *qh, const float *kcl, const float *vcl, int nkv, int hd, int kvh, int pos, float *sc, float *aop);
void orcq_router_topk(const float *w, const float *xn, int ne, int d, int topk, float *logits, int32_t *top, float *wts);
void orcq_embed_row(const uint8_t *row, int d, float *x);

/* ---- model ---- */
orc_model *orc_open_dir(const char *dir, const char *blob);
orc_model *orc_open_synth(const orc_cfg *c, uint64_t seed);
void orc_close(orc_model *m);
void orc_get_cfg(const orc_model *m, orc_cfg *out);
/* == run(tok,pos,want) of engine_gpt2.rs:1379; returns the greedy token when want != 0 */
uint32_t orc_forward(orc_model *m, uint32_t tok, uint32_t pos, int want);
const float *orc_logits(const orc_model *m);   /* full-Q8 logits of the last want=1 step */
const float *orc_hidden(const orc_model *m);   /* residual stream after the last step */
/* optional trace: x after embed and after each layer, [(nl+1)][d] */
void orc_set_trace(orc_model *m, float *buf);
/* tensors of a layer in run-time form (for stage-level parity tests) */
const orc_q8mat *orc_layer_q8(const orc_model *m, int il, int which /*0 q,1 k,2 v,3 o*/);
const orc_quadmx *orc_layer_mx(const orc_model *m, int il, int which /*0 gate,1 up,2 down*/);
const float *orc_layer_f32(const orc_model *m, int il, int kind /* BRRR_T_* */);
void orc_synth_prompt(uint64_t seed, int n, uint32_t bound, uint32_t *out);
void orc_set_threads(int n);
int orc_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
