/* TEST INFRASTRUCTURE — CPU oracle: gpt-oss model container, loaders and the single-token
 * forward pass, restating src/bin/engine_gpt2.rs (load: 1276-1315; forward_worker: 751-934;
 * head semantics: full-Q8 argmax, first strict maximum, as in sample_logits 95-100). */
#include "oracle_src.h"
#include "oracle.h"
#include "oracle_math.h"
#include "../cpubrrr_b200/csrc/brrr_synth.h"
#include <stdio.h>
#include <stdlib.h>
#include <float.h>

typedef struct {
    float *attn_norm, *ffn_norm;
    orc_q8mat wq, wk, wv, wo;
    float *bq, *bk, *bv, *bo, *sinks, *ginp, *ginp_b;
    orc_quadmx gate, up, down;
    float *gate_b, *up_b, *down_b;
} orc_layer;

struct orc_model {
    orc_cfg c;
    orc_layer *L;
    float *out_norm;
    orc_q8mat head;
    uint16_t *tok_embd;
    float *rope;
    /* activations (engine_gpt2.rs:1340-1347) */
    float *x, *xn, *xsb, *q, *k, *v, *ao, *asb, *gu, *hsb, *rlogits, *logits, *scores;
    int8_t *xq, *aq, *hq;
    float *kc, *vc;
    float *trace;
};

/* ------------------------------------------------------------------ tensor sources */
typedef orc_source source;

static const char *kind_name(int kind) {
    switch (kind) {
    case BRRR_T_ATTN_NORM: return "attn_norm.weight"; case BRRR_T_FFN_NORM: return "ffn_norm.weight";
    case BRRR_T_WQ: return "attn_q.weight"; case BRRR_T_WK: return "attn_k.weight";
    case BRRR_T_WV: return "attn_v.weight"; case BRRR_T_WO: return "attn_out.weight";
    case BRRR_T_BQ: return "attn_q.bias"; case BRRR_T_BK: return "attn_k.bias";
    case BRRR_T_BV: return "attn_v.bias"; case BRRR_T_BO: return "attn_out.bias";
    case BRRR_T_SINKS: return "attn_sinks"; case BRRR_T_ROUTER_W: return "ffn_gate_inp.weight";
    case BRRR_T_ROUTER_B: return "ffn_gate_inp.bias"; case BRRR_T_GATE: return "ffn_gate_exps.weight";
    case BRRR_T_UP: return "ffn_up_exps.weight"; case BRRR_T_DOWN: return "ffn_down_exps.weight";
    case BRRR_T_GATE_B: return "ffn_gate_exps.bias"; case BRRR_T_UP_B: return "ffn_up_exps.bias";
    case BRRR_T_DOWN_B: return "ffn_down_exps.bias";
    case BRRR_T_TOK_EMBD: return "token_embd.weight"; case BRRR_T_OUT_NORM: return "output_norm.weight";
    case BRRR_T_OUTPUT: return "output.weight";
    }
    return "?";
}

#define die orc_die

static const uint8_t *file_tensor(const source *s, int layer, int kind, uint32_t want_type, size_t nel) {
    char name[128];
    if (layer == (int)BRRR_L_GLOBAL) snprintf(name, sizeof name, "%s", kind_name(kind));
    else snprintf(name, sizeof name, "blk.%d.%s", layer, kind_name(kind));
    uint32_t ty; size_t n;
    const uint8_t *p = orc_source_find(s, name, &ty, &n);
    if (ty != want_type) die("tensor type mismatch", name);
    if (n != nel) die("tensor size mismatch", name);
    return p;
}

/* f32 tensor: synthetic mean/sigma follow the seeded-input recipe: norms 1+N(0,.02), sinks N(0,1),
 * everything else N(0,.02) */
static float *get_f32(const source *s, int layer, int kind, size_t n) {
    float *out = malloc(sizeof(float) * n);
    if (s->synth) {
        uint64_t key = brrr_tensor_key(s->seed, layer, kind);
        float mean = (kind == BRRR_T_ATTN_NORM || kind == BRRR_T_FFN_NORM || kind == BRRR_T_OUT_NORM) ? 1.0f : 0.0f;
        float sigma = kind == BRRR_T_SINKS ? 1.0f : 0.02f;
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < n; i++) out[i] = brrr_synth_f32(key, i, mean, sigma);
    } else memcpy(out, file_tensor(s, layer, kind, 0, n), sizeof(float) * n);
    return out;
}

static uint16_t *get_bf16(const source *s, int layer, int kind, size_t n) {
    uint16_t *out = malloc(sizeof(uint16_t) * n);
    if (s->synth) {
        uint64_t key = brrr_tensor_key(s->seed, layer, kind);
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < n; i++) out[i] = brrr_synth_bf16(key, i, 0.02f);
    } else memcpy(out, file_tensor(s, layer, kind, 30, n), sizeof(uint16_t) * n);
    return out;
}

static orc_q8mat get_q8(const source *s, int layer, int kind, int rows, int cols) {
    orc_q8mat m = {malloc((size_t)rows * cols), malloc(sizeof(float) * rows * (cols / 32)), rows, cols};
    uint16_t *w = get_bf16(s, layer, kind, (size_t)rows * cols);
    orc_q8_from_bf16(w, rows, cols, m.q, m.s);
    free(w);
    return m;
}

static orc_quadmx get_mx(const source *s, int layer, int kind, int rows, int blocks) {
    orc_quadmx m = {malloc((size_t)rows * blocks * 16), malloc((size_t)rows * blocks), rows, blocks};
    size_t nblk = (size_t)rows * blocks;
    if (s->synth) {
        uint8_t *raw = malloc(nblk * 17);
        uint64_t key = brrr_tensor_key(s->seed, layer, kind);
#pragma omp parallel for schedule(static)
        for (size_t b = 0; b < nblk; b++) brrr_synth_mxfp4_block(key, b, raw + b * 17);
        orc_repack_mx(raw, rows, blocks, m.nib, m.exps);
        free(raw);
    } else orc_repack_mx(file_tensor(s, layer, kind, 39, nblk * 32), rows, blocks, m.nib, m.exps);
    return m;
}

static orc_model *build(const orc_cfg *c, const source *s) {
    orc_model *m = calloc(1, sizeof *m);
    m->c = *c;
    int d = c->d, nh = c->nh, nkv = c->nkv, hd = c->hd, nb = d / 32, ne = c->ne;
    if (d % 64 || hd % 16 || (nh * hd) % 64 || c->topk > 8 || c->topk > ne) die("unsupported config", NULL);
    m->L = calloc(c->nl, sizeof(orc_layer));
    for (int i = 0; i < c->nl; i++) {
        orc_layer *l = &m->L[i];
        l->attn_norm = get_f32(s, i, BRRR_T_ATTN_NORM, d);
        l->ffn_norm = get_f32(s, i, BRRR_T_FFN_NORM, d);
        l->wq = get_q8(s, i, BRRR_T_WQ, nh * hd, d);
        l->wk = get_q8(s, i, BRRR_T_WK, nkv * hd, d);
        l->wv = get_q8(s, i, BRRR_T_WV, nkv * hd, d);
        l->wo = get_q8(s, i, BRRR_T_WO, d, nh * hd);
        l->bq = get_f32(s, i, BRRR_T_BQ, nh * hd);
        l->bk = get_f32(s, i, BRRR_T_BK, nkv * hd);
        l->bv = get_f32(s, i, BRRR_T_BV, nkv * hd);
        l->bo = get_f32(s, i, BRRR_T_BO, d);
        l->sinks = get_f32(s, i, BRRR_T_SINKS, nh);
        l->ginp = get_f32(s, i, BRRR_T_ROUTER_W, (size_t)ne * d);
        l->ginp_b = get_f32(s, i, BRRR_T_ROUTER_B, ne);
        l->gate = get_mx(s, i, BRRR_T_GATE, ne * d, nb);
        l->up = get_mx(s, i, BRRR_T_UP, ne * d, nb);
        l->down = get_mx(s, i, BRRR_T_DOWN, ne * d, nb);
        l->gate_b = get_f32(s, i, BRRR_T_GATE_B, (size_t)ne * d);
        l->up_b = get_f32(s, i, BRRR_T_UP_B, (size_t)ne * d);
        l->down_b = get_f32(s, i, BRRR_T_DOWN_B, (size_t)ne * d);
    }
    m->tok_embd = get_bf16(s, BRRR_L_GLOBAL, BRRR_T_TOK_EMBD, (size_t)c->nvocab * d);
    m->out_norm = get_f32(s, BRRR_L_GLOBAL, BRRR_T_OUT_NORM, d);
    m->head = get_q8(s, BRRR_L_GLOBAL, BRRR_T_OUTPUT, c->nvocab, d);
    m->rope = malloc(sizeof(float) * ORC_MAXSEQ * hd);
    orc_rope_table(c, m->rope);
    m->x = calloc(d, 4); m->xn = calloc(d, 4); m->xq = calloc(d, 1); m->xsb = calloc(nb, 4);
    m->q = calloc(nh * hd, 4); m->k = calloc(nkv * hd, 4); m->v = calloc(nkv * hd, 4); m->ao = calloc(nh * hd, 4);
    m->aq = calloc(nh * hd, 1); m->asb = calloc(nh * hd / 32, 4);
    m->gu = calloc((size_t)c->topk * 2 * d, 4); m->hq = calloc((size_t)c->topk * d, 1); m->hsb = calloc((size_t)c->topk * nb, 4);
    m->rlogits = calloc(ne, 4); m->logits = calloc(c->nvocab, 4);
    m->scores = calloc((size_t)nh * ORC_MAXSEQ, 4);
    m->kc = calloc((size_t)c->nl * ORC_MAXSEQ * nkv * hd, 4);
    m->vc = calloc((size_t)c->nl * ORC_MAXSEQ * nkv * hd, 4);
    return m;
}

orc_model *orc_open_synth(const orc_cfg *c, uint64_t seed) {
    source s = {0};
    s.synth = 1; s.seed = seed;
    return build(c, &s);
}

/* data-directory contract: config.txt (engine_gpt2.rs:64-80), manifest.txt (1279-1284) */
orc_model *orc_open_dir(const char *dir, const char *blobp) {
    char path[4096], key[128], val[128];
    orc_cfg c; memset(&c, 0, sizeof c);
    c.swa = 1 << 30;
    int ffexp = -1;
    snprintf(path, sizeof path, "%s/config.txt", dir);
    FILE *f = fopen(path, "r");
    if (!f) die("cannot open", path);
    char line[512];
    while (fgets(line, sizeof line, f)) {
        if (sscanf(line, "%127s %127s", key, val) != 2) continue;
        if (!strcmp(key, "n_embd")) c.d = atoi(val); else if (!strcmp(key, "n_layer")) c.nl = atoi(val);
        else if (!strcmp(key, "n_head")) c.nh = atoi(val); else if (!strcmp(key, "n_head_kv")) c.nkv = atoi(val);
        else if (!strcmp(key, "head_dim")) c.hd = atoi(val); else if (!strcmp(key, "n_expert")) c.ne = atoi(val);
        else if (!strcmp(key, "n_expert_used")) c.topk = atoi(val); else if (!strcmp(key, "n_ff_exp")) ffexp = atoi(val);
        else if (!strcmp(key, "sliding_window")) c.swa = atoi(val); else if (!strcmp(key, "n_vocab")) c.nvocab = atoi(val);
        else if (!strcmp(key, "rope_freq_base")) c.rope_base = strtof(val, NULL);
        else if (!strcmp(key, "rms_eps")) c.rms_eps = strtof(val, NULL);
    }
    fclose(f);
    if (ffexp != c.d) die("engine assumes expert ff dim == d", NULL);   /* engine_gpt2.rs:73 */
    if (c.hd != 64) die("attention kernels assume hd=64", NULL);        /* engine_gpt2.rs:74 */
    source s;
    orc_source_open(&s, dir, blobp);
    orc_model *m = build(&c, &s);
    orc_source_close(&s);
    return m;
}

static void free_q8(orc_q8mat *m) { free(m->q); free(m->s); }
static void free_mx(orc_quadmx *m) { free(m->nib); free(m->exps); }
void orc_close(orc_model *m) {
    if (!m) return;
    for (int i = 0; i < m->c.nl; i++) {
        orc_layer *l = &m->L[i];
        free(l->attn_norm); free(l->ffn_norm); free_q8(&l->wq); free_q8(&l->wk); free_q8(&l->wv); free_q8(&l->wo);
        free(l->bq); free(l->bk); free(l->bv); free(l->bo); free(l->sinks); free(l->ginp); free(l->ginp_b);
        free_mx(&l->gate); free_mx(&l->up); free_mx(&l->down); free(l->gate_b); free(l->up_b); free(l->down_b);
    }
    free(m->L); free(m->out_norm); free_q8(&m->head); free(m->tok_embd); free(m->rope);
    free(m->x); free(m->xn); free(m->xq); free(m->xsb); free(m->q); free(m->k); free(m->v); free(m->ao);
    free(m->aq); free(m->asb); free(m->gu); free(m->hq); free(m->hsb); free(m->rlogits); free(m->logits);
    free(m->scores); free(m->kc); free(m->vc);
    free(m);
}

void orc_get_cfg(const orc_model *m, orc_cfg *out) { *out = m->c; }
const float *orc_logits(const orc_model *m) { return m->logits; }
const float *orc_hidden(const orc_model *m) { return m->x; }
void orc_set_trace(orc_model *m, float *buf) { m->trace = buf; }
const orc_q8mat *orc_layer_q8(const orc_model *m, int il, int which) {
    if (il < 0) return &m->head;
    orc_layer *l = &m->L[il];
    return which == 0 ? &l->wq : which == 1 ? &l->wk : which == 2 ? &l->wv : &l->wo;
}
const orc_quadmx *orc_layer_mx(const orc_model *m, int il, int which) {
    orc_layer *l = &m->L[il];
    return which == 0 ? &l->gate : which == 1 ? &l->up : &l->down;
}
const float *orc_layer_f32(const orc_model *m, int il, int kind) {
    if (kind == BRRR_T_OUT_NORM) return m->out_norm;
    orc_layer *l = &m->L[il];
    switch (kind) {
    case BRRR_T_ATTN_NORM: return l->attn_norm; case BRRR_T_FFN_NORM: return l->ffn_norm;
    case BRRR_T_BQ: return l->bq; case BRRR_T_BK: return l->bk; case BRRR_T_BV: return l->bv; case BRRR_T_BO: return l->bo;
    case BRRR_T_SINKS: return l->sinks; case BRRR_T_ROUTER_W: return l->ginp; case BRRR_T_ROUTER_B: return l->ginp_b;
    case BRRR_T_GATE_B: return l->gate_b; case BRRR_T_UP_B: return l->up_b; case BRRR_T_DOWN_B: return l->down_b;
    }
    return NULL;
}
void orc_synth_prompt(uint64_t seed, int n, uint32_t bound, uint32_t *out) {
    uint64_t key = brrr_tensor_key(seed, BRRR_L_GLOBAL, BRRR_T_PROMPT);
    for (int i = 0; i < n; i++) out[i] = brrr_synth_token(key, i, bound);
}

/* ------------------------------------------------------------------ forward (engine_gpt2.rs:751-934) */
uint32_t orc_forward(orc_model *m, uint32_t tok, uint32_t pos_u, int want) {
    const orc_cfg c = m->c;
    const int d = c.d, nh = c.nh, nkv = c.nkv, hd = c.hd, nb = d / 32, topk = c.topk, dq = d / 4;
    const int pos = (int)pos_u;
    for (int j = 0; j < d; j++) m->x[j] = orc_bf16_to_f32(m->tok_embd[(size_t)tok * d + j]);
    if (m->trace) memcpy(m->trace, m->x, sizeof(float) * d);
    for (int il = 0; il < c.nl; il++) {
        orc_layer *ly = &m->L[il];
        float *kcl = m->kc + (size_t)il * ORC_MAXSEQ * nkv * hd;
        float *vcl = m->vc + (size_t)il * ORC_MAXSEQ * nkv * hd;
        /* attn rmsnorm + quant (773) */
        orc_rmsnorm(m->x, ly->attn_norm, c.rms_eps, d, m->xn);
        orc_quant_q8(m->xn, d, m->xq, m->xsb);
        /* qkv + bias + rope + cache write (779-797) */
#pragma omp parallel for schedule(dynamic, 1)
        for (int h = 0; h < nh + nkv; h++) {
            if (h < nh) {
                int base = h * hd;
                for (int r = 0; r < hd; r++)
                    m->q[base + r] = orc_dot_q8_i8(ly->wq.q + (size_t)(base + r) * d, ly->wq.s + (size_t)(base + r) * nb, m->xq, m->xsb, d) + ly->bq[base + r];
                orc_rope_apply(m->q + base, m->rope, pos, hd);
            } else {
                int hh = h - nh, base = hh * hd;
                for (int r = 0; r < hd; r++) {
                    m->k[base + r] = orc_dot_q8_i8(ly->wk.q + (size_t)(base + r) * d, ly->wk.s + (size_t)(base + r) * nb, m->xq, m->xsb, d) + ly->bk[base + r];
                    m->v[base + r] = orc_dot_q8_i8(ly->wv.q + (size_t)(base + r) * d, ly->wv.s + (size_t)(base + r) * nb, m->xq, m->xsb, d) + ly->bv[base + r];
                }
                orc_rope_apply(m->k + base, m->rope, pos, hd);
                for (int j = 0; j < hd; j++) {
                    kcl[((size_t)pos * nkv + hh) * hd + j] = m->k[base + j];
                    vcl[((size_t)pos * nkv + hh) * hd + j] = m->v[base + j];
                }
            }
        }
        /* attention; sliding window on even layer index (801-837) */
        int start = ((il + 1) % 2 != 0) ? (pos >= c.swa - 1 ? pos - (c.swa - 1) : 0) : 0;
#pragma omp parallel for schedule(dynamic, 1)
        for (int h = 0; h < nh; h++) {
            int kvh = h / (nh / nkv);
            orc_attn_head(m->q + h * hd, kcl, vcl, nkv, hd, kvh, start, pos, ly->sinks[h], m->scores + (size_t)h * ORC_MAXSEQ, m->ao + h * hd);
            for (int b = 0; b < hd / 32; b++) orc_qblock32(m->ao, m->aq, m->asb, h * (hd / 32) + b);
        }
        /* o-proj + bias + residual (840) */
        int ocols = nh * hd, onb = ocols / 32;
#pragma omp parallel for schedule(static)
        for (int r = 0; r < d; r++)
            m->x[r] += orc_dot_q8_i8(ly->wo.q + (size_t)r * ocols, ly->wo.s + (size_t)r * onb, m->aq, m->asb, ocols) + ly->bo[r];
        /* MoE FFN (846-923) */
        orc_rmsnorm(m->x, ly->ffn_norm, c.rms_eps, d, m->xn);
        orc_moe_ffn_step(&c, m->xn, ly->ginp, ly->ginp_b, &ly->gate, &ly->up, &ly->down, ly->gate_b, ly->up_b, ly->down_b, m->x, NULL, NULL);
        if (m->trace) memcpy(m->trace + (size_t)(il + 1) * d, m->x, sizeof(float) * d);
    }
    (void)topk; (void)dq;
    if (!want) return 0;
    /* head: rmsnorm + quant (948), full-Q8 logits, first strict max */
    orc_rmsnorm(m->x, m->out_norm, c.rms_eps, d, m->xn);
    orc_quant_q8(m->xn, d, m->xq, m->xsb);
    orc_q8_matvec(m->head.q, m->head.s, c.nvocab, d, m->xq, m->xsb, m->logits);
    float best = -FLT_MAX; uint32_t bi = 0;
    for (int i = 0; i < c.nvocab; i++) if (m->logits[i] > best) { best = m->logits[i]; bi = i; }
    return bi;
}
