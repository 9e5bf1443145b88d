/* TEST INFRASTRUCTURE — CPU oracle: qwen3moe model container, loaders and the single-token forward
 * pass, restating src/bin/engine_qwen2.rs (load: 512-545; forward_worker: 302-451; rmsnorm_par:
 * 453-465; head_norm_rope: 466-482).  Weights stay in the GGUF K-quant byte layout, as in the
 * reference.  The 12-way partial sums of the RMS norm follow the reference's 12 workers; every other
 * float chain is the reference's scalar order.  exp() is the oracle's fixed operation sequence;
 * powf/cosf/sinf of the RoPE angles come from the host libm. */
#include "oracle_src.h"
#include "oracle.h"
#include "oracle_math.h"
#include "../cpubrrr_b200/csrc/brrr_synth.h"
#include <float.h>
#include <math.h>

#define NT 12 /* engine_qwen2.rs:15 */

typedef struct { uint8_t *p; uint32_t type; int rows, cols; size_t bpr; } kmat;

typedef struct {
    float *attn_norm, *ffn_norm, *q_norm, *k_norm, *ginp;
    kmat wq, wk, wv, wo, gate, up, down;
} qlayer;

struct orcq_model {
    orcq_cfg c;
    qlayer *L;
    float *out_norm;
    kmat head, embd;
    float *rope; /* [MAXSEQ][hd/2][2] */
    float *x, *xn, *xs, *q, *k, *v, *ao, *as, *hbuf, *hs, *rlogits, *logits, *scores, *kc, *vc, *trace;
    int8_t *xq, *aq, *hq;
    int32_t *xsum, *asum, *hsum;
};

static const char *qkind_name(int kind) {
    switch (kind) {
    case BRRR_T_ATTN_NORM: return "attn_norm.weight"; case BRRR_T_FFN_NORM: return "ffn_norm.weight";
    case BRRR_T_Q_NORM: return "attn_q_norm.weight"; case BRRR_T_K_NORM: return "attn_k_norm.weight";
    case BRRR_T_WQ: return "attn_q.weight"; case BRRR_T_WK: return "attn_k.weight";
    case BRRR_T_WV: return "attn_v.weight"; case BRRR_T_WO: return "attn_output.weight";
    case BRRR_T_ROUTER_W: return "ffn_gate_inp.weight"; case BRRR_T_GATE: return "ffn_gate_exps.weight";
    case BRRR_T_UP: return "ffn_up_exps.weight"; case BRRR_T_DOWN: return "ffn_down_exps.weight";
    case BRRR_T_TOK_EMBD: return "token_embd.weight"; case BRRR_T_OUT_NORM: return "output_norm.weight";
    case BRRR_T_OUTPUT: return "output.weight";
    }
    return "?";
}

static void tensor_name(char *name, size_t n, int layer, int kind) {
    if (layer == (int)BRRR_L_GLOBAL) snprintf(name, n, "%s", qkind_name(kind));
    else snprintf(name, n, "blk.%d.%s", layer, qkind_name(kind));
}

static float *get_f32(const orc_source *s, int layer, int kind, size_t n) {
    float *out = malloc(sizeof(float) * n);
    if (s->synth) {
        uint64_t key = brrr_tensor_key(s->seed, layer, kind);
        float mean = kind == BRRR_T_ROUTER_W ? 0.0f : 1.0f;
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < n; i++) out[i] = brrr_synth_f32(key, i, mean, 0.02f);
    } else {
        char name[128]; uint32_t ty; size_t nel;
        tensor_name(name, sizeof name, layer, kind);
        const uint8_t *p = orc_source_find(s, name, &ty, &nel);
        if (ty != 0 || nel != n) orc_die("tensor type/size mismatch", name);
        memcpy(out, p, sizeof(float) * n);
    }
    return out;
}

/* K-quant matrix.  Synthetic type scheme: attention, gate/up experts and the embedding Q4_K (12);
 * down experts and the output head Q6_K (14). */
static kmat get_k(const orc_source *s, int layer, int kind, int rows, int cols) {
    kmat m; m.rows = rows; m.cols = cols;
    size_t nsb = (size_t)rows * (cols / 256);
    if (s->synth) {
        m.type = (kind == BRRR_T_DOWN || kind == BRRR_T_OUTPUT) ? 14 : 12;
        size_t bs = m.type == 12 ? 144 : 210;
        m.bpr = (size_t)(cols / 256) * bs;
        m.p = malloc(nsb * bs);
        uint64_t key = brrr_tensor_key(s->seed, layer, kind);
#pragma omp parallel for schedule(static)
        for (size_t b = 0; b < nsb; b++) {
            if (m.type == 12) brrr_synth_q4k_block(key, b, m.p + b * 144);
            else brrr_synth_q6k_block(key, b, m.p + b * 210);
        }
    } else {
        char name[128]; size_t nel;
        tensor_name(name, sizeof name, layer, kind);
        const uint8_t *p = orc_source_find(s, name, &m.type, &nel);
        if (m.type != 12 && m.type != 14) orc_die("tensor is neither Q4_K nor Q6_K", name);   /* engine_qwen2.rs:229 */
        if (nel != (size_t)rows * cols) orc_die("tensor size mismatch", name);
        size_t bs = m.type == 12 ? 144 : 210;
        m.bpr = (size_t)(cols / 256) * bs;
        m.p = malloc(nsb * bs);
        memcpy(m.p, p, nsb * bs);
    }
    return m;
}

static inline float kdot(const kmat *m, size_t row, const int8_t *xq, const float *xs, const int32_t *xsum) {
    const uint8_t *r = m->p + row * m->bpr;
    return m->type == 12 ? orc_q4k_dot(r, xq, xs, xsum, m->cols, NULL) : orc_q6k_dot(r, xq, xs, m->cols, NULL);
}

/* cos/sin of pos * base^(-2i/hd) (engine_qwen2.rs:472-474), tabulated for every position */
void orcq_rope_table(const orcq_cfg *c, float *tab) {
    int half = c->hd / 2;
    for (int i = 0; i < half; i++) {
        float f = powf(c->rope_base, -(2.0f * (float)i) / (float)c->hd);
        for (int pos = 0; pos < ORC_MAXSEQ; pos++) {
            float theta = (float)pos * f;
            tab[((size_t)pos * half + i) * 2] = cosf(theta);
            tab[((size_t)pos * half + i) * 2 + 1] = sinf(theta);
        }
    }
}

static orcq_model *qbuild(const orcq_cfg *c, const orc_source *s) {
    orcq_model *m = calloc(1, sizeof *m);
    m->c = *c;
    int d = c->d, nh = c->nh, nkv = c->nkv, hd = c->hd, ne = c->ne, ff = c->ff;
    if (d % 256 || (nh * hd) % 256 || ff % 256 || hd % 8 || c->topk > ne || nh % nkv) orc_die("unsupported qwen3moe config", NULL);
    m->L = calloc(c->nl, sizeof(qlayer));
    for (int i = 0; i < c->nl; i++) {
        qlayer *l = &m->L[i];
        l->attn_norm = get_f32(s, i, BRRR_T_ATTN_NORM, d);
        l->ffn_norm = get_f32(s, i, BRRR_T_FFN_NORM, d);
        l->q_norm = get_f32(s, i, BRRR_T_Q_NORM, hd);
        l->k_norm = get_f32(s, i, BRRR_T_K_NORM, hd);
        l->wq = get_k(s, i, BRRR_T_WQ, nh * hd, d);
        l->wk = get_k(s, i, BRRR_T_WK, nkv * hd, d);
        l->wv = get_k(s, i, BRRR_T_WV, nkv * hd, d);
        l->wo = get_k(s, i, BRRR_T_WO, d, nh * hd);
        l->ginp = get_f32(s, i, BRRR_T_ROUTER_W, (size_t)ne * d);
        l->gate = get_k(s, i, BRRR_T_GATE, ne * ff, d);
        l->up = get_k(s, i, BRRR_T_UP, ne * ff, d);
        l->down = get_k(s, i, BRRR_T_DOWN, ne * d, ff);
    }
    m->embd = get_k(s, BRRR_L_GLOBAL, BRRR_T_TOK_EMBD, c->nvocab, d);
    if (m->embd.type != 12) orc_die("token embedding must be Q4_K", NULL);   /* engine_qwen2.rs:311 */
    m->out_norm = get_f32(s, BRRR_L_GLOBAL, BRRR_T_OUT_NORM, d);
    m->head = get_k(s, BRRR_L_GLOBAL, BRRR_T_OUTPUT, c->nvocab, d);
    m->rope = malloc(sizeof(float) * ORC_MAXSEQ * hd);
    orcq_rope_table(c, m->rope);
    m->x = calloc(d, 4); m->xn = calloc(d, 4); m->xq = calloc(d, 1); m->xs = calloc(d / 256, 4); m->xsum = calloc(d / 32, 4);
    m->q = calloc(nh * hd, 4); m->k = calloc(nkv * hd, 4); m->v = calloc(nkv * hd, 4); m->ao = calloc(nh * hd, 4);
    m->aq = calloc(nh * hd, 1); m->as = calloc(nh * hd / 256, 4); m->asum = calloc(nh * hd / 32, 4);
    m->hbuf = calloc((size_t)c->topk * ff, 4); m->hq = calloc((size_t)c->topk * ff, 1);
    m->hs = calloc((size_t)c->topk * ff / 256, 4); m->hsum = calloc((size_t)c->topk * ff / 32, 4);
    m->rlogits = calloc(ne, 4); m->logits = calloc(c->nvocab, 4);
    m->scores = calloc((size_t)nh * ORC_MAXSEQ, 4);
    m->kc = calloc((size_t)c->nl * ORC_MAXSEQ * nkv * hd, 4);
    m->vc = calloc((size_t)c->nl * ORC_MAXSEQ * nkv * hd, 4);
    return m;
}

orcq_model *orcq_open_synth(const orcq_cfg *c, uint64_t seed) {
    orc_source s; memset(&s, 0, sizeof s);
    s.synth = 1; s.seed = seed;
    return qbuild(c, &s);
}

/* config.txt keys of engine_qwen2.rs:27-38 */
orcq_model *orcq_open_dir(const char *dir, const char *blobp) {
    orcq_cfg c; memset(&c, 0, sizeof c);
    char v[128];
    struct { const char *k; int32_t *dst; } ints[] = {{"n_embd", &c.d}, {"n_head", &c.nh}, {"n_head_kv", &c.nkv}, {"head_dim", &c.hd},
        {"n_layer", &c.nl}, {"n_expert", &c.ne}, {"n_expert_used", &c.topk}, {"n_ff_exp", &c.ff}, {"n_vocab", &c.nvocab}};
    for (size_t i = 0; i < sizeof ints / sizeof ints[0]; i++) {
        if (!orc_config_get(dir, ints[i].k, v)) orc_die("config.txt lacks", ints[i].k);
        *ints[i].dst = atoi(v);
    }
    if (!orc_config_get(dir, "rope_freq_base", v)) orc_die("config.txt lacks", "rope_freq_base");
    c.rope_base = strtof(v, NULL);
    if (!orc_config_get(dir, "rms_eps", v)) orc_die("config.txt lacks", "rms_eps");
    c.rms_eps = strtof(v, NULL);
    orc_source s;
    orc_source_open(&s, dir, blobp);
    orcq_model *m = qbuild(&c, &s);
    orc_source_close(&s);
    return m;
}

void orcq_close(orcq_model *m) {
    if (!m) return;
    for (int i = 0; i < m->c.nl; i++) {
        qlayer *l = &m->L[i];
        free(l->attn_norm); free(l->ffn_norm); free(l->q_norm); free(l->k_norm); free(l->ginp);
        free(l->wq.p); free(l->wk.p); free(l->wv.p); free(l->wo.p); free(l->gate.p); free(l->up.p); free(l->down.p);
    }
    free(m->L); free(m->out_norm); free(m->head.p); free(m->embd.p); free(m->rope);
    free(m->x); free(m->xn); free(m->xq); free(m->xs); free(m->xsum); free(m->q); free(m->k); free(m->v); free(m->ao);
    free(m->aq); free(m->as); free(m->asum); free(m->hbuf); free(m->hq); free(m->hs); free(m->hsum);
    free(m->rlogits); free(m->logits); free(m->scores); free(m->kc); free(m->vc);
    free(m);
}

void orcq_get_cfg(const orcq_model *m, orcq_cfg *out) { *out = m->c; }
const float *orcq_logits(const orcq_model *m) { return m->logits; }
const float *orcq_hidden(const orcq_model *m) { return m->x; }
void orcq_set_trace(orcq_model *m, float *buf) { m->trace = buf; }
/* tensor access for stage-level tests: which 0 q,1 k,2 v,3 o,4 gate,5 up,6 down; il < 0: 0 head, 1 embedding */
const uint8_t *orcq_layer_k(const orcq_model *m, int il, int which, uint32_t *type, int *rows, int *cols) {
    const kmat *k;
    if (il < 0) k = which == 0 ? &m->head : &m->embd;
    else { qlayer *l = &m->L[il]; const kmat *t[7] = {&l->wq, &l->wk, &l->wv, &l->wo, &l->gate, &l->up, &l->down}; k = t[which]; }
    *type = k->type; *rows = k->rows; *cols = k->cols;
    return k->p;
}
const float *orcq_layer_f32(const orcq_model *m, int il, int kind) {
    if (kind == BRRR_T_OUT_NORM) return m->out_norm;
    qlayer *l = &m->L[il];
    switch (kind) {
    case BRRR_T_ATTN_NORM: return l->attn_norm; case BRRR_T_FFN_NORM: return l->ffn_norm;
    case BRRR_T_Q_NORM: return l->q_norm; case BRRR_T_K_NORM: return l->k_norm; case BRRR_T_ROUTER_W: return l->ginp;
    }
    return NULL;
}

/* worker slice of n items (engine_qwen2.rs:246-252) */
static void sl(int wid, int n, int *a, int *b) {
    int base = n / NT, rem = n % NT;
    *a = wid * base + (wid < rem ? wid : rem);
    *b = *a + base + (wid < rem ? 1 : 0);
}

/* rmsnorm_par (engine_qwen2.rs:453-465): 12 contiguous partial sums, summed in worker order */
void orcq_rmsnorm(const float *x, const float *w, float eps, int d, float *out) {
    float part[NT];
    for (int wid = 0; wid < NT; wid++) {
        int a, b; sl(wid, d, &a, &b);
        float ps = 0.0f;
        for (int i = a; i < b; i++) { float v = x[i]; ps += v * v; }
        part[wid] = ps;
    }
    float tot = 0.0f;
    for (int k = 0; k < NT; k++) tot += part[k];
    float inv = 1.0f / sqrtf(tot / (float)d + eps);
    for (int i = 0; i < d; i++) out[i] = x[i] * inv * w[i];
}

/* head_norm_rope (engine_qwen2.rs:466-482) with the angle table */
void orcq_head_norm_rope(float *v, const float *w, int hd, int pos, float eps, const float *tab) {
    float ms = 0.0f;
    for (int i = 0; i < hd; i++) ms += v[i] * v[i];
    float inv = 1.0f / sqrtf(ms / (float)hd + eps);
    for (int i = 0; i < hd; i++) v[i] = v[i] * inv * w[i];
    int half = hd / 2;
    for (int i = 0; i < half; i++) {
        float co = tab[((size_t)pos * half + i) * 2], si = tab[((size_t)pos * half + i) * 2 + 1];
        float aa = v[i], bb = v[half + i];
        v[i] = aa * co - bb * si;
        v[half + i] = bb * co + aa * si;
    }
}

/* one q-head of full causal attention (engine_qwen2.rs:365-389); cache layout [pos][nkv][hd] */
void orcq_attn_head(const float *qh, const float *kcl, const float *vcl, int nkv, int hd, int kvh, int pos, float *sc, float *aop) {
    float scale = 1.0f / sqrtf((float)hd);
    for (int t = 0; t <= pos; t++) {
        const float *kp = kcl + ((size_t)t * nkv + kvh) * hd;
        float a0[4] = {0, 0, 0, 0}, a1[4] = {0, 0, 0, 0};
        for (int j = 0; j < hd; j += 8)
            for (int l = 0; l < 4; l++) { a0[l] = fmaf(kp[j + l], qh[j + l], a0[l]); a1[l] = fmaf(kp[j + 4 + l], qh[j + 4 + l], a1[l]); }
        float s0 = a0[0] + a1[0], s1 = a0[1] + a1[1], s2 = a0[2] + a1[2], s3 = a0[3] + a1[3];
        sc[t] = ((s0 + s1) + (s2 + s3)) * scale;
    }
    float mx = -FLT_MAX;
    for (int t = 0; t <= pos; t++) if (sc[t] > mx) mx = sc[t];
    float den = 0.0f;
    for (int t = 0; t <= pos; t++) { sc[t] = orc_expf(sc[t] - mx); den += sc[t]; }
    float inv = 1.0f / den;
    for (int j = 0; j < hd; j++) aop[j] = 0.0f;
    for (int t = 0; t <= pos; t++) {
        const float *vp = vcl + ((size_t)t * nkv + kvh) * hd;
        float sct = sc[t];
        for (int j = 0; j < hd; j++) aop[j] = fmaf(vp[j], sct, aop[j]);
    }
    for (int j = 0; j < hd; j++) aop[j] *= inv;
}

/* router (engine_qwen2.rs:405-417): serial unfused logits, stable descending order, softmax over the k */
void orcq_router_topk(const float *w, const float *xn, int ne, int d, int topk, float *logits, int32_t *top, float *wts) {
#pragma omp parallel for schedule(static)
    for (int e = 0; e < ne; e++) {
        float acc = 0.0f;
        for (int j = 0; j < d; j++) acc += w[(size_t)e * d + j] * xn[j];
        logits[e] = acc;
    }
    uint8_t used[1024] = {0};
    for (int i = 0; i < topk; i++) {
        int best = -1;
        for (int e = 0; e < ne; e++) if (!used[e] && (best < 0 || logits[e] > logits[best])) best = e;
        used[best] = 1; top[i] = best;
    }
    float lmax = -FLT_MAX;
    for (int i = 0; i < topk; i++) if (logits[top[i]] > lmax) lmax = logits[top[i]];
    float ex[64], wsum = 0.0f;
    for (int i = 0; i < topk; i++) { ex[i] = orc_expf(logits[top[i]] - lmax); wsum += ex[i]; }
    for (int i = 0; i < topk; i++) wts[i] = ex[i] / wsum;
}

/* Q4_K embedding row (engine_qwen2.rs:310-330) */
void orcq_embed_row(const uint8_t *row, int d, float *x) {
    for (int sb = 0; sb < d / 256; sb++) {
        const uint8_t *bb = row + (size_t)sb * 144;
        float dd = orc_half_to_f32((uint16_t)(bb[0] | (bb[1] << 8))), dmin = orc_half_to_f32((uint16_t)(bb[2] | (bb[3] << 8)));
        const uint8_t *scales = bb + 4, *qs = bb + 16;
        for (int jj = 0; jj < 4; jj++) {
            uint8_t s1, m1, s2, m2;
            orc_scale_min_k4(2 * jj, scales, &s1, &m1);
            orc_scale_min_k4(2 * jj + 1, scales, &s2, &m2);
            for (int l = 0; l < 32; l++) x[sb * 256 + jj * 64 + l] = dd * (float)s1 * (float)(qs[jj * 32 + l] & 0xF) - dmin * (float)m1;
            for (int l = 0; l < 32; l++) x[sb * 256 + jj * 64 + 32 + l] = dd * (float)s2 * (float)(qs[jj * 32 + l] >> 4) - dmin * (float)m2;
        }
    }
}

/* == run(tok, pos) of engine_qwen2.rs:587-595; the head runs when want != 0 */
uint32_t orcq_forward(orcq_model *m, uint32_t tok, uint32_t pos_u, int want) {
    const orcq_cfg c = m->c;
    const int d = c.d, nh = c.nh, nkv = c.nkv, hd = c.hd, ff = c.ff, topk = c.topk, pos = (int)pos_u;
    orcq_embed_row(m->embd.p + (size_t)tok * m->embd.bpr, d, m->x);
    if (m->trace) memcpy(m->trace, m->x, sizeof(float) * d);
    for (int il = 0; il < c.nl; il++) {
        qlayer *ly = &m->L[il];
        float *kcl = m->kc + (size_t)il * ORC_MAXSEQ * nkv * hd, *vcl = m->vc + (size_t)il * ORC_MAXSEQ * nkv * hd;
        orcq_rmsnorm(m->x, ly->attn_norm, c.rms_eps, d, m->xn);
        orc_quant_q8k(m->xn, d, m->xq, m->xs, m->xsum);
#pragma omp parallel for schedule(static)
        for (int r = 0; r < nh * hd + 2 * nkv * hd; r++) {
            if (r < nh * hd) m->q[r] = kdot(&ly->wq, r, m->xq, m->xs, m->xsum);
            else if (r < nh * hd + nkv * hd) m->k[r - nh * hd] = kdot(&ly->wk, r - nh * hd, m->xq, m->xs, m->xsum);
            else m->v[r - nh * hd - nkv * hd] = kdot(&ly->wv, r - nh * hd - nkv * hd, m->xq, m->xs, m->xsum);
        }
        for (int h = 0; h < nh + nkv; h++) {
            if (h < nh) orcq_head_norm_rope(m->q + h * hd, ly->q_norm, hd, pos, c.rms_eps, m->rope);
            else {
                int hh = h - nh;
                orcq_head_norm_rope(m->k + hh * hd, ly->k_norm, hd, pos, c.rms_eps, m->rope);
                memcpy(kcl + ((size_t)pos * nkv + hh) * hd, m->k + hh * hd, sizeof(float) * hd);
                memcpy(vcl + ((size_t)pos * nkv + hh) * hd, m->v + hh * hd, sizeof(float) * hd);
            }
        }
#pragma omp parallel for schedule(dynamic, 1)
        for (int h = 0; h < nh; h++)
            orcq_attn_head(m->q + h * hd, kcl, vcl, nkv, hd, h / (nh / nkv), pos, m->scores + (size_t)h * ORC_MAXSEQ, m->ao + h * hd);
        orc_quant_q8k(m->ao, nh * hd, m->aq, m->as, m->asum);
#pragma omp parallel for schedule(static)
        for (int r = 0; r < d; r++) m->x[r] += kdot(&ly->wo, r, m->aq, m->as, m->asum);
        /* MoE FFN */
        orcq_rmsnorm(m->x, ly->ffn_norm, c.rms_eps, d, m->xn);
        orc_quant_q8k(m->xn, d, m->xq, m->xs, m->xsum);
        int32_t top[64]; float wts[64];
        orcq_router_topk(ly->ginp, m->xn, c.ne, d, topk, m->rlogits, top, wts);
#pragma omp parallel for schedule(static)
        for (int it = 0; it < topk * ff; it++) {
            int ei = it / ff, r = it % ff;
            size_t gr = (size_t)top[ei] * ff + r;
            float g = kdot(&ly->gate, gr, m->xq, m->xs, m->xsum), u = kdot(&ly->up, gr, m->xq, m->xs, m->xsum);
            m->hbuf[it] = (g / (1.0f + orc_expf(-g))) * u;
        }
        orc_quant_q8k(m->hbuf, topk * ff, m->hq, m->hs, m->hsum);
        for (int ei = 0; ei < topk; ei++) {
            const int8_t *hq = m->hq + (size_t)ei * ff; const float *hs = m->hs + (size_t)ei * (ff / 256); const int32_t *hm = m->hsum + (size_t)ei * (ff / 32);
            float w = wts[ei]; size_t base = (size_t)top[ei] * d;
#pragma omp parallel for schedule(static)
            for (int r = 0; r < d; r++) m->x[r] += w * kdot(&ly->down, base + r, hq, hs, hm);
        }
        if (m->trace) memcpy(m->trace + (size_t)(il + 1) * d, m->x, sizeof(float) * d);
    }
    if (!want) return 0;
    orcq_rmsnorm(m->x, m->out_norm, c.rms_eps, d, m->xn);
    orc_quant_q8k(m->xn, d, m->xq, m->xs, m->xsum);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < c.nvocab; r++) m->logits[r] = kdot(&m->head, r, m->xq, m->xs, m->xsum);
    float best = -FLT_MAX; uint32_t bi = 0;   /* f32::MIN start, strict > (engine_qwen2.rs:439-448) */
    for (int i = 0; i < c.nvocab; i++) if (m->logits[i] > best) { best = m->logits[i]; bi = i; }
    return bi;
}
