/* TEST INFRASTRUCTURE — CPU oracle kernels (see oracle.h).  Build with -ffp-contract=off: the
 * reference's scalar Rust never fuses a*b+c, its NEON vfma always does, and this file calls
 * fmaf exactly where the reference uses vfma. */
#include "oracle.h"
#include "oracle_math.h"
#include <stdlib.h>
#include <float.h>
#include <omp.h>

static const int8_t KVI[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12}; /* engine_gpt2.rs:152 */

float orc_expf_c(float x) { return orc_expf(x); }

/* Worker threads of the parallel loops (the reference runs NT worker threads, engine_gpt2.rs:26-38);
 * set explicitly because launchers such as torchrun export OMP_NUM_THREADS=1.  Results do not
 * depend on it: every loop iteration owns its outputs. */
void orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int orc_max_threads(void) { return omp_get_max_threads(); }

/* vaddvq_f32: pairwise (l0+l1)+(l2+l3) */
static inline float hsum4(const float v[4]) { return (v[0] + v[1]) + (v[2] + v[3]); }

/* engine_gpt2.rs:689-699 — per-32 block int8 quantiser; Rust f32::round = half away from zero */
void orc_qblock32(const float *src, int8_t *xq, float *xsb, int blk) {
    float amax = 1e-12f;
    for (int i = 0; i < 32; i++) { float a = fabsf(src[blk * 32 + i]); if (a > amax) amax = a; }
    float sc = amax / 127.0f;
    xsb[blk] = sc;
    for (int i = 0; i < 32; i++) {
        float r = roundf(src[blk * 32 + i] / sc);
        if (r < -127.0f) r = -127.0f;
        if (r > 127.0f) r = 127.0f;
        xq[blk * 32 + i] = (int8_t)r;
    }
}

void orc_quant_q8(const float *x, int n, int8_t *q, float *s) {
    for (int b = 0; b < n / 32; b++) orc_qblock32(x, q, s, b);
}

/* engine_gpt2.rs:709-726 — 4 NEON accumulators x 4 lanes, fused, stride 16; scalar unfused tail */
float orc_ssq(const float *x, int d) {
    float a[4][4] = {{0}};
    int i = 0;
    while (i + 16 <= d) {
        for (int u = 0; u < 4; u++)
            for (int l = 0; l < 4; l++) { float v = x[i + 4 * u + l]; a[u][l] = fmaf(v, v, a[u][l]); }
        i += 16;
    }
    float v[4];
    for (int l = 0; l < 4; l++) v[l] = (a[0][l] + a[1][l]) + (a[2][l] + a[3][l]);
    float s = hsum4(v);
    while (i < d) { s += x[i] * x[i]; i++; }
    return s;
}

/* engine_gpt2.rs:732-734, 744-746 */
void orc_rmsnorm(const float *x, const float *w, float eps, int d, float *out) {
    float inv = 1.0f / sqrtf(orc_ssq(x, d) / (float)d + eps);
    for (int i = 0; i < d; i++) out[i] = x[i] * inv * w[i];
}

/* engine_gpt2.rs:466-494 */
void orc_q8_from_bf16(const uint16_t *w, int rows, int cols, int8_t *q, float *s) {
    int nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        for (int blk = 0; blk < nb; blk++) {
            float vals[32];
            float amax = 1e-12f;
            for (int i = 0; i < 32; i++) {
                float v = orc_bf16_to_f32(w[(size_t)r * cols + blk * 32 + i]);
                vals[i] = v;
                float a = fabsf(v);
                if (a > amax) amax = a;
            }
            float sc = amax / 127.0f;
            s[(size_t)r * nb + blk] = sc;
            for (int i = 0; i < 32; i++) {
                float t = roundf(vals[i] / sc);
                if (t < -127.0f) t = -127.0f;
                if (t > 127.0f) t = 127.0f;
                q[(size_t)r * cols + blk * 32 + i] = (int8_t)t;
            }
        }
    }
}

/* one sdot pair: lanes j = sum_{i<4} a[4j+i]*b[4j+i] over the two 16-byte halves of a block */
static inline void blockdot_q8(const int8_t *w, const int8_t *x, int32_t t[4]) {
    for (int j = 0; j < 4; j++) {
        int32_t s = 0;
        for (int i = 0; i < 4; i++) s += (int32_t)w[4 * j + i] * x[4 * j + i] + (int32_t)w[16 + 4 * j + i] * x[16 + 4 * j + i];
        t[j] = s;
    }
}

/* engine_gpt2.rs:169-191 — even blocks feed chain 0, odd blocks chain 1; per-lane fused
 * accumulate with the rounded product ws[b]*xs[b]; result vaddv(acc0 + acc1). */
float orc_dot_q8_i8(const int8_t *wq, const float *ws, const int8_t *xq, const float *xsb, int cols) {
    float acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0};
    int nb = cols / 32, b = 0;
    int32_t t[4];
    while (b + 2 <= nb) {
        float s0 = ws[b] * xsb[b], s1 = ws[b + 1] * xsb[b + 1];
        blockdot_q8(wq + b * 32, xq + b * 32, t);
        for (int j = 0; j < 4; j++) acc0[j] = fmaf((float)t[j], s0, acc0[j]);
        blockdot_q8(wq + b * 32 + 32, xq + b * 32 + 32, t);
        for (int j = 0; j < 4; j++) acc1[j] = fmaf((float)t[j], s1, acc1[j]);
        b += 2;
    }
    if (b < nb) {
        float s0 = ws[b] * xsb[b];
        blockdot_q8(wq + b * 32, xq + b * 32, t);
        for (int j = 0; j < 4; j++) acc0[j] = fmaf((float)t[j], s0, acc0[j]);
    }
    float v[4];
    for (int j = 0; j < 4; j++) v[j] = acc0[j] + acc1[j];
    return hsum4(v);
}

void orc_q8_matvec(const int8_t *wq, const float *ws, int rows, int cols, const int8_t *xq, const float *xsb, float *y) {
    int nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) y[r] = orc_dot_q8_i8(wq + (size_t)r * cols, ws + (size_t)r * nb, xq, xsb, cols);
}

/* engine_gpt2.rs:439-461 — GGUF MXFP4 rows (17 B per block: e8m0 byte + 16 nibble bytes) to
 * nib[quad][block][row 0..3][16], exps[quad][block][4] */
void orc_repack_mx(const uint8_t *raw, int rows, int blocks, uint8_t *nib, uint8_t *exps) {
#pragma omp parallel for schedule(static)
    for (int q = 0; q < rows / 4; q++)
        for (int blk = 0; blk < blocks; blk++)
            for (int r = 0; r < 4; r++) {
                const uint8_t *src = raw + ((size_t)(q * 4 + r) * blocks + blk) * 17;
                exps[((size_t)q * blocks + blk) * 4 + r] = src[0];
                memcpy(nib + ((size_t)q * blocks + blk) * 64 + r * 16, src + 1, 16);
            }
}

/* engine_gpt2.rs:194-228 */
void orc_dot4_mx_i8(const uint8_t *nib, const uint8_t *sc, const int8_t *xq, const float *xsb, int blocks, float out[4], int32_t *dbg) {
    float a[4][4] = {{0}};
    for (int b = 0; b < blocks; b++) {
        const int8_t *x0 = xq + b * 32, *x1 = xq + b * 32 + 16;
        for (int r = 0; r < 4; r++) {
            float sv = orc_exp_tbl(sc[b * 4 + r]) * xsb[b];
            const uint8_t *w = nib + (size_t)b * 64 + r * 16;
            for (int j = 0; j < 4; j++) {
                int32_t t = 0;
                for (int i = 0; i < 4; i++)
                    t += (int32_t)KVI[w[4 * j + i] & 0xF] * x0[4 * j + i] + (int32_t)KVI[w[4 * j + i] >> 4] * x1[4 * j + i];
                if (dbg) dbg[(b * 4 + r) * 4 + j] = t;
                a[r][j] = fmaf((float)t, sv, a[r][j]);
            }
        }
    }
    for (int r = 0; r < 4; r++) out[r] = hsum4(a[r]);
}

void orc_mx_matvec(const uint8_t *nib, const uint8_t *exps, int rows, int blocks, const int8_t *xq, const float *xsb, float *y, int32_t *dbg) {
#pragma omp parallel for schedule(static)
    for (int q = 0; q < rows / 4; q++)
        orc_dot4_mx_i8(nib + (size_t)q * blocks * 64, exps + (size_t)q * blocks * 4, xq, xsb, blocks, y + q * 4,
                       dbg ? dbg + (size_t)q * blocks * 16 : NULL);
}

/* value = KVI[nibble] * 2^(e-128); byte j low nibble = element j, high nibble = element j+16
 * (engine.rs:178-182) */
void orc_mx_dequant_row(const uint8_t *raw_row, int blocks, float *out) {
    for (int b = 0; b < blocks; b++) {
        const uint8_t *p = raw_row + b * 17;
        float s = orc_exp_tbl(p[0]);
        for (int j = 0; j < 16; j++) {
            out[b * 32 + j] = (float)KVI[p[1 + j] & 0xF] * s;
            out[b * 32 + 16 + j] = (float)KVI[p[1 + j] >> 4] * s;
        }
    }
}

/* engine_gpt2.rs:536-572 — YaRN table built by rotating (1,0) with the slow path */
void orc_rope_table(const orc_cfg *c, float *tab) {
    int hd = c->hd, half = hd / 2;
    float base = c->rope_base;
    const float PI = 3.14159265358979323846f;
    float lb = logf(base);
    float fd32 = (float)hd * logf(4096.0f / (32.0f * 2.0f * PI)) / (2.0f * lb);
    float fd1 = (float)hd * logf(4096.0f / (1.0f * 2.0f * PI)) / (2.0f * lb);
    float low = floorf(fd32); if (low < 0.0f) low = 0.0f;
    float high = ceilf(fd1); if (high > (float)hd - 1.0f) high = (float)hd - 1.0f;
    float mscale = 1.0f + 0.1f * logf(32.0f);
    float den = high - low; if (den < 0.001f) den = 0.001f;
    for (int pos = 0; pos < ORC_MAXSEQ; pos++)
        for (int i = 0; i < half; i++) {
            float theta_ex = (float)pos * powf(base, -(2.0f * (float)i) / (float)hd);
            float theta_in = theta_ex / 32.0f;
            float y = ((float)i - low) / den;
            if (y < 0.0f) y = 0.0f;
            if (y > 1.0f) y = 1.0f;
            float mix = 1.0f - y;
            float theta = theta_in * (1.0f - mix) + theta_ex * mix;
            float cc = cosf(theta) * mscale, ss = sinf(theta) * mscale;
            /* a = 1, b = 0: v[i] = 1*c - 0*s, v[half+i] = 0*c + 1*s */
            float a = 1.0f, b = 0.0f;
            tab[((size_t)pos * half + i) * 2] = a * cc - b * ss;
            tab[((size_t)pos * half + i) * 2 + 1] = b * cc + a * ss;
        }
}

/* engine_gpt2.rs:575-587 */
void orc_rope_apply(float *v, const float *tab, int pos, int hd) {
    int half = hd / 2;
    const float *t = tab + (size_t)pos * half * 2;
    for (int i = 0; i < half; i++) {
        float c = t[i * 2], s = t[i * 2 + 1];
        float a = v[i], b = v[half + i];
        v[i] = a * c - b * s;
        v[half + i] = b * c + a * s;
    }
}

/* engine_gpt2.rs:849-867 — serial unfused router GEMV, insertion top-k (strict >), softmax over
 * the selected k in rank order */
void orc_router_topk(const float *w, const float *b, const float *xn, int ne, int d, int topk, float *logits, int32_t *top, float *wts) {
#pragma omp parallel for schedule(static)
    for (int e = 0; e < ne; e++) {
        float acc = b ? b[e] : 0.0f;
        for (int j = 0; j < d; j++) acc += w[(size_t)e * d + j] * xn[j];
        logits[e] = acc;
    }
    int tp[8] = {0};
    float tv[8];
    for (int i = 0; i < 8; i++) tv[i] = -FLT_MAX;
    for (int e = 0; e < ne; e++) {
        float v = logits[e];
        if (v > tv[topk - 1]) {
            int p = topk - 1;
            while (p > 0 && tv[p - 1] < v) { tv[p] = tv[p - 1]; tp[p] = tp[p - 1]; p--; }
            tv[p] = v; tp[p] = e;
        }
    }
    float lmax = tv[0], wsum = 0.0f, ex[8];
    for (int i = 0; i < topk; i++) { ex[i] = orc_expf(tv[i] - lmax); wsum += ex[i]; }
    for (int i = 0; i < topk; i++) { wts[i] = ex[i] / wsum; top[i] = tp[i]; }
}

/* engine_gpt2.rs:888-906 — gu[ei][2d] = gate | up; clamped SwiGLU then per-32 Q8 */
void orc_swiglu_quant(const float *gu, int topk, int d, int8_t *hq, float *hsb, float *h_out) {
    const float ALPHA = 1.702f, LIM = 7.0f;
    int nb = d / 32;
    for (int it = 0; it < topk * nb; it++) {
        int ei = it / nb, blk = it % nb;
        const float *g = gu + (size_t)ei * 2 * d + blk * 32;
        const float *u = gu + (size_t)ei * 2 * d + d + blk * 32;
        float h[32];
        float amax = 1e-12f;
        for (int k = 0; k < 32; k++) {
            float xg = g[k] < LIM ? g[k] : LIM;
            float yu = u[k];
            if (yu < -LIM) yu = -LIM;
            if (yu > LIM) yu = LIM;
            float v = (xg / (1.0f + orc_expf(-ALPHA * xg))) * (yu + 1.0f);
            h[k] = v;
            float a = fabsf(v);
            if (a > amax) amax = a;
        }
        float sc = amax / 127.0f;
        hsb[ei * nb + blk] = sc;
        for (int k = 0; k < 32; k++) {
            float r = roundf(h[k] / sc);
            if (r < -127.0f) r = -127.0f;
            if (r > 127.0f) r = 127.0f;
            hq[(size_t)ei * d + blk * 32 + k] = (int8_t)r;
            if (h_out) h_out[(size_t)ei * d + blk * 32 + k] = h[k];
        }
    }
}

/* engine_gpt2.rs:803-833 — one q-head over keys start..=pos; hd must be a multiple of 16 */
void orc_attn_head(const float *q, const float *kc, const float *vc, int nkv, int hd, int kvh, int start, int pos, float sink, float *sc, float *ao) {
    float scale = 1.0f / sqrtf((float)hd);
    for (int t = start; t <= pos; t++) {
        const float *kp = kc + ((size_t)t * nkv + kvh) * hd;
        float a[4][4] = {{0}};
        for (int j = 0; j < hd; j += 16)
            for (int u = 0; u < 4; u++)
                for (int l = 0; l < 4; l++) a[u][l] = fmaf(kp[j + 4 * u + l], q[j + 4 * u + l], a[u][l]);
        float v[4];
        for (int l = 0; l < 4; l++) v[l] = (a[0][l] + a[1][l]) + (a[2][l] + a[3][l]);
        sc[t - start] = hsum4(v) * scale;
    }
    int n = pos - start + 1;
    float mx = sink;
    for (int t = 0; t < n; t++) if (sc[t] > mx) mx = sc[t];
    float den = orc_expf(sink - mx);
    for (int t = 0; t < n; t++) { float e = orc_expf(sc[t] - mx); sc[t] = e; den += e; }
    float acc[256];
    for (int u = 0; u < hd; u++) acc[u] = 0.0f;
    for (int t = start; t <= pos; t++) {
        const float *vp = vc + ((size_t)t * nkv + kvh) * hd;
        float sct = sc[t - start];
        for (int u = 0; u < hd; u++) acc[u] = fmaf(vp[u], sct, acc[u]);
    }
    float inv = 1.0f / den;
    for (int u = 0; u < hd; u++) ao[u] = acc[u] * inv;
}

void orc_moe_ffn_step(const orc_cfg *c, const float *xn, const float *ginp, const float *ginp_b,
                      const orc_quadmx *gate, const orc_quadmx *up, const orc_quadmx *down,
                      const float *gate_b, const float *up_b, const float *down_b,
                      float *x_io, int32_t *top_out, float *wts_out) {
    int d = c->d, nb = d / 32, topk = c->topk, dq = d / 4;
    int8_t *xq = malloc(d); float *xsb = malloc(sizeof(float) * nb);
    float *logits = malloc(sizeof(float) * c->ne);
    float *gu = malloc(sizeof(float) * topk * 2 * d);
    int8_t *hq = malloc((size_t)topk * d); float *hsb = malloc(sizeof(float) * topk * nb);
    int32_t top[8]; float wts[8];
    orc_quant_q8(xn, d, xq, xsb);
    orc_router_topk(ginp, ginp_b, xn, c->ne, d, topk, logits, top, wts);
    /* engine_gpt2.rs:874-883 */
#pragma omp parallel for schedule(static)
    for (int it = 0; it < topk * 2 * dq; it++) {
        int ei = it / (2 * dq), e = top[ei], rem = it % (2 * dq);
        int isup = rem >= dq, qd = isup ? rem - dq : rem;
        const orc_quadmx *w = isup ? up : gate;
        const float *bias = isup ? up_b : gate_b;
        size_t qg = (size_t)e * dq + qd;
        float acc[4];
        orc_dot4_mx_i8(w->nib + qg * nb * 64, w->exps + qg * nb * 4, xq, xsb, nb, acc, NULL);
        for (int i = 0; i < 4; i++) gu[(size_t)ei * 2 * d + (isup ? d : 0) + qd * 4 + i] = acc[i] + bias[(size_t)e * d + qd * 4 + i];
    }
    orc_swiglu_quant(gu, topk, d, hq, hsb, NULL);
    /* engine_gpt2.rs:911-922 */
#pragma omp parallel for schedule(static)
    for (int qd = 0; qd < dq; qd++) {
        float s[4];
        for (int i = 0; i < 4; i++) s[i] = x_io[qd * 4 + i];
        for (int ei = 0; ei < topk; ei++) {
            int e = top[ei];
            size_t qg = (size_t)e * dq + qd;
            float acc[4];
            orc_dot4_mx_i8(down->nib + qg * nb * 64, down->exps + qg * nb * 4, hq + (size_t)ei * d, hsb + ei * nb, nb, acc, NULL);
            for (int i = 0; i < 4; i++) s[i] += wts[ei] * (acc[i] + down_b[(size_t)e * d + qd * 4 + i]);
        }
        for (int i = 0; i < 4; i++) x_io[qd * 4 + i] = s[i];
    }
    for (int i = 0; i < topk; i++) { if (top_out) top_out[i] = top[i]; if (wts_out) wts_out[i] = wts[i]; }
    free(xq); free(xsb); free(logits); free(gu); free(hq); free(hsb);
}
