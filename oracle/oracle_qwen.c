/* TEST INFRASTRUCTURE — CPU oracle, qwen3moe kernels: Q8_K activation quantiser and the
 * Q4_K / Q6_K x Q8_K superblock dots, restating src/bin/engine_qwen2.rs:40-114, 164-200, 287-300.
 * Integer parts are exact; the float update per 256-value superblock is unfused scalar arithmetic
 * in the reference's order.  Build with -ffp-contract=off. */
#include "oracle.h"
#include "oracle_math.h"
#include <math.h>

/* engine_qwen2.rs:40-51 — IEEE half to single, subnormals included */
float orc_half_to_f32(uint16_t h) {
    uint32_t s = (h >> 15) & 1u, e = (h >> 10) & 0x1fu, m = h & 0x3ffu, bits;
    if (e == 0) {
        if (m == 0) bits = s << 31;
        else {
            int ex = -1;
            do { ex++; m <<= 1; } while (!(m & 0x400u));
            bits = (s << 31) | ((uint32_t)(112 - ex) << 23) | ((m & 0x3ffu) << 13);
        }
    } else if (e == 0x1f) bits = (s << 31) | (0xffu << 23) | (m << 13);
    else bits = (s << 31) | ((e + 112u) << 23) | (m << 13);
    return orc_bits2f(bits);
}

/* engine_qwen2.rs:52-56 — 6-bit scale / min of sub-block j from the 12 packed bytes */
void orc_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn) {
    if (j < 4) { *sc = q[j] & 63; *mn = q[j + 4] & 63; }
    else { *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)); *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}

/* engine_qwen2.rs:287-300 — one f32 scale per 256, int8 quants, eight per-32 sums */
void orc_qblock_q8k(const float *xn, int8_t *xq, float *ys, int32_t *xsum, int sb) {
    float amax = 1e-12f;
    for (int i = 0; i < 256; i++) { float a = fabsf(xn[sb * 256 + i]); if (a > amax) amax = a; }
    float sc = amax / 127.0f;
    ys[sb] = sc;
    for (int j = 0; j < 8; j++) {
        int32_t acc = 0;
        for (int i = 0; i < 32; i++) {
            float r = roundf(xn[sb * 256 + j * 32 + i] / sc);
            if (r < -127.0f) r = -127.0f;
            if (r > 127.0f) r = 127.0f;
            int8_t qi = (int8_t)r;
            xq[sb * 256 + j * 32 + i] = qi;
            acc += qi;
        }
        xsum[sb * 8 + j] = acc;
    }
}

void orc_quant_q8k(const float *x, int n, int8_t *q, float *s, int32_t *bsum) {
    for (int sb = 0; sb < n / 256; sb++) orc_qblock_q8k(x, q, s, bsum, sb);
}

/* engine_qwen2.rs:84-114.  dbg (nullable): per superblock {sum of the 4 int32 lanes, mint}. */
float orc_q4k_dot(const uint8_t *row, const int8_t *xq, const float *ys, const int32_t *xsum32, int cols, int32_t *dbg) {
    float sumf = 0.0f;
    for (int sb = 0; sb < cols / 256; sb++) {
        const uint8_t *b = row + (size_t)sb * 144;
        float d = orc_half_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        float dmin = orc_half_to_f32((uint16_t)(b[2] | (b[3] << 8)));
        const uint8_t *qs = b + 16;
        int32_t acc = 0, mint = 0;
        for (int jj = 0; jj < 4; jj++) {
            int j0 = jj * 2, j1 = jj * 2 + 1;
            uint8_t sc0, mn0, sc1, mn1;
            orc_scale_min_k4(j0, b + 4, &sc0, &mn0);
            orc_scale_min_k4(j1, b + 4, &sc1, &mn1);
            int32_t s0 = 0, s1 = 0;
            for (int k = 0; k < 32; k++) {
                s0 += (int32_t)(qs[jj * 32 + k] & 0xF) * xq[(sb * 8 + j0) * 32 + k];
                s1 += (int32_t)(qs[jj * 32 + k] >> 4) * xq[(sb * 8 + j1) * 32 + k];
            }
            acc += s0 * (int32_t)sc0 + s1 * (int32_t)sc1;
            mint += (int32_t)mn0 * xsum32[sb * 8 + j0] + (int32_t)mn1 * xsum32[sb * 8 + j1];
        }
        if (dbg) { dbg[sb * 2] = acc; dbg[sb * 2 + 1] = mint; }
        float ysb = ys[sb];
        sumf += ysb * d * (float)acc - ysb * dmin * (float)mint;
    }
    return sumf;
}

/* engine_qwen2.rs:164-200.  dbg (nullable): per superblock integer accumulator. */
float orc_q6k_dot(const uint8_t *row, const int8_t *xq, const float *ys, int cols, int32_t *dbg) {
    float sumf = 0.0f;
    for (int sb = 0; sb < cols / 256; sb++) {
        const uint8_t *b = row + (size_t)sb * 210;
        const uint8_t *ql = b, *qh = b + 128;
        const int8_t *scp = (const int8_t *)(b + 192);
        float d = orc_half_to_f32((uint16_t)(b[208] | (b[209] << 8)));
        int8_t t[256];
        for (int h = 0; h < 2; h++)
            for (int p = 0; p < 32; p++) {
                uint8_t qla = ql[h * 64 + p], qlb = ql[h * 64 + 32 + p], qhv = qh[h * 32 + p];
                t[h * 128 + p] = (int8_t)(((qla & 0xF) | ((qhv & 3) << 4)) - 32);
                t[h * 128 + 32 + p] = (int8_t)(((qlb & 0xF) | (((qhv >> 2) & 3) << 4)) - 32);
                t[h * 128 + 64 + p] = (int8_t)(((qla >> 4) | (((qhv >> 4) & 3) << 4)) - 32);
                t[h * 128 + 96 + p] = (int8_t)(((qlb >> 4) | ((qhv >> 6) << 4)) - 32);
            }
        int32_t acc = 0;
        for (int s16 = 0; s16 < 16; s16++) {
            int32_t sd = 0;
            for (int i = 0; i < 16; i++) sd += (int32_t)t[s16 * 16 + i] * xq[sb * 256 + s16 * 16 + i];
            acc += sd * (int32_t)scp[s16];
        }
        if (dbg) dbg[sb] = acc;
        sumf += ys[sb] * d * (float)acc;
    }
    return sumf;
}

void orc_q4k_matvec(const uint8_t *w, int rows, int cols, const int8_t *xq, const float *ys, const int32_t *xsum, float *y, int32_t *dbg) {
    size_t bpr = (size_t)cols / 256 * 144;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) y[r] = orc_q4k_dot(w + r * bpr, xq, ys, xsum, cols, dbg ? dbg + (size_t)r * (cols / 256) * 2 : NULL);
}

void orc_q6k_matvec(const uint8_t *w, int rows, int cols, const int8_t *xq, const float *ys, float *y, int32_t *dbg) {
    size_t bpr = (size_t)cols / 256 * 210;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) y[r] = orc_q6k_dot(w + r * bpr, xq, ys, cols, dbg ? dbg + (size_t)r * (cols / 256) : NULL);
}
