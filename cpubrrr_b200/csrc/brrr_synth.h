/* Counter-based synthetic tensor generator.
 *
 * Every byte of a synthetic model is a pure function of (seed, layer, tensor kind, element
 * index), built from integer arithmetic and single IEEE float operations only, so that plain
 * C on the host, CUDA device code and a numpy port produce the same bytes.  No tensor ever has
 * to be materialised on the host to fill the device, and a CPU checker can regenerate any
 * tensor it needs.
 *
 * The generator emits tensors in the GGUF on-disk formats the engine reads
 * (f32, bf16, MXFP4 17-byte blocks, Q4_K 144-byte and Q6_K 210-byte superblocks), i.e. the same bytes a data directory's blob would hold.
 *
 * This header is C99 / C++ / CUDA compatible and has no dependencies.
 */
#ifndef BRRR_SYNTH_H
#define BRRR_SYNTH_H

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define BRRR_HD __host__ __device__ static inline
#else
#define BRRR_HD static inline
#endif

/* tensor kinds (per layer unless marked global) */
enum {
    BRRR_T_ATTN_NORM = 0, BRRR_T_FFN_NORM = 1,
    BRRR_T_WQ = 2, BRRR_T_WK = 3, BRRR_T_WV = 4, BRRR_T_WO = 5,
    BRRR_T_BQ = 6, BRRR_T_BK = 7, BRRR_T_BV = 8, BRRR_T_BO = 9,
    BRRR_T_SINKS = 10, BRRR_T_ROUTER_W = 11, BRRR_T_ROUTER_B = 12,
    BRRR_T_GATE = 13, BRRR_T_UP = 14, BRRR_T_DOWN = 15,
    BRRR_T_GATE_B = 16, BRRR_T_UP_B = 17, BRRR_T_DOWN_B = 18,
    BRRR_T_Q_NORM = 19, BRRR_T_K_NORM = 20,
    /* global tensors use layer = BRRR_L_GLOBAL */
    BRRR_T_TOK_EMBD = 32, BRRR_T_OUT_NORM = 33, BRRR_T_OUTPUT = 34,
    BRRR_T_PROMPT = 40, BRRR_T_INPUT = 41
};
#define BRRR_L_GLOBAL 0xFFFFu

#define BRRR_PHI 0x9E3779B97F4A7C15ull

/* splitmix64 output function */
BRRR_HD uint64_t brrr_mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* one independent stream per (seed, layer, kind) */
BRRR_HD uint64_t brrr_tensor_key(uint64_t seed, uint32_t layer, uint32_t kind) {
    return brrr_mix64(brrr_mix64(seed + BRRR_PHI) ^ ((((uint64_t)layer << 8) | kind) * BRRR_PHI));
}

/* idx-th 64-bit draw of a stream */
BRRR_HD uint64_t brrr_draw(uint64_t key, uint64_t idx) {
    return brrr_mix64(key + (idx + 1) * BRRR_PHI);
}

BRRR_HD uint32_t brrr_bytesum64(uint64_t x) {
    x = (x & 0x00FF00FF00FF00FFull) + ((x >> 8) & 0x00FF00FF00FF00FFull);
    x = (x & 0x0000FFFF0000FFFFull) + ((x >> 16) & 0x0000FFFF0000FFFFull);
    return (uint32_t)((x + (x >> 32)) & 0xFFFFu);
}

/* Approximately standard-normal draw: the centred sum of 16 uniform bytes (Irwin-Hall, n = 16),
 * scaled to unit variance.  Support is +-6.9 sigma, excess kurtosis -0.075.  Two draws per
 * element; the result is one int->float convert and one float multiply, hence reproducible. */
BRRR_HD float brrr_normal(uint64_t key, uint64_t idx) {
    int32_t s = (int32_t)(brrr_bytesum64(brrr_draw(key, 2 * idx)) +
                          brrr_bytesum64(brrr_draw(key, 2 * idx + 1))) - 2040;
    return (float)s * 0.0033829376f; /* 1 / sqrt(16 * (256^2 - 1) / 12) */
}

/* f32 element: mean + sigma * z, computed as two separately rounded float operations */
BRRR_HD float brrr_synth_f32(uint64_t key, uint64_t idx, float mean, float sigma) {
    float z = brrr_normal(key, idx);
    float v = z * sigma;
    return v + mean;
}

/* round-to-nearest-even f32 -> bf16 (bit pattern) */
BRRR_HD uint16_t brrr_f32_to_bf16(float v) {
    uint32_t b;
#if defined(__CUDA_ARCH__)
    b = __float_as_uint(v);
#else
    memcpy(&b, &v, 4);
#endif
    return (uint16_t)(((b + 0x7fffu + ((b >> 16) & 1u)) >> 16) & 0xffffu);
}

BRRR_HD uint16_t brrr_synth_bf16(uint64_t key, uint64_t idx, float sigma) {
    return brrr_f32_to_bf16(brrr_normal(key, idx) * sigma);
}

/* One 17-byte GGUF MXFP4 block (block index blk over the whole tensor): byte 0 is the e8m0
 * exponent, uniform over 117..123 (value scale 2^(e-128) on the doubled e2m1 table, i.e.
 * e2m1 * 2^k with k uniform in -10..-4); bytes 1..16 hold 32 uniform 4-bit codes. */
BRRR_HD void brrr_synth_mxfp4_block(uint64_t key, uint64_t blk, uint8_t out[17]) {
    uint64_t d0 = brrr_draw(key, 3 * blk), d1 = brrr_draw(key, 3 * blk + 1), d2 = brrr_draw(key, 3 * blk + 2);
    out[0] = (uint8_t)(117u + (uint32_t)(d2 % 7u));
    for (int i = 0; i < 8; i++) { out[1 + i] = (uint8_t)(d0 >> (8 * i)); out[9 + i] = (uint8_t)(d1 >> (8 * i)); }
}

/* One 144-byte GGUF Q4_K superblock (256 values): f16 d, f16 dmin, 12 bytes of packed 6-bit
 * scales/mins, 128 bytes of nibbles.  Scales, mins and nibbles are uniform random bytes.  d is an
 * f16 2^-13 * (1 + 8k/1024), k uniform in 0..7, and dmin = 7.5 * d exactly (an f16 too), which makes
 * the weights d*sc*q - dmin*mn zero-mean (E[q] = 7.5, E[sc] = E[mn]): a deep random network whose
 * weights have a common mean collapses onto one token.  One block in 16 has a subnormal d
 * (m * 2^-24, m even in 64..126) with dmin = 7.5 d, subnormal too.  20 draws per block. */
BRRR_HD void brrr_synth_q4k_block(uint64_t key, uint64_t blk, uint8_t out[144]) {
    uint64_t h = brrr_draw(key, 20 * blk);
    uint32_t k = (uint32_t)(h & 7u), sub = ((h >> 10) & 15u) == 0, ms = 64u + 2u * (uint32_t)((h >> 3) & 31u);
    uint16_t d = (uint16_t)(sub ? ms : ((2u << 10) | (8u * k)));
    uint16_t dmin = (uint16_t)(sub ? (ms * 15u) >> 1 : ((4u << 10) | (896u + 15u * k)));
    out[0] = (uint8_t)d; out[1] = (uint8_t)(d >> 8); out[2] = (uint8_t)dmin; out[3] = (uint8_t)(dmin >> 8);
    out[4] = (uint8_t)(h >> 32); out[5] = (uint8_t)(h >> 40); out[6] = (uint8_t)(h >> 48); out[7] = (uint8_t)(h >> 56);
    for (int j = 0; j < 17; j++) {
        uint64_t v = brrr_draw(key, 20 * blk + 1 + j);
        for (int i = 0; i < 8; i++) out[8 + 8 * j + i] = (uint8_t)(v >> (8 * i));
    }
}

/* One 210-byte GGUF Q6_K superblock: 128 bytes of low nibbles, 64 bytes of 2-bit fields, 16 int8
 * scales (uniform over -128..127), f16 d (a subnormal, m * 2^-24 with m in 128..639, the range real
 * checkpoints use).  All other bytes random.  27 draws per block. */
BRRR_HD void brrr_synth_q6k_block(uint64_t key, uint64_t blk, uint8_t out[210]) {
    for (int j = 0; j < 26; j++) {
        uint64_t v = brrr_draw(key, 27 * blk + j);
        for (int i = 0; i < 8; i++) out[8 * j + i] = (uint8_t)(v >> (8 * i));
    }
    uint64_t h = brrr_draw(key, 27 * blk + 26);
    uint16_t d = (uint16_t)(128u + (uint32_t)(h & 0x1ffu));
    out[208] = (uint8_t)d; out[209] = (uint8_t)(d >> 8);
}

/* uniform token id in [0, bound) */
BRRR_HD uint32_t brrr_synth_token(uint64_t key, uint64_t idx, uint32_t bound) {
    return (uint32_t)(brrr_draw(key, idx) % bound);
}

#endif /* BRRR_SYNTH_H */
