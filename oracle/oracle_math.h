/* TEST INFRASTRUCTURE — CPU oracle.  Nothing under oracle/ is part of the shipped product path;
 * only tests, the smoke check and the benchmark's CPU-baseline leg may call it.
 *
 * Transcendentals of the decode path.  The reference (Rust, Apple libm) calls f32::exp in
 * three places: attention softmax (src/bin/engine_gpt2.rs:824-825), router softmax (865)
 * and the clamped SwiGLU (898).  The bits of Apple's libm are not knowable here, so exp is
 * *defined* as the fixed sequence of IEEE-754 single operations below (Cephes-style range
 * reduction + degree-5 polynomial, every multiply-add fused).  The CUDA kernels implement the
 * same sequence, so the checker and the device agree bit for bit; tests pin this function to
 * libm's expf within 2 ulp.
 */
#ifndef ORACLE_MATH_H
#define ORACLE_MATH_H
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline float orc_bits2f(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t orc_f2bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

static inline float orc_expf(float x) {
    if (x != x) return x + x;
    if (x > 88.72283935546875f) return INFINITY;
    if (x < -104.0f) return 0.0f;
    float kf = rintf(x * 1.44269504088896341f);
    float r = fmaf(kf, -0.693145751953125f, x);
    r = fmaf(kf, -1.42860682030941723212e-6f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float r2 = r * r;
    float y = fmaf(p, r2, r);
    y = y + 1.0f;
    int k = (int)kf;
    int k1 = k >> 1, k2 = k - k1;
    float s1 = orc_bits2f((uint32_t)(k1 + 127) << 23);
    float s2 = orc_bits2f((uint32_t)(k2 + 127) << 23);
    return (y * s1) * s2;
}

/* 2^(e-128) for an e8m0 byte on the doubled e2m1 table (src/bin/engine_gpt2.rs:435-438),
 * exact for every e including the two subnormal results (e = 0, 1). */
static inline float orc_exp_tbl(uint8_t e) { return ldexpf(1.0f, (int)e - 128); }

/* bf16 <-> f32 (src/bin/engine_gpt2.rs:302-309, 762) */
static inline float orc_bf16_to_f32(uint16_t v) { return orc_bits2f((uint32_t)v << 16); }

#endif
