// Device-side math and layout definitions shared by all kernels.
//
// Float semantics: every kernel reproduces one fixed order of IEEE-754 single operations (the
// lane structure of the reference's NEON code), so results do not depend on grid shape.  The
// translation units are compiled with -fmad=false; fused multiply-adds are written explicitly
// (__fmaf_rn) exactly where the reference fuses.  No fast-math, no flush-to-zero.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define BRRR_MAXSEQ 4096

// ---------------------------------------------------------------- scalar helpers
__device__ __forceinline__ float brrr_expf_dev(float x) {
    // Cephes-style expf as a fixed operation sequence (range reduction by ln2 hi/lo, degree-5
    // polynomial, every multiply-add fused, two-step power-of-two scaling).
    if (x != x) return x + x;
    if (x > 88.72283935546875f) return __int_as_float(0x7f800000);
    if (x < -104.0f) return 0.0f;
    float kf = rintf(__fmul_rn(x, 1.44269504088896341f));
    float r = __fmaf_rn(kf, -0.693145751953125f, x);
    r = __fmaf_rn(kf, -1.42860682030941723212e-6f, r);
    float p = 1.9875691500e-4f;
    p = __fmaf_rn(p, r, 1.3981999507e-3f);
    p = __fmaf_rn(p, r, 8.3334519073e-3f);
    p = __fmaf_rn(p, r, 4.1665795894e-2f);
    p = __fmaf_rn(p, r, 1.6666665459e-1f);
    p = __fmaf_rn(p, r, 5.0000001201e-1f);
    float r2 = __fmul_rn(r, r);
    float y = __fmaf_rn(p, r2, r);
    y = __fadd_rn(y, 1.0f);
    int k = (int)kf;
    int k1 = k >> 1, k2 = k - k1;
    float s1 = __int_as_float((k1 + 127) << 23);
    float s2 = __int_as_float((k2 + 127) << 23);
    return __fmul_rn(__fmul_rn(y, s1), s2);
}

// 2^(e-128) for an e8m0 byte (the doubled e2m1 table), exact including e = 0, 1 (subnormal).
__device__ __forceinline__ float brrr_e8m0_scale(uint32_t e) {
    return __int_as_float(e >= 2u ? (e - 1u) << 23 : 0x00200000u << e);
}

// int8 quantisation of one value given the block scale: round half away from zero of the true
// quotient, clamped to +-127.
__device__ __forceinline__ int brrr_q8_round(float v, float sc) {
    float r = roundf(__fdiv_rn(v, sc));
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    return (int)r;
}

__device__ __forceinline__ float brrr_bf16_to_f32(uint16_t v) { return __int_as_float((uint32_t)v << 16); }

__device__ __forceinline__ uint32_t brrr_prmt(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// pairwise horizontal sum over the 4 lanes of a chain group: (l0+l1)+(l2+l3).  The lanes of a
// group are 4 consecutive threads; xor-shuffles make both operands of each add identical on
// both sides, so every lane ends with the same value.
__device__ __forceinline__ float brrr_hsum4(float v) {
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
    return v;
}

// ---------------------------------------------------------------- MXFP4 lane dot
// One 32-bit word holds bytes 4j..4j+3 of a row-block: 8 e2m1 codes (low nibble = element 4j+i,
// high nibble = element 16+4j+i).  The magnitudes {0,1,2,3,4,6,8,12} are looked up with prmt,
// whose selector bit 3 replicates the sign bit of the selected byte:
//   P: table mag+1 (0 for code 0), raw selector      -> mag+1 for positive codes, 0 for negative
//   N: table -mag, selector with bit 3 flipped       -> -mag for negative codes, -1 (0 for
//                                                       magnitude 0) for positive codes
// P + N is the signed value, so four dp4a into one accumulator give the exact lane sum
//   sum_i lo[4j+i]*x[4j+i] + hi[4j+i]*x[16+4j+i].
// xa / xb are the activations pre-interleaved to the prmt output order:
//   xa = {x[4j], x[16+4j], x[4j+1], x[16+4j+1]}, xb = {x[4j+2], x[16+4j+2], x[4j+3], x[16+4j+3]}.
__device__ __forceinline__ int brrr_mx_lane_dot(uint32_t w, int xa, int xb) {
    const uint32_t P_LO = 0x04030200u, P_HI = 0x0D090705u;
    const uint32_t N_LO = 0xFDFEFF00u, N_HI = 0xF4F8FAFCu;
    uint32_t wx = w ^ 0x88888888u;
    int t = 0;
    t = __dp4a((int)brrr_prmt(P_LO, P_HI, w), xa, t);
    t = __dp4a((int)brrr_prmt(N_LO, N_HI, wx), xa, t);
    t = __dp4a((int)brrr_prmt(P_LO, P_HI, w >> 16), xb, t);
    t = __dp4a((int)brrr_prmt(N_LO, N_HI, wx >> 16), xb, t);
    return t;
}

// ---------------------------------------------------------------- layouts
// Q8 matrix, rows % 4 == 0, cols % 64 == 0, np = cols / 64 block pairs.
//   wq: [rows/4][np][4 rows][2 parity][4 lanes][8 B]; the 8 bytes of (row, block b = 2i+p, lane j)
//       are w[32b+4j .. +3] then w[32b+16+4j .. +3]
//   ws: [rows/4][np][4 rows][2 parity] f32 block scales
// A warp (4 rows x 8 chains) reads 256 contiguous bytes per step.
struct Q8Dev {
    int8_t *wq;
    float *ws;
    int rows, cols;
};
__host__ __device__ __forceinline__ size_t q8_woff(int row, int pair, int np) {
    return ((size_t)(row >> 2) * np + pair) * 256 + (size_t)(row & 3) * 64;
}
__host__ __device__ __forceinline__ size_t q8_soff(int row, int pair, int np) {
    return ((size_t)(row >> 2) * np + pair) * 8 + (size_t)(row & 3) * 2;
}

// MXFP4 matrix, rows % 8 == 0, blocks % 2 == 0, np = blocks / 2.
//   nib:  [rows/8][np][8 rows][4 lanes][8 B]; the 8 bytes of (row, pair i, lane j) are the lane
//         word of block 2i then of block 2i+1
//   exps: [rows/8][np][8 rows][2] e8m0 bytes
// A warp (8 rows x 4 lanes) reads 256 contiguous bytes per step.
struct MxDev {
    uint8_t *nib;
    uint8_t *exps;
    int rows, blocks;
};
__host__ __device__ __forceinline__ size_t mx_noff(int row, int pair, int np) {
    return ((size_t)(row >> 3) * np + pair) * 256 + (size_t)(row & 7) * 32;
}
__host__ __device__ __forceinline__ size_t mx_eoff(int row, int pair, int np) {
    return ((size_t)(row >> 3) * np + pair) * 16 + (size_t)(row & 7) * 2;
}

// Device-resident decode state: the token and position of the step being run, the running
// argmax of the vocabulary projection and the ring of emitted tokens.
struct DevState {
    uint32_t tok;
    uint32_t pos;
    uint32_t n_out;
    uint32_t router_done;          // CTA arrival counter of the router kernel
    unsigned long long best;       // (orderable logit << 32) | ~index
    uint32_t out[BRRR_MAXSEQ];
};
