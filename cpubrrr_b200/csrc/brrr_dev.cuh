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
#ifndef BRRR_TILE_MAX
#define BRRR_TILE_MAX 512     // token rows per pass over the layers (same value as in the public header)
#endif

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
// Both weight formats are stored as fixed-size *units* that hold everything 16 rows need for two
// consecutive 32-blocks (a block pair): quants and scales together, so one contiguous stream
// feeds a CTA and any run of units is a valid bulk-copy source (unit sizes are multiples of 16).
// Units are ordered [row / 16][pair]; a CTA that owns consecutive 16-row groups owns one
// contiguous byte range.
//
// Q8 unit (1152 B), rows padded to a multiple of 16, cols % 64 == 0, np = cols / 64:
//   bytes [0, 1024):    [16 rows][2 parity][4 lanes][8 B]; the 8 bytes of (row, block b = 2i+p,
//                       lane j) are w[32b+4j .. +3] then w[32b+16+4j .. +3]
//   bytes [1024, 1152): [16 rows][2 parity] f32 block scales
// A warp (4 rows x 8 chains) reads 256 contiguous bytes per step.
constexpr int Q8_UNIT = 1152;
constexpr int Q8_UNIT_SCALES = 1024;
struct Q8Dev {
    uint8_t *data;
    int rows, cols;      // logical shape; storage holds ceil(rows / 16) * 16 rows
};
__host__ __device__ __forceinline__ int q8_urows(int rows) { return (rows + 15) >> 4; }
__host__ __device__ __forceinline__ size_t q8_bytes(int rows, int cols) { return (size_t)q8_urows(rows) * (cols / 64) * Q8_UNIT; }
__host__ __device__ __forceinline__ size_t q8_unit_off(int urow, int pair, int np) { return ((size_t)urow * np + pair) * Q8_UNIT; }

// MXFP4 unit (544 B), rows % 16 == 0, blocks % 2 == 0, np = blocks / 2:
//   bytes [0, 512):   [16 rows][4 lanes][8 B]; the 8 bytes of (row, pair i, lane j) are the lane
//                     word (bytes 4j..4j+3 of the 16 nibble bytes) of block 2i then of block 2i+1
//   bytes [512, 544): [16 rows][2] e8m0 bytes
// A warp (8 rows x 4 lanes) reads 256 contiguous bytes per step.
constexpr int MX_UNIT = 544;
constexpr int MX_UNIT_EXPS = 512;
struct MxDev {
    uint8_t *data;
    int rows, blocks;
};
__host__ __device__ __forceinline__ size_t mx_bytes(int rows, int blocks) { return (size_t)(rows / 16) * (blocks / 2) * MX_UNIT; }
__host__ __device__ __forceinline__ size_t mx_unit_off(int urow, int pair, int np) { return ((size_t)urow * np + pair) * MX_UNIT; }

// Values of DevState.err: a bounded wait on a bulk copy, or on a word another kernel publishes, ran out.
enum { DEV_ERR_NONE = 0, DEV_ERR_COPY_TIMEOUT = 1, DEV_ERR_PEER_TIMEOUT = 2 };

// Device-resident decode state: the token and position of the step being run, the running
// argmax of the vocabulary projection, the ring of emitted tokens and a sticky error word.
struct DevState {
    uint32_t tok;
    uint32_t pos;
    uint32_t n_out;
    uint32_t router_done;          // CTA arrival counter of the router kernel
    unsigned long long best;       // (orderable logit << 32) | ~index
    uint32_t err;                  // DEV_ERR_* (0 = none); set by a kernel whose bounded wait ran out
    uint32_t spec_fail_step;       // smallest n_out at which speculative routing missed (0xFFFFFFFF = never)
    uint32_t hint_done;            // CTA arrival counter of the routing-hint kernel
    uint32_t router_seq;           // exact-router launches that have published their routing (speculative step)
    uint32_t fold_seq;             // fold launches that have consumed one
    uint32_t test_hooks;           // read by BRRR_TEST_HOOKS builds only: bit 0 = spoil the routing estimate on every third position,
                                   // bit 1 = the exact router does not publish its routing (the fold's bounded wait runs out)
    uint32_t out[BRRR_MAXSEQ];
    long long stamps[256];          // optional in-kernel clock stamps (timeline builds only)
    // routing of the exact router, published for a consumer that runs beside it: word k = (router_seq << 32) | top[k],
    // word 8 + k = (router_seq << 32) | bits of wts[k]; every word validates itself, so no fence is needed
    unsigned long long route_pub[16];
};
// In-kernel clock stamps: BRRR_TEST_HOOKS builds only (timeline of one step, read back by brrr_debug_stamps).
#ifdef BRRR_TEST_HOOKS
__device__ __forceinline__ unsigned long long brrr_gtime() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
// wall-clock (ns) marks: END = latest finish over all CTAs of a kernel, GO = CTA 0 released from its dependency wait
#define BRRR_GT_END(state, i) do { if ((state) && threadIdx.x == 0) atomicMax((unsigned long long *)&(state)->stamps[i], brrr_gtime()); } while (0)
#define BRRR_GT_GO(state, i) do { if ((state) && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) (state)->stamps[i] = (long long)brrr_gtime(); } while (0)
#define BRRR_GT_START(state, i) BRRR_GT_GO(state, i)
#ifndef BRRR_STAMP_BX
#define BRRR_STAMP_BX 0
#endif
#define BRRR_STAMP(state, i) do { if ((state) && threadIdx.x == 0 && blockIdx.x == BRRR_STAMP_BX && blockIdx.y == 0) (state)->stamps[i] = clock64(); } while (0)
#else
#define BRRR_GT_END(state, i) do { } while (0)
#define BRRR_GT_GO(state, i) do { } while (0)
#define BRRR_GT_START(state, i) do { } while (0)
#define BRRR_STAMP(state, i) do { } while (0)
#endif
