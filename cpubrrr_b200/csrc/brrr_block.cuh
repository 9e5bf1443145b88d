// Warp- and block-level building blocks shared by several kernels.
#pragma once
#include "brrr_dev.cuh"

namespace brrr {

// order-preserving map float -> uint32 (larger float = larger uint)
__device__ __forceinline__ uint32_t float_orderable(float v) {
    uint32_t b = __float_as_uint(v);
    return b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Quantise one 32-block held one element per lane; writes 32 int8 and the block scale.
// scale = max(1e-12, amax) / 127 (true division); q = round-half-away(v / scale) clamped +-127.
__device__ __forceinline__ void warp_quant_block(float v, int lane, int8_t *q, float *s) {
    float amax = fmaxf(warp_max(fabsf(v)), 1e-12f);
    float sc = __fdiv_rn(amax, 127.0f);
    if (lane == 0) *s = sc;
    q[lane] = (int8_t)brrr_q8_round(v, sc);
}

// Sum of squares in the 16-chain order: chain c (0..15) accumulates x[c], x[c+16], ... with fused
// multiply-adds; chains combine as ((a0+a1)+(a2+a3)) per lane, then (l0+l1)+(l2+l3); a scalar
// unfused tail covers n % 16.  Returns 1 / sqrt(ss / n + eps) to every thread of the block.
// Must be called by all threads; x must be visible to warp 0 (shared or global).
__device__ __forceinline__ float block_rms_inv(const float *x, int n, float eps, float *sh_out) {
    if (threadIdx.x < 32) {
        int c = threadIdx.x;
        float acc = 0.0f;
        int n16 = n & ~15;
        if (c < 16) {
            // chain c: x[c], x[c+16], ... in order; values are fetched 12 at a time so that only
            // the fused multiply-adds sit on the dependent path
            int i = c;
            for (; i + 16 * 11 < n16; i += 16 * 12) {
                float v[12];
#pragma unroll
                for (int k = 0; k < 12; k++) v[k] = x[i + 16 * k];
#pragma unroll
                for (int k = 0; k < 12; k++) acc = __fmaf_rn(v[k], v[k], acc);
            }
            for (; i < n16; i += 16) { float v = x[i]; acc = __fmaf_rn(v, v, acc); }
        }
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
        if (c == 0) {
            for (int i = n16; i < n; i++) acc = __fadd_rn(acc, __fmul_rn(x[i], x[i]));
            *sh_out = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(acc, (float)n), eps)));
        }
    }
    __syncthreads();
    return *sh_out;
}

// Block-wide RMSNorm + per-32 Q8 quantisation of x[0..n) into a staged activation image.
// Each thread owns 4 consecutive elements (one 32-bit word of quants), 8 consecutive threads own
// a 32-block, so a block's amax needs three shuffles.  norm_w == nullptr: quantise x as it is.
//   NQ_Q8:      xp[b*4+j] = {elements 4j..4j+3, elements 16+4j..16+4j+3}   (Q8 GEMV image)
//   NQ_MX:      xp[b*4+j] = the same two words byte-interleaved for the MXFP4 lane dot
//   NQ_NATURAL: quants in element order to (int8_t*)xp, scales to xsc       (global buffers)
// xf: n floats of shared scratch.  The static norm weights of the first MAXG passes are taken
// from wreg[], which the caller fills with norm_prefetch() before it waits on the previous
// kernel, so no cold global load sits on the critical path; later passes read norm_w directly.
// Must be called by all threads; nthreads % 32 == 0, n % 32 == 0, x and norm_w 16-byte aligned.
// Ends with the image complete but NOT yet synchronised.
enum { NQ_Q8 = 0, NQ_MX = 1, NQ_NATURAL = 2 };
// global -> shared copy of n floats (n % 4 == 0, 16-byte aligned).  Up to eight loads are issued before the first
// store: a store to shared memory between them would keep the compiler from overlapping the loads
// (it cannot rule out aliasing), and every load is a full round trip to L2.
__device__ __forceinline__ void stage_vec4(const float *__restrict__ src, float *dst, int n, int tid, int nthreads) {
    const int groups = n >> 2;
    const float4 *s4 = reinterpret_cast<const float4 *>(src);
    float4 *d4 = reinterpret_cast<float4 *>(dst);
    for (int g0 = tid; g0 < groups; g0 += 8 * nthreads) {
        float4 v[8];
#pragma unroll
        for (int k = 0; k < 8; k++) if (g0 + k * nthreads < groups) v[k] = s4[g0 + k * nthreads];
#pragma unroll
        for (int k = 0; k < 8; k++) if (g0 + k * nthreads < groups) d4[g0 + k * nthreads] = v[k];
    }
}

template <int MAXG>
__device__ __forceinline__ void norm_prefetch(const float *__restrict__ norm_w, int n, float4 (&wreg)[MAXG], int tid, int nthreads) {
#pragma unroll
    for (int p = 0; p < MAXG; p++) {
        const int g = tid + p * nthreads;
        wreg[p] = (norm_w && g < (n >> 2)) ? reinterpret_cast<const float4 *>(norm_w)[g] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

template <int LAYOUT, int MAXG>
__device__ __forceinline__ void block_norm_quant_staged(const float *norm_w, const float4 (&wreg)[MAXG], float eps, int n,
                                                        float *xf, int2 *xp, float *xsc, float *inv_sh, int tid, int nthreads);

template <int LAYOUT, int MAXG>
__device__ __forceinline__ void block_norm_quant(const float *__restrict__ x, const float *norm_w, const float4 (&wreg)[MAXG], float eps, int n,
                                                 float *xf, int2 *xp, float *xsc, float *inv_sh, int tid, int nthreads) {
    stage_vec4(x, xf, n, tid, nthreads);
    __syncthreads();
    block_norm_quant_staged<LAYOUT, MAXG>(norm_w, wreg, eps, n, xf, xp, xsc, inv_sh, tid, nthreads);
}

// The same with x already in xf (shared memory) and visible to the whole block.
template <int LAYOUT, int MAXG>
__device__ __forceinline__ void block_norm_quant_staged(const float *norm_w, const float4 (&wreg)[MAXG], float eps, int n,
                                                        float *xf, int2 *xp, float *xsc, float *inv_sh, int tid, int nthreads) {
    const int groups = n >> 2;
    float4 *xf4 = reinterpret_cast<float4 *>(xf);
    float inv = 1.0f;
    if (norm_w) inv = block_rms_inv(xf, n, eps, inv_sh);
    const int npass = (groups + nthreads - 1) / nthreads;
    // The passes are independent; unrolling lets their divisions and shuffles overlap.
#pragma unroll
    for (int p = 0; p < 8; p++) {
        if (p >= npass) break;
        const int g = tid + p * nthreads;
        const bool live = g < groups;
        float4 v = live ? xf4[g] : make_float4(0.f, 0.f, 0.f, 0.f);
        if (norm_w && live) {
            float4 w;
            if (p < MAXG) w = wreg[p < MAXG ? p : 0];
            else w = reinterpret_cast<const float4 *>(norm_w)[g];
            v.x = __fmul_rn(__fmul_rn(v.x, inv), w.x); v.y = __fmul_rn(__fmul_rn(v.y, inv), w.y);
            v.z = __fmul_rn(__fmul_rn(v.z, inv), w.z); v.w = __fmul_rn(__fmul_rn(v.w, inv), w.w);
        }
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        const float sc = __fdiv_rn(fmaxf(amax, 1e-12f), 127.0f);
        uint32_t word = (uint32_t)(brrr_q8_round(v.x, sc) & 0xFF) | ((uint32_t)(brrr_q8_round(v.y, sc) & 0xFF) << 8) |
                        ((uint32_t)(brrr_q8_round(v.z, sc) & 0xFF) << 16) | ((uint32_t)(brrr_q8_round(v.w, sc) & 0xFF) << 24);
        const int t = g & 7, b = g >> 3;
        if (LAYOUT == NQ_MX) {
            uint32_t other = __shfl_xor_sync(0xffffffffu, word, 4);
            if (live && t < 4)
                xp[b * 4 + t] = make_int2((int)brrr_prmt(word, other, 0x5140u), (int)brrr_prmt(word, other, 0x7362u));
        } else if (LAYOUT == NQ_Q8) {
            if (live) reinterpret_cast<int *>(&xp[b * 4 + (t & 3)])[t >> 2] = (int)word;
        } else {
            if (live) reinterpret_cast<uint32_t *>(xp)[g] = word;
        }
        if (live && t == 0) xsc[b] = sc;
    }
}

// The k largest of est[0..ne) by (value, lower index first): sel[r] gets the expert of rank r.
// Every thread ranks the experts it owns against all others in shared memory (no shuffles, one
// global round trip).  Used identically by every kernel that needs the speculative expert set
// (the set comes from an order-free router estimate; correctness never depends on it).
// Builds with BRRR_TEST_HOOKS only: when the state's test_hooks word has bit 0 set, the last pick is
// replaced on every third position (the tests use it to force a missed speculation).
// Block-wide; ends with sel[] written but not yet synchronised.  lg: ne floats of scratch.
__device__ __forceinline__ void block_spec_select(const float *est, int ne, int topk, const DevState *state,
                                                  float *lg, int *sel, int tid, int nthreads) {
#ifdef BRRR_TEST_HOOKS
    const bool sabotage = state && (state->test_hooks & 1u);
    const uint32_t pos = sabotage ? state->pos : 0u;
#else
    constexpr bool sabotage = false;
    constexpr uint32_t pos = 0u;
    (void)state;
#endif
    for (int e = tid; e < ne; e += nthreads) lg[e] = __ldcg(est + e);
    __syncthreads();
    for (int e = tid; e < ne; e += nthreads) {
        const float v = lg[e];
        int rank = 0;
        for (int o = 0; o < ne; o++) {
            const float u = lg[o];
            rank += (u > v || (u == v && o < e)) ? 1 : 0;
        }
        if (rank < topk) sel[rank] = (sabotage && rank == topk - 1 && pos % 3 == 0) ? (e + 1) % ne : e;
    }
}

// The same selection for ne <= 32 inside one warp, without shared memory or block-wide barriers:
// returns the expert of rank `want` (what block_spec_select would leave in sel[want]).  All 32
// lanes must call it.
__device__ __forceinline__ int warp_spec_expert(const float *est, int ne, int topk, const DevState *state, int want, int lane) {
#ifdef BRRR_TEST_HOOKS
    const bool sabotage = state && (state->test_hooks & 1u);
    const uint32_t pos = sabotage ? state->pos : 0u;
#else
    constexpr bool sabotage = false;
    constexpr uint32_t pos = 0u;
    (void)state;
#endif
    const float v = lane < ne ? __ldcg(est + lane) : 0.0f;
    int rank = 0;
#pragma unroll 8
    for (int o = 0; o < 32; o++) {
        const float u = __shfl_sync(0xffffffffu, v, o);
        rank += (o < ne && (u > v || (u == v && o < lane))) ? 1 : 0;
    }
    const unsigned hit = __ballot_sync(0xffffffffu, lane < ne && rank == want);
    const int e = __ffs(hit) - 1;
    return (sabotage && want == topk - 1 && pos % 3 == 0) ? (e + 1) % ne : e;
}

// gpt-oss clamped SwiGLU: xg = min(g, 7), yu = clamp(u, -7, 7), (xg / (1 + exp(-1.702 xg))) (yu + 1)
__device__ __forceinline__ float swiglu_oai(float g, float u) {
    float xg = fminf(g, 7.0f);
    float yu = fminf(fmaxf(u, -7.0f), 7.0f);
    float den = __fadd_rn(1.0f, brrr_expf_dev(__fmul_rn(-1.702f, xg)));
    return __fmul_rn(__fdiv_rn(xg, den), __fadd_rn(yu, 1.0f));
}


}  // namespace brrr
