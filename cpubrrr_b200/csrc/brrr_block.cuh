// Warp- and block-level building blocks shared by several kernels.
#pragma once
#include "brrr_dev.cuh"

namespace brrr {

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
#pragma unroll 8
            for (int i = c; i < n16; i += 16) { float v = x[i]; acc = __fmaf_rn(v, v, acc); }
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

// gpt-oss clamped SwiGLU: xg = min(g, 7), yu = clamp(u, -7, 7), (xg / (1 + exp(-1.702 xg))) (yu + 1)
__device__ __forceinline__ float swiglu_oai(float g, float u) {
    float xg = fminf(g, 7.0f);
    float yu = fminf(fmaxf(u, -7.0f), 7.0f);
    float den = __fadd_rn(1.0f, brrr_expf_dev(__fmul_rn(-1.702f, xg)));
    return __fmul_rn(__fdiv_rn(xg, den), __fadd_rn(yu, 1.0f));
}

// order-preserving map float -> uint32 (larger float = larger uint)
__device__ __forceinline__ uint32_t float_orderable(float v) {
    uint32_t b = __float_as_uint(v);
    return b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u);
}

}  // namespace brrr
