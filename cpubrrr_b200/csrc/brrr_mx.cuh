// Building blocks of the MXFP4 expert kernels shared by the single-GPU and the expert-parallel
// kernels: activation staging, the per-chain block-pair loop on the integer units, and the
// multi-stream bulk-copy ring.
#pragma once
#include "brrr_kernels.h"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"

namespace brrr {

// ---------------------------------------------------------------- activation staging
// Shared-memory image of a Q8 activation for the MXFP4 lane dot: one int2 {xa, xb} per
// (block, lane), bytes interleaved to the prmt output order (see brrr_mx_lane_dot).
__device__ __forceinline__ int2 mx_interleave(uint32_t lo, uint32_t hi) {
    return make_int2((int)brrr_prmt(lo, hi, 0x5140u), (int)brrr_prmt(lo, hi, 0x7362u));
}

__device__ __forceinline__ void mx_stage_x(const int8_t *__restrict__ xq, const float *__restrict__ xs, int nb, int2 *xp, float *xsc, int tid, int nthreads) {
    for (int idx = tid; idx < nb * 4; idx += nthreads) {
        int b = idx >> 2, j = idx & 3;
        const uint32_t *xw = reinterpret_cast<const uint32_t *>(xq + b * 32);
        xp[idx] = mx_interleave(xw[j], xw[4 + j]);
    }
    for (int b = tid; b < nb; b += nthreads) xsc[b] = xs[b];
}

// Quantise one 32-block held one value per lane straight into the staged layout.
__device__ __forceinline__ void mx_quant_stage_block(float v, int lane, int b, int2 *xp, float *xsc) {
    float amax = fmaxf(warp_max(fabsf(v)), 1e-12f);
    float sc = __fdiv_rn(amax, 127.0f);
    uint32_t q = (uint32_t)(brrr_q8_round(v, sc) & 0xFF);
    uint32_t word = q << (8 * (lane & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);           // lanes 4j..4j+3 hold lo word j, lanes 16+4j.. hi word j
    uint32_t other = __shfl_xor_sync(0xffffffffu, word, 16);
    if (lane < 16 && (lane & 3) == 0) xp[b * 4 + (lane >> 2)] = mx_interleave(word, other);
    if (lane == 0) xsc[b] = sc;
}


// N consecutive block pairs of one lane chain from units resident in shared memory: operands
// first, then the 2N exact lane dots and scales (independent work), then the 2N fused
// multiply-adds in block order.
// 2^(e-128) for every e8m0 byte, built once per CTA: one shared-memory read replaces the
// compare/select/shift sequence in the inner loop.
__device__ __forceinline__ void mx_fill_scale_table(float *tbl, int tid, int nthreads) {
    for (int e = tid; e < 256; e += nthreads) tbl[e] = brrr_e8m0_scale((uint32_t)e);
}

template <int N>
__device__ __forceinline__ float mx_pairs(const unsigned char *unit, int rl, int j, const int2 *xpj, const float *xsc, const float *tbl, int pair, float acc) {
    uint2 w[N];
    uint32_t e2[N];
    int2 x0[N], x1[N];
    float xs0[N], xs1[N];
#pragma unroll
    for (int i = 0; i < N; i++) {
        const unsigned char *u = unit + (size_t)i * MX_UNIT;
        w[i] = *reinterpret_cast<const uint2 *>(u + rl * 32 + j * 8);
        e2[i] = *reinterpret_cast<const unsigned short *>(u + MX_UNIT_EXPS + rl * 2);
        x0[i] = xpj[(pair + i) * 8]; x1[i] = xpj[(pair + i) * 8 + 4];
        xs0[i] = xsc[2 * (pair + i)]; xs1[i] = xsc[2 * (pair + i) + 1];
    }
    float t0[N], t1[N], s0[N], s1[N];
#pragma unroll
    for (int i = 0; i < N; i++) {
        t0[i] = (float)brrr_mx_lane_dot(w[i].x, x0[i].x, x0[i].y);
        t1[i] = (float)brrr_mx_lane_dot(w[i].y, x1[i].x, x1[i].y);
        s0[i] = __fmul_rn(tbl[e2[i] & 0xFFu], xs0[i]);
        s1[i] = __fmul_rn(tbl[e2[i] >> 8], xs1[i]);
    }
#pragma unroll
    for (int i = 0; i < N; i++) { acc = __fmaf_rn(t0[i], s0[i], acc); acc = __fmaf_rn(t1[i], s1[i], acc); }
    return acc;
}

__device__ __forceinline__ float mx_chunk(const unsigned char *base, int cnt, int rl, int j, const int2 *xpj, const float *xsc, const float *tbl, int pair0, float acc) {
    int i = 0;
#ifndef MX_UNROLL
#define MX_UNROLL 1
#endif
#ifndef MX_TAIL_UNROLL
#define MX_TAIL_UNROLL 4
#endif
#define MX_PRAGMA_(x) _Pragma(#x)
#define MX_PRAGMA_UNROLL(n) MX_PRAGMA_(unroll n)
#if MX_UNROLL > 1
    for (; i + MX_UNROLL <= cnt; i += MX_UNROLL) acc = mx_pairs<MX_UNROLL>(base + (size_t)i * MX_UNIT, rl, j, xpj, xsc, tbl, pair0 + i, acc);
#endif
MX_PRAGMA_UNROLL(MX_TAIL_UNROLL)
    for (; i < cnt; i++) acc = mx_pairs<1>(base + (size_t)i * MX_UNIT, rl, j, xpj, xsc, tbl, pair0 + i, acc);
    return acc;
}

// ---------------------------------------------------------------- multi-stream ring
// NS streams of np units each; chunk c covers pairs [c*ch, ...) of every stream.  Stage layout:
// [stream][ch][MX_UNIT].
struct MxRing {
    unsigned char *ring;
    uint64_t *bars;
    int ch, stages, np, ns;
    size_t stream_bytes, stage_bytes;
    // Lane `lane` of one warp issues the copy of stream lane % ns of chunk c0 + lane / ns, for nc
    // chunks at once (nc * ns <= 32).  Issued by one thread one after the other, every copy waits
    // for the address translation of the one before (about 500 cycles each on cold expert
    // weights); issued by different lanes they overlap.  A chunk's barrier cannot complete before
    // its arrive.expect_tx, so the order of the lanes does not matter.
    __device__ __forceinline__ void issue_warp(int c0, int nc, const uint8_t *const *src, int lane) const {
        const int c = c0 + lane / ns, s = lane % ns;
        if (lane < nc * ns) {
            const int cnt = min(ch, np - c * ch), slot = c % stages;
            fence_proxy_async();
            if (s == 0) mbar_expect_tx(&bars[slot], (uint32_t)cnt * MX_UNIT * ns);
            bulk_g2s(ring + stage_bytes * slot + stream_bytes * s, src[s] + (size_t)c * ch * MX_UNIT, (uint32_t)cnt * MX_UNIT, &bars[slot]);
        }
    }
};

struct MxLaunchShape { int ch, stages; };
static inline MxLaunchShape mx_shape(int np, int ns, size_t budget) {
    MxLaunchShape s;
    s.ch = np;
    for (int c = 16; c >= 12; c--) if (np % c == 0) { s.ch = c; break; }
    if (s.ch == np) for (int c = 17; c <= 24; c++) if (np % c == 0) { s.ch = c; break; }
    if (s.ch == np && np > 24) s.ch = 16;
    int nchunks = (np + s.ch - 1) / s.ch;
    int maxs = (int)(budget / ((size_t)ns * s.ch * MX_UNIT));
    if (maxs < 2) maxs = 2;
    s.stages = nchunks < maxs ? nchunks : maxs;
    return s;
}

}  // namespace brrr
