// Warp-level building blocks of the K-quant path (Q8_K activations, Q4_K / Q6_K weight rows in the
// GGUF byte layout), shared by the stage kernels and the qwen3moe decode kernels.
//
// Reference arithmetic (src/bin/engine_qwen2.rs:84-114, 164-200, 287-300): per 256-value
// superblock the dot is an exact integer sum scaled once, sumf += (ys*d)*acc - (ys*dmin)*mint
// (Q4_K) or sumf += (ys*d)*acc (Q6_K), unfused, superblocks in order.  The integer sum is
// order-free, so one warp owns a row, its lanes split each superblock (one 32-bit word of nibbles
// per lane for Q4_K, one byte pair of each field for Q6_K), the partial sums meet in a warp
// integer reduction and every lane carries the same float chain.
#pragma once
#include "brrr_dev.cuh"

#include <cuda_fp16.h>

namespace brrr {

__device__ __forceinline__ float half_bits_to_f32(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// byte i (0..11) of the 12 packed scale bytes held in three words
__device__ __forceinline__ uint32_t k4_byte(uint32_t s0, uint32_t s1, uint32_t s2, int i) {
    uint32_t w = i < 4 ? s0 : (i < 8 ? s1 : s2);
    return (w >> ((i & 3) * 8)) & 0xffu;
}

// 6-bit scale and min of sub-block j (src/bin/engine_qwen2.rs:52-56)
__device__ __forceinline__ void k4_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int j, int &sc, int &mn) {
    if (j < 4) {
        sc = (int)(k4_byte(s0, s1, s2, j) & 63u);
        mn = (int)(k4_byte(s0, s1, s2, j + 4) & 63u);
    } else {
        uint32_t hi = k4_byte(s0, s1, s2, j + 4);
        sc = (int)((hi & 0xFu) | ((k4_byte(s0, s1, s2, j - 4) >> 6) << 4));
        mn = (int)((hi >> 4) | ((k4_byte(s0, s1, s2, j) >> 6) << 4));
    }
}

// Q8_K quantisation of one 256-value superblock by one warp: lane l holds values 8l..8l+7 (so
// sub-block j is lanes 4j..4j+3).  Writes the quants, the scale and the eight 32-sums.
__device__ __forceinline__ void warp_quant_q8k(const float (&v)[8], int lane, int8_t *q, float *s, int32_t *bsum) {
    float amax = 1e-12f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float sc = __fdiv_rn(amax, 127.0f);
    int qi[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) { qi[i] = brrr_q8_round(v[i], sc); sum += qi[i]; }
    uint32_t lo = (qi[0] & 0xff) | ((qi[1] & 0xff) << 8) | ((qi[2] & 0xff) << 16) | ((uint32_t)(qi[3] & 0xff) << 24);
    uint32_t hi = (qi[4] & 0xff) | ((qi[5] & 0xff) << 8) | ((qi[6] & 0xff) << 16) | ((uint32_t)(qi[7] & 0xff) << 24);
    *reinterpret_cast<uint2 *>(q + lane * 8) = make_uint2(lo, hi);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if ((lane & 3) == 0) bsum[lane >> 2] = sum;
    if (lane == 0) *s = sc;
}

// Q4_K row x Q8_K activation by one warp; the result is valid in every lane.  Superblock: f16 d,
// f16 dmin, 12 scale bytes, 128 nibble bytes.  Lane l owns word l of the nibble bytes: bytes
// 4l..4l+3 of 32-byte chunk jj = l/8, whose low nibbles belong to sub-block 2jj and high nibbles to
// sub-block 2jj+1.  dbg (nullable): {scaled quant sum, min sum} per superblock.
__device__ __forceinline__ float q4k_row_dot(const uint8_t *row, int nsb, const int8_t *xq, const float *ys, const int32_t *bsum,
                                             int lane, int32_t *dbg = nullptr) {
    const uint32_t *b32 = reinterpret_cast<const uint32_t *>(row);
    const int jj = lane >> 3, k4 = (lane & 7) * 4;
    float sumf = 0.0f;
#pragma unroll 4
    for (int sb = 0; sb < nsb; sb++, b32 += 36) {
        uint32_t dd = __ldg(b32), s0 = __ldg(b32 + 1), s1 = __ldg(b32 + 2), s2 = __ldg(b32 + 3);
        uint32_t qv = __ldg(b32 + 4 + lane);
        int x0 = *reinterpret_cast<const int *>(xq + (sb * 8 + 2 * jj) * 32 + k4);
        int x1 = *reinterpret_cast<const int *>(xq + (sb * 8 + 2 * jj + 1) * 32 + k4);
        int sc0, mn0, sc1, mn1;
        k4_scale_min(s0, s1, s2, 2 * jj, sc0, mn0);
        k4_scale_min(s0, s1, s2, 2 * jj + 1, sc1, mn1);
        int a = __dp4a((int)(qv & 0x0F0F0F0Fu), x0, 0) * sc0 + __dp4a((int)((qv >> 4) & 0x0F0F0F0Fu), x1, 0) * sc1;
        int mt = 0;
        if (lane < 8) {
            int scj, mnj;
            k4_scale_min(s0, s1, s2, lane, scj, mnj);
            mt = mnj * bsum[sb * 8 + lane];
        }
        a = __reduce_add_sync(0xffffffffu, a);
        mt = __reduce_add_sync(0xffffffffu, mt);
        float ysb = ys[sb];
        float d = half_bits_to_f32(dd & 0xffffu), dmin = half_bits_to_f32(dd >> 16);
        float pos = __fmul_rn(__fmul_rn(ysb, d), (float)a);
        float neg = __fmul_rn(__fmul_rn(ysb, dmin), (float)mt);
        sumf = __fadd_rn(sumf, __fsub_rn(pos, neg));
        if (dbg && lane == 0) { dbg[sb * 2] = a; dbg[sb * 2 + 1] = mt; }
    }
    return sumf;
}

// Q6_K row x Q8_K activation by one warp; the result is valid in every lane.  Superblock: 128 B low
// nibbles (ql), 64 B 2-bit fields (qh), 16 int8 scales, f16 d; 210 bytes, so rows are only 2-byte
// aligned and fields are read as byte pairs.  Lane (h = l/16, pp = l%16) owns positions p = 2pp,
// 2pp+1 of half h: with la = ql[64h+p], lb = ql[64h+32+p], hv = qh[32h+p] the four values at
// 128h + {0,32,64,96} + p are (la&15 | (hv&3)<<4), (lb&15 | (hv>>2&3)<<4), (la>>4 | (hv>>4&3)<<4),
// (lb>>4 | (hv>>6)<<4), each - 32.  dbg (nullable): the integer accumulator per superblock.
__device__ __forceinline__ float q6k_row_dot(const uint8_t *row, int nsb, const int8_t *xq, const float *ys, int lane, int32_t *dbg = nullptr) {
    const uint8_t *b = row;
    const int h = lane >> 4, pp = lane & 15;
    float sumf = 0.0f;
#pragma unroll 2
    for (int sb = 0; sb < nsb; sb++, b += 210) {
        uint32_t la2 = __ldg(reinterpret_cast<const unsigned short *>(b + h * 64 + 2 * pp));
        uint32_t lb2 = __ldg(reinterpret_cast<const unsigned short *>(b + h * 64 + 32 + 2 * pp));
        uint32_t hv2 = __ldg(reinterpret_cast<const unsigned short *>(b + 128 + h * 32 + 2 * pp));
        const signed char *scp = reinterpret_cast<const signed char *>(b + 192) + h * 8 + (pp >> 3);
        const int8_t *xb = xq + sb * 256 + h * 128 + 2 * pp;
        int a = 0;
#pragma unroll
        for (int qd = 0; qd < 4; qd++) {
            uint32_t x2 = *reinterpret_cast<const unsigned short *>(xb + qd * 32);
            int part = 0;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                uint32_t la = (la2 >> (8 * e)) & 0xffu, lb = (lb2 >> (8 * e)) & 0xffu, hv = (hv2 >> (8 * e)) & 0xffu;
                uint32_t lowsrc = (qd & 1) ? lb : la;
                uint32_t low = (qd & 2) ? (lowsrc >> 4) : (lowsrc & 0xFu);
                uint32_t high = (hv >> (2 * qd)) & 3u;
                int val = (int)(low | (high << 4)) - 32;
                int xv = (int)(signed char)((x2 >> (8 * e)) & 0xffu);
                part += val * xv;
            }
            a += part * (int)__ldg(scp + qd * 2);
        }
        a = __reduce_add_sync(0xffffffffu, a);
        float d = half_bits_to_f32(__ldg(reinterpret_cast<const unsigned short *>(b + 208)));
        sumf = __fadd_rn(sumf, __fmul_rn(__fmul_rn(ys[sb], d), (float)a));
        if (dbg && lane == 0) dbg[sb] = a;
    }
    return sumf;
}

// A K-quant matrix on the device: rows in the GGUF byte layout, type 12 (Q4_K) or 14 (Q6_K).
struct KMatDev {
    const uint8_t *p;
    int type, rows, cols;
    __host__ __device__ size_t bpr() const { return (size_t)(cols / 256) * (type == 12 ? 144 : 210); }
};

__device__ __forceinline__ float kq_row_dot(const KMatDev &m, size_t row, const int8_t *xq, const float *ys, const int32_t *bsum, int lane) {
    const uint8_t *r = m.p + row * m.bpr();
    return m.type == 12 ? q4k_row_dot(r, m.cols / 256, xq, ys, bsum, lane) : q6k_row_dot(r, m.cols / 256, xq, ys, lane);
}

}  // namespace brrr
