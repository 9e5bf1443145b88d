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

// A K-quant matrix on the device, type 12 (Q4_K) or 14 (Q6_K).  Q4_K rows stay in the GGUF byte
// layout (144-byte superblocks, 16-byte aligned).  Q6_K rows are either in the GGUF layout (210-byte
// superblocks, 2-byte aligned: planes == 0) or re-laid at load time into four aligned planes per row
// (planes == 1): ql [nsb][128] | qh [nsb][64] | scales [nsb][16] | d [nsb] f16, padded to 16 bytes -
// a byte permutation, so every integer of the dot is unchanged.
struct KMatDev {
    const uint8_t *p;
    int type, rows, cols;
    int planes;
    __host__ __device__ size_t bpr() const {
        const size_t nsb = (size_t)(cols / 256);
        if (type == 12) return nsb * 144;
        return planes ? nsb * 208 + ((nsb * 2 + 15) & ~(size_t)15) : nsb * 210;
    }
};
// bytes of a row in the GGUF layout (the algorithmic figure, whatever the device layout)
__host__ __device__ __forceinline__ size_t kq_gguf_row_bytes(int type, int cols) { return (size_t)(cols / 256) * (type == 12 ? 144 : 210); }
__host__ __device__ __forceinline__ size_t q6k_plane_row_bytes(int nsb) { return (size_t)nsb * 208 + (((size_t)nsb * 2 + 15) & ~(size_t)15); }

// The qwen3moe RMS norm sums squares in 12 contiguous slices (the reference's 12 workers), each
// serially and unfused, and adds the partial sums in worker order (engine_qwen2.rs:15, 453-465).
constexpr int QW_NT = 12;
// worker w's contiguous slice of n items (engine_qwen2.rs:246-252)
__device__ __forceinline__ void qw_slice(int w, int n, int &a, int &b) {
    int base = n / QW_NT, rem = n % QW_NT;
    a = w * base + min(w, rem);
    b = a + base + (w < rem ? 1 : 0);
}

// ---------------------------------------------------------------- lane-group form (decode kernels)
// Eight lanes own one superblock (a warp covers four superblocks at a time) and every lane moves 16
// bytes per load.  A unit = what one lane holds of one superblock.
//   Q4_K:         a = the 16-byte header (d | dmin, 12 packed scale bytes), b = nibble bytes 16 l8 .. 16 l8 + 15
//   Q6_K planes:  a = ql bytes 16 l8 .. +15, b = the 16 qh bytes that go with them,
//                 c = scale of the low nibbles | scale of the high nibbles << 8 | d (f16 bits) << 16
struct KUnit { uint4 a, b; uint32_t c; };

__device__ __forceinline__ void kq_unit_load(const KMatDev &m, const uint8_t *row, int sb, int l8, KUnit &u) {
    if (m.type == 12) {
        const uint4 *p = reinterpret_cast<const uint4 *>(row + (size_t)sb * 144);
        u.a = __ldg(p);
        u.b = __ldg(p + 1 + l8);
        u.c = 0u;
    } else {
        const int nsb = m.cols / 256, h = l8 >> 2, q = l8 & 3;
        u.a = __ldg(reinterpret_cast<const uint4 *>(row + (size_t)sb * 128 + 16 * l8));
        u.b = __ldg(reinterpret_cast<const uint4 *>(row + (size_t)nsb * 128 + (size_t)sb * 64 + 32 * h + 16 * (q & 1)));
        const uint8_t *sc = row + (size_t)nsb * 192 + (size_t)sb * 16 + 8 * h + (q >= 2 ? 2 : 0) + (q & 1);
        const uint32_t dh = __ldg(reinterpret_cast<const unsigned short *>(row + (size_t)nsb * 208 + (size_t)sb * 2));
        u.c = (uint32_t)__ldg(sc) | ((uint32_t)__ldg(sc + 4) << 8) | (dh << 16);
    }
}

// The superblock's term of the row sum, valid in all eight lanes of the group: (ys d) acc - (ys dmin) mint
// for Q4_K, (ys d) acc for Q6_K, every product rounded separately as in q4k_row_dot / q6k_row_dot.
// xsb: the 256 int8 activations of the superblock (16-byte aligned), bs: its eight 32-sums, gmask: the
// group's lanes.
__device__ __forceinline__ float kq_unit_term(int type, const KUnit &u, int l8, const int8_t *xsb, float ys, const int32_t *bs, unsigned gmask) {
    if (type == 12) {
        const int jj = l8 >> 1, hh = l8 & 1;
        const int4 x0 = *reinterpret_cast<const int4 *>(xsb + (2 * jj) * 32 + 16 * hh);
        const int4 x1 = *reinterpret_cast<const int4 *>(xsb + (2 * jj + 1) * 32 + 16 * hh);
        int sc0, mn0, sc1, mn1, scj, mnj;
        k4_scale_min(u.a.y, u.a.z, u.a.w, 2 * jj, sc0, mn0);
        k4_scale_min(u.a.y, u.a.z, u.a.w, 2 * jj + 1, sc1, mn1);
        k4_scale_min(u.a.y, u.a.z, u.a.w, l8, scj, mnj);
        const uint32_t M = 0x0F0F0F0Fu;
        int lo = __dp4a((int)(u.b.x & M), x0.x, 0);
        lo = __dp4a((int)(u.b.y & M), x0.y, lo);
        lo = __dp4a((int)(u.b.z & M), x0.z, lo);
        lo = __dp4a((int)(u.b.w & M), x0.w, lo);
        int hi = __dp4a((int)((u.b.x >> 4) & M), x1.x, 0);
        hi = __dp4a((int)((u.b.y >> 4) & M), x1.y, hi);
        hi = __dp4a((int)((u.b.z >> 4) & M), x1.z, hi);
        hi = __dp4a((int)((u.b.w >> 4) & M), x1.w, hi);
        int a = lo * sc0 + hi * sc1;
        int mt = mnj * bs[l8];
        a = __reduce_add_sync(gmask, a);
        mt = __reduce_add_sync(gmask, mt);
        const float d = half_bits_to_f32(u.a.x & 0xffffu), dmin = half_bits_to_f32(u.a.x >> 16);
        return __fsub_rn(__fmul_rn(__fmul_rn(ys, d), (float)a), __fmul_rn(__fmul_rn(ys, dmin), (float)mt));
    }
    const int h = l8 >> 2, q = l8 & 3;
    const int base = 128 * h + (q >= 2 ? 32 : 0) + 16 * (q & 1);
    const int4 xl = *reinterpret_cast<const int4 *>(xsb + base);
    const int4 xh = *reinterpret_cast<const int4 *>(xsb + base + 64);
    const int sl = q >= 2 ? 2 : 0, sh = sl + 4;
    const uint32_t M4 = 0x0F0F0F0Fu, M2 = 0x03030303u;
    int accl = 0, acch = 0, sxl = 0, sxh = 0;
#define BRRR_Q6_WORD(QL, QH, XL, XH)                                                                   \
    accl = __dp4a((int)(((QL) & M4) | ((((QH) >> sl) & M2) << 4)), (XL), accl);                         \
    acch = __dp4a((int)((((QL) >> 4) & M4) | ((((QH) >> sh) & M2) << 4)), (XH), acch);                  \
    sxl = __dp4a(0x01010101, (XL), sxl);                                                                \
    sxh = __dp4a(0x01010101, (XH), sxh);
    BRRR_Q6_WORD(u.a.x, u.b.x, xl.x, xh.x)
    BRRR_Q6_WORD(u.a.y, u.b.y, xl.y, xh.y)
    BRRR_Q6_WORD(u.a.z, u.b.z, xl.z, xh.z)
    BRRR_Q6_WORD(u.a.w, u.b.w, xl.w, xh.w)
#undef BRRR_Q6_WORD
    const int scl = (int)(signed char)(u.c & 0xffu), sch = (int)(signed char)((u.c >> 8) & 0xffu);
    int a = (accl - 32 * sxl) * scl + (acch - 32 * sxh) * sch;
    a = __reduce_add_sync(gmask, a);
    return __fmul_rn(__fmul_rn(ys, half_bits_to_f32(u.c >> 16)), (float)a);
}

__device__ __forceinline__ float kq_row_dot(const KMatDev &m, size_t row, const int8_t *xq, const float *ys, const int32_t *bsum, int lane) {
    const uint8_t *r = m.p + row * m.bpr();
    return m.type == 12 ? q4k_row_dot(r, m.cols / 256, xq, ys, bsum, lane) : q6k_row_dot(r, m.cols / 256, xq, ys, lane);
}

}  // namespace brrr
