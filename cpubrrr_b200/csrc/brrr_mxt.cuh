// Operand B of the fp4 tensor-core expert matvecs (kernels_mxt.cu): the digit-plane image of a Q8
// activation, written by whichever kernel quantises the activation.
//
// An activation byte x in [-127, 127] is 49 a + 7 b + c with digits in [-3, 3]; twice a digit
// (0, +-2, +-4, +-6) is an e2m1 value.  Image of one block pair p (768 bytes): for kc = 0, 1 (the
// block of the pair), digit plane t = 0..2 (a, b, c), column q * 4 + j (q = block of the pair,
// j = lane chain): 16 bytes at p * 768 + kc * 384 + t * 128 + (q * 4 + j) * 16, byte i holding the
// codes of positions i (low nibble) and 16 + i (high nibble) of block 2 p + kc.  Column (q, j) is
// non-zero only for kc = q and bytes 4 j .. 4 j + 3, so a producer writes one word per (block, lane,
// plane) and the rest of the image stays zero from its allocation.
#pragma once
#include "brrr_dev.cuh"

namespace brrr {

constexpr int XT_N = 24;                 // MMA N: 3 digit planes x 2 blocks x 4 lanes
constexpr int XT_B_PAIR = XT_N * 32;     // operand B bytes per block pair

// e2m1 codes of twice the digits of x: a | b << 4 | c << 8
__device__ __forceinline__ uint32_t xt_digits(int x) {
    const int a = (x + 171) / 49 - 3;
    const int r = x - 49 * a;
    const int b = (r + 24) / 7 - 3;
    const int c = r - 7 * b;
    auto code = [](int v) -> uint32_t {
        const int m = v < 0 ? -v : v;
        const uint32_t mag = m == 0 ? 0u : (m == 1 ? 4u : (m == 2 ? 6u : 7u));
        return mag | (v < 0 ? 8u : 0u);
    };
    return code(a) | (code(b) << 4) | (code(c) << 8);
}

// One 32-block held one quantised value per lane: writes the block's 12 words of the image.
// Must be called by all 32 lanes.
__device__ __forceinline__ void xt_emit_block(int qv, int lane, int b, uint8_t *bimg) {
    const uint32_t dig = xt_digits(qv);
    const int p = b >> 1, q = b & 1, j = (lane & 15) >> 2;
    uint8_t *base = bimg + (size_t)p * XT_B_PAIR + q * (XT_B_PAIR / 2) + (q * 4 + j) * 16 + 4 * j;
#pragma unroll
    for (int t = 0; t < 3; t++) {
        const uint32_t nib = (dig >> (4 * t)) & 15u;
        const uint32_t other = __shfl_xor_sync(0xffffffffu, nib, 16);
        uint32_t w = (nib | (other << 4)) << (8 * (lane & 3));     // lanes < 16: byte i = code(i) | code(16 + i) << 4
        w |= __shfl_xor_sync(0xffffffffu, w, 1);
        w |= __shfl_xor_sync(0xffffffffu, w, 2);
        if (lane < 16 && (lane & 3) == 0) *reinterpret_cast<uint32_t *>(base + t * 128) = w;
    }
}

}  // namespace brrr
