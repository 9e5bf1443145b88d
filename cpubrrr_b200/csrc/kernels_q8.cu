// Q8 weight matrices: load-time quantisation from bf16 and the row . Q8-activation GEMV.
//
// Float order of one row (fixed): 8 chains = 2 block parities x 4 lanes.  Chain (p, j) walks the
// blocks b = p, p+2, ... accumulating fma(float(t_j(b)), ws[b]*xs[b], acc) where t_j(b) is the
// exact int32 dot of bytes 4j..4j+3 of both 16-byte halves of the block.  The row result is
// hsum4(acc_even + acc_odd).  One thread owns one chain; the chains of 4 rows make a warp and
// every step of the warp is one contiguous 256-byte read.
#include "brrr_kernels.h"
#include "brrr_block.cuh"

namespace brrr {

// ---------------------------------------------------------------- pack: bf16 [rows][cols] -> Q8Dev
// One warp per (row, block): lane i owns element i.
__global__ void q8_pack_kernel(const uint16_t *__restrict__ w, int rows_src, int row0_dst, Q8Dev m) {
    int nb = m.cols / 32, np = m.cols / 64;
    size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (warp >= (size_t)rows_src * nb) return;
    int r = (int)(warp / nb), b = (int)(warp % nb);
    float v = brrr_bf16_to_f32(w[(size_t)r * m.cols + b * 32 + lane]);
    float amax = fmaxf(warp_max(fabsf(v)), 1e-12f);
    float sc = __fdiv_rn(amax, 127.0f);
    int row = row0_dst + r, pair = b >> 1, p = b & 1;
    int j = (lane & 15) >> 2, byte = (lane & 3) + (lane >= 16 ? 4 : 0);
    m.wq[q8_woff(row, pair, np) + p * 32 + j * 8 + byte] = (int8_t)brrr_q8_round(v, sc);
    if (lane == 0) m.ws[q8_soff(row, pair, np) + p] = sc;
}

void launch_q8_pack(const uint16_t *w, int rows_src, int row0_dst, Q8Dev m, cudaStream_t st) {
    size_t warps = (size_t)rows_src * (m.cols / 32);
    if (!warps) return;
    q8_pack_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(w, rows_src, row0_dst, m);
}

__global__ void q8_export_kernel(Q8Dev m, int8_t *__restrict__ q, float *__restrict__ s) {
    int nb = m.cols / 32, np = m.cols / 64;
    size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (warp >= (size_t)m.rows * nb) return;
    int r = (int)(warp / nb), b = (int)(warp % nb);
    int pair = b >> 1, p = b & 1;
    int j = (lane & 15) >> 2, byte = (lane & 3) + (lane >= 16 ? 4 : 0);
    q[(size_t)r * m.cols + b * 32 + lane] = m.wq[q8_woff(r, pair, np) + p * 32 + j * 8 + byte];
    if (lane == 0) s[(size_t)r * nb + b] = m.ws[q8_soff(r, pair, np) + p];
}

void launch_q8_export(Q8Dev m, int8_t *q, float *s, cudaStream_t st) {
    size_t warps = (size_t)m.rows * (m.cols / 32);
    q8_export_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(m, q, s);
}

// ---------------------------------------------------------------- GEMV
// ROWS rows per CTA, 8 threads per row.  Shared memory: the activation re-laid as one int2 per
// (block, lane) = {x[32b+4j..+3], x[32b+16+4j..+3]} and the block scales.
template <int ROWS, int EPI>
__global__ void __launch_bounds__(ROWS * 8) q8_gemv_kernel(Q8Dev m, const int8_t *__restrict__ xq, const float *__restrict__ xs,
                                                           const float *__restrict__ bias, float *__restrict__ y, DevState *state) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int nb = m.cols / 32, np = m.cols / 64;
    int2 *xp = reinterpret_cast<int2 *>(smraw);
    float *xsc = reinterpret_cast<float *>(smraw + (size_t)nb * 4 * sizeof(int2));
    for (int idx = threadIdx.x; idx < nb * 4; idx += ROWS * 8) {
        int b = idx >> 2, j = idx & 3;
        const int *xw = reinterpret_cast<const int *>(xq + b * 32);
        xp[idx] = make_int2(xw[j], xw[4 + j]);
    }
    for (int b = threadIdx.x; b < nb; b += ROWS * 8) xsc[b] = xs[b];
    __syncthreads();

    const int row = blockIdx.x * ROWS + (threadIdx.x >> 3);
    const int c = threadIdx.x & 7, p = c >> 2, j = c & 3;
    const bool live = row < m.rows;
    float acc = 0.0f;
    if (live) {
        const int2 *wp = reinterpret_cast<const int2 *>(m.wq + q8_woff(row, 0, np) + p * 32 + j * 8);
        const float *sp = m.ws + q8_soff(row, 0, np) + p;
        const int2 *xpp = xp + p * 4 + j;
        const float *xsp = xsc + p;
#pragma unroll 8
        for (int i = 0; i < np; i++) {
            int2 w = __ldg(wp + (size_t)i * 32);
            float s = __ldg(sp + (size_t)i * 8);
            int2 xv = xpp[i * 8];
            int t = __dp4a(w.y, xv.y, __dp4a(w.x, xv.x, 0));
            acc = __fmaf_rn((float)t, __fmul_rn(s, xsp[i * 2]), acc);
        }
    }
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));   // acc_even + acc_odd, per lane
    acc = brrr_hsum4(acc);

    if (EPI == Q8_EPI_HEAD) {
        // logits + running argmax: first strict maximum = lowest index among equal values
        unsigned long long key = 0ull;
        if (live && c == 0) {
            y[row] = acc;
            key = ((unsigned long long)float_orderable(acc) << 32) | (0xFFFFFFFFu - (uint32_t)row);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
            key = other > key ? other : key;
        }
        __shared__ unsigned long long wbest[ROWS * 8 / 32];
        if ((threadIdx.x & 31) == 0) wbest[threadIdx.x >> 5] = key;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < ROWS * 8 / 32; w++) key = wbest[w] > key ? wbest[w] : key;
            atomicMax(&state->best, key);
        }
    } else if (live && c == 0) {
        if (EPI == Q8_EPI_PLAIN) y[row] = acc;
        else if (EPI == Q8_EPI_BIAS) y[row] = __fadd_rn(acc, bias[row]);
        else y[row] = __fadd_rn(y[row], __fadd_rn(acc, bias[row]));   // x += dot + bias
    }
}

template <int ROWS>
static void q8_gemv_dispatch(Q8Dev m, const int8_t *xq, const float *xs, const float *bias, float *y, int epi, DevState *state, cudaStream_t st) {
    int nb = m.cols / 32;
    size_t smem = (size_t)nb * 4 * sizeof(int2) + nb * sizeof(float);
    unsigned grid = (m.rows + ROWS - 1) / ROWS;
    switch (epi) {
    case Q8_EPI_PLAIN: q8_gemv_kernel<ROWS, Q8_EPI_PLAIN><<<grid, ROWS * 8, smem, st>>>(m, xq, xs, bias, y, state); break;
    case Q8_EPI_BIAS: q8_gemv_kernel<ROWS, Q8_EPI_BIAS><<<grid, ROWS * 8, smem, st>>>(m, xq, xs, bias, y, state); break;
    case Q8_EPI_RESID_BIAS: q8_gemv_kernel<ROWS, Q8_EPI_RESID_BIAS><<<grid, ROWS * 8, smem, st>>>(m, xq, xs, bias, y, state); break;
    case Q8_EPI_HEAD: q8_gemv_kernel<ROWS, Q8_EPI_HEAD><<<grid, ROWS * 8, smem, st>>>(m, xq, xs, bias, y, state); break;
    }
}

void launch_q8_gemv(Q8Dev m, const int8_t *xq, const float *xs, const float *bias, float *y, int epi, DevState *state, cudaStream_t st) {
    // Small matrices use 16 rows per CTA so the grid still covers the SMs.
    if (m.rows <= 148 * 32) q8_gemv_dispatch<16>(m, xq, xs, bias, y, epi, state, st);
    else q8_gemv_dispatch<32>(m, xq, xs, bias, y, epi, state, st);
}

}  // namespace brrr
