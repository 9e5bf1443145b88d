// MXFP4 expert matrices: load-time re-layout of GGUF blocks and the expert matvecs.
//
// Float order of one row (fixed): 4 lane chains.  Chain j walks the blocks b = 0, 1, ...
// accumulating fma(float(t_j(b)), 2^(e_b - 128) * xs[b], acc), t_j(b) being the exact int32
// lane dot (brrr_mx_lane_dot); the row result is (a0+a1)+(a2+a3).  One thread owns one chain;
// 8 rows x 4 lanes make a warp and every step of the warp is one contiguous 256-byte read
// covering two blocks.
#include "brrr_kernels.h"
#include "brrr_block.cuh"

namespace brrr {

// ---------------------------------------------------------------- pack: GGUF rows -> MxDev
// raw: [rows][blocks][17] (e8m0 byte, then 16 nibble bytes).  One thread per (row, block, lane).
__global__ void mx_pack_kernel(const uint8_t *__restrict__ raw, MxDev m) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)m.rows * m.blocks * 4;
    if (idx >= total) return;
    int j = (int)(idx & 3);
    size_t rb = idx >> 2;
    int b = (int)(rb % m.blocks), row = (int)(rb / m.blocks);
    const uint8_t *src = raw + rb * 17;
    int np = m.blocks / 2;
    uint32_t w = (uint32_t)src[1 + 4 * j] | ((uint32_t)src[2 + 4 * j] << 8) | ((uint32_t)src[3 + 4 * j] << 16) | ((uint32_t)src[4 + 4 * j] << 24);
    *reinterpret_cast<uint32_t *>(m.nib + mx_noff(row, b >> 1, np) + j * 8 + (b & 1) * 4) = w;
    if (j == 0) m.exps[mx_eoff(row, b >> 1, np) + (b & 1)] = src[0];
}

void launch_mx_pack(const uint8_t *raw, MxDev m, cudaStream_t st) {
    size_t total = (size_t)m.rows * m.blocks * 4;
    if (!total) return;
    mx_pack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(raw, m);
}

// ---------------------------------------------------------------- activation staging
// Shared-memory image of a Q8 activation for the MXFP4 lane dot: one int2 {xa, xb} per
// (block, lane), bytes interleaved to the prmt output order (see brrr_mx_lane_dot).
__device__ __forceinline__ void mx_stage_x(const int8_t *__restrict__ xq, const float *__restrict__ xs, int nb, int2 *xp, float *xsc, int tid, int nthreads) {
    for (int idx = tid; idx < nb * 4; idx += nthreads) {
        int b = idx >> 2, j = idx & 3;
        const uint32_t *xw = reinterpret_cast<const uint32_t *>(xq + b * 32);
        uint32_t lo = xw[j], hi = xw[4 + j];
        xp[idx] = make_int2((int)brrr_prmt(lo, hi, 0x5140u), (int)brrr_prmt(lo, hi, 0x7362u));
    }
    for (int b = tid; b < nb; b += nthreads) xsc[b] = xs[b];
}

// One lane chain over all blocks of a row.  nibp / expp point at the thread's first 8 / 2 bytes.
template <bool DBG>
__device__ __forceinline__ float mx_chain(const uint8_t *__restrict__ nibp, const uint8_t *__restrict__ expp, const int2 *xpj, const float *xsc,
                                          int np, int32_t *dbg /* [blocks][4], this lane's column */) {
    float acc = 0.0f;
#pragma unroll 8
    for (int i = 0; i < np; i++) {
        uint2 w = __ldg(reinterpret_cast<const uint2 *>(nibp + (size_t)i * 256));
        uint32_t e2 = __ldg(reinterpret_cast<const unsigned short *>(expp + (size_t)i * 16));
        int2 x0 = xpj[i * 8], x1 = xpj[i * 8 + 4];
        int t0 = brrr_mx_lane_dot(w.x, x0.x, x0.y);
        int t1 = brrr_mx_lane_dot(w.y, x1.x, x1.y);
        if (DBG) { dbg[(2 * i) * 4] = t0; dbg[(2 * i + 1) * 4] = t1; }
        float sv0 = __fmul_rn(brrr_e8m0_scale(e2 & 0xFFu), xsc[2 * i]);
        float sv1 = __fmul_rn(brrr_e8m0_scale(e2 >> 8), xsc[2 * i + 1]);
        acc = __fmaf_rn((float)t0, sv0, acc);
        acc = __fmaf_rn((float)t1, sv1, acc);
    }
    return acc;
}

// ---------------------------------------------------------------- plain matvec (stage-level / tests)
template <bool DBG>
__global__ void __launch_bounds__(256) mx_gemv_kernel(MxDev m, int row0, int nrows, const int8_t *__restrict__ xq, const float *__restrict__ xs,
                                                      float *__restrict__ y, int32_t *__restrict__ blockdots) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int nb = m.blocks, np = nb / 2;
    int2 *xp = reinterpret_cast<int2 *>(smraw);
    float *xsc = reinterpret_cast<float *>(smraw + (size_t)nb * 4 * sizeof(int2));
    mx_stage_x(xq, xs, nb, xp, xsc, threadIdx.x, 256);
    __syncthreads();
    int rl = blockIdx.x * 64 + (threadIdx.x >> 2), j = threadIdx.x & 3;
    bool live = rl < nrows;
    float acc = 0.0f;
    if (live) {
        int row = row0 + rl;
        acc = mx_chain<DBG>(m.nib + mx_noff(row, 0, np) + j * 8, m.exps + mx_eoff(row, 0, np), xp + j, xsc, np,
                            DBG ? blockdots + (size_t)rl * nb * 4 + j : nullptr);
    }
    acc = brrr_hsum4(acc);
    if (live && j == 0) y[rl] = acc;
}

void launch_mx_gemv(MxDev m, int row0, int nrows, const int8_t *xq, const float *xs, float *y, int32_t *blockdots, cudaStream_t st) {
    size_t smem = (size_t)m.blocks * 4 * sizeof(int2) + m.blocks * sizeof(float);
    unsigned grid = (nrows + 63) / 64;
    if (blockdots) mx_gemv_kernel<true><<<grid, 256, smem, st>>>(m, row0, nrows, xq, xs, y, blockdots);
    else mx_gemv_kernel<false><<<grid, 256, smem, st>>>(m, row0, nrows, xq, xs, y, blockdots);
}

// ---------------------------------------------------------------- gate / up of the selected experts
// grid (ceil(d/64), 2, topk): 64 rows of expert top[z]'s gate (y = 0) or up (y = 1) matrix.
// gu[ei][2d] = gate | up, bias added.
__global__ void __launch_bounds__(256) gate_up_kernel(MxDev gate, MxDev up, const float *__restrict__ gate_b, const float *__restrict__ up_b,
                                                      const int32_t *__restrict__ top, int d, const int8_t *__restrict__ xq,
                                                      const float *__restrict__ xs, float *__restrict__ gu) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int nb = gate.blocks, np = nb / 2;
    int2 *xp = reinterpret_cast<int2 *>(smraw);
    float *xsc = reinterpret_cast<float *>(smraw + (size_t)nb * 4 * sizeof(int2));
    mx_stage_x(xq, xs, nb, xp, xsc, threadIdx.x, 256);
    __syncthreads();
    const int ei = blockIdx.z, isup = blockIdx.y;
    const int e = top[ei];
    const MxDev &m = isup ? up : gate;
    const float *bias = isup ? up_b : gate_b;
    int r = blockIdx.x * 64 + (threadIdx.x >> 2), j = threadIdx.x & 3;
    bool live = r < d;
    float acc = 0.0f;
    if (live) {
        int row = e * d + r;
        acc = mx_chain<false>(m.nib + mx_noff(row, 0, np) + j * 8, m.exps + mx_eoff(row, 0, np), xp + j, xsc, np, nullptr);
    }
    acc = brrr_hsum4(acc);
    if (live && j == 0) gu[(size_t)ei * 2 * d + (size_t)isup * d + r] = __fadd_rn(acc, bias[(size_t)e * d + r]);
}

void launch_gate_up(MxDev gate, MxDev up, const float *gate_b, const float *up_b, const int32_t *top, int topk, int d,
                    const int8_t *xq, const float *xs, float *gu, cudaStream_t st) {
    size_t smem = (size_t)gate.blocks * 4 * sizeof(int2) + gate.blocks * sizeof(float);
    dim3 grid((d + 63) / 64, 2, topk);
    gate_up_kernel<<<grid, 256, smem, st>>>(gate, up, gate_b, up_b, top, d, xq, xs, gu);
}

// ---------------------------------------------------------------- down + weighted combine
// 16 output rows per CTA; warp (ei, half) computes 8 rows of expert top[ei]; then one thread per
// row folds s = x; s += wts[ei] * (acc_ei + bias) for ei ascending (multiply then add).
__global__ void down_combine_kernel(MxDev down, const float *__restrict__ down_b, const int32_t *__restrict__ top, const float *__restrict__ wts,
                                    int topk, int d, const int8_t *__restrict__ hq, const float *__restrict__ hs, float *__restrict__ x) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int nb = down.blocks, np = nb / 2;
    const size_t per = (size_t)nb * 4 * sizeof(int2) + nb * sizeof(float);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ei = warp >> 1, half = warp & 1;
    // each pair of warps stages its own expert slot's activation
    int2 *xp = reinterpret_cast<int2 *>(smraw + per * ei);
    float *xsc = reinterpret_cast<float *>(smraw + per * ei + (size_t)nb * 4 * sizeof(int2));
    float *part = reinterpret_cast<float *>(smraw + per * topk);   // [topk][16]
    mx_stage_x(hq + (size_t)ei * d, hs + (size_t)ei * nb, nb, xp, xsc, half * 32 + lane, 64);
    __syncthreads();
    const int e = top[ei];
    int rl = half * 8 + (lane >> 2), j = lane & 3;
    int r = blockIdx.x * 16 + rl;
    bool live = r < d;
    float acc = 0.0f;
    if (live) {
        int row = e * d + r;
        acc = mx_chain<false>(down.nib + mx_noff(row, 0, np) + j * 8, down.exps + mx_eoff(row, 0, np), xp + j, xsc, np, nullptr);
    }
    acc = brrr_hsum4(acc);
    if (j == 0) part[ei * 16 + rl] = acc;
    __syncthreads();
    if (threadIdx.x < 16) {
        int rr = blockIdx.x * 16 + threadIdx.x;
        if (rr < d) {
            float s = x[rr];
            for (int k = 0; k < topk; k++) {
                int ek = top[k];
                s = __fadd_rn(s, __fmul_rn(wts[k], __fadd_rn(part[k * 16 + threadIdx.x], down_b[(size_t)ek * d + rr])));
            }
            x[rr] = s;
        }
    }
}

void launch_down_combine(MxDev down, const float *down_b, const int32_t *top, const float *wts, int topk, int d,
                         const int8_t *hq, const float *hs, float *x, cudaStream_t st) {
    size_t per = (size_t)down.blocks * 4 * sizeof(int2) + down.blocks * sizeof(float);
    size_t smem = per * topk + (size_t)topk * 16 * sizeof(float);
    down_combine_kernel<<<(d + 15) / 16, topk * 64, smem, st>>>(down, down_b, top, wts, topk, d, hq, hs, x);
}

}  // namespace brrr
