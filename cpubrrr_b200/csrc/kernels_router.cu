// FFN entry stage: RMSNorm of the residual stream, Q8 quantisation of the result, router GEMV
// and top-k softmax.
//
// The router logit of expert e is the *serial* f32 sum  acc = b[e]; acc += W[e][j] * xn[j]
// for j ascending, multiply and add rounded separately.  That chain cannot be split without
// changing bits, so one lane owns one expert and walks the whole row; the other warps of the CTA
// stream W from memory and pre-multiply the products into shared-memory tiles (double buffered),
// leaving the chain lane one LDS + one FADD per element.  Experts are split 32 per CTA; the last
// CTA to finish performs the top-k.
#include "brrr_kernels.h"
#include "brrr_block.cuh"

namespace brrr {

constexpr int RT_TJ = 256;                 // tile width (elements of d)
constexpr int RT_STRIDE = RT_TJ + 1;       // padded row stride: lane e reads bank (e + j) % 32
constexpr int RT_THREADS = 1024;

__global__ void __launch_bounds__(RT_THREADS) ffn_in_kernel(const float *__restrict__ x_in, const float *__restrict__ norm_w, float eps, int d,
                                                            int8_t *__restrict__ xq_out, float *__restrict__ xs_out,
                                                            const float *__restrict__ W, const float *__restrict__ b, int ne, int topk,
                                                            float *__restrict__ logits, int32_t *__restrict__ top, float *__restrict__ wts,
                                                            unsigned int *counter) {
    extern __shared__ __align__(16) unsigned char smraw[];
    float *xn = reinterpret_cast<float *>(smraw);                 // d floats
    float *prod = xn + d;                                         // [2][32][RT_STRIDE]
    __shared__ float inv_sh;
    __shared__ int last_sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    for (int i = tid; i < d; i += RT_THREADS) xn[i] = x_in[i];
    __syncthreads();
    if (norm_w) {
        float inv = block_rms_inv(xn, d, eps, &inv_sh);
        for (int i = tid; i < d; i += RT_THREADS) xn[i] = __fmul_rn(__fmul_rn(xn[i], inv), norm_w[i]);
        __syncthreads();
    }
    if (xq_out && blockIdx.x == 0)
        for (int blk = warp; blk < d / 32; blk += RT_THREADS / 32) warp_quant_block(xn[blk * 32 + lane], lane, xq_out + blk * 32, xs_out + blk);

    const int e0 = blockIdx.x * 32;
    const int nloc = min(32, ne - e0);
    const int ntiles = (d + RT_TJ - 1) / RT_TJ;
    const int ptid = tid - 32;                                    // producer thread id (warps 1..31)
    float acc = (warp == 0 && lane < nloc && b) ? b[e0 + lane] : 0.0f;

    // producers fill tile t into buffer t & 1
    auto fill = [&](int t) {
        float *buf = prod + (size_t)(t & 1) * 32 * RT_STRIDE;
        int j0 = t * RT_TJ;
        for (int idx = ptid; idx < 32 * RT_TJ; idx += RT_THREADS - 32) {
            int e = idx / RT_TJ, jj = idx % RT_TJ, j = j0 + jj;
            if (e < nloc && j < d) buf[e * RT_STRIDE + jj] = __fmul_rn(__ldg(W + (size_t)(e0 + e) * d + j), xn[j]);
        }
    };
    if (warp != 0) fill(0);
    __syncthreads();
    for (int t = 0; t < ntiles; t++) {
        if (warp != 0) {
            if (t + 1 < ntiles) fill(t + 1);
        } else if (lane < nloc) {
            const float *row = prod + (size_t)(t & 1) * 32 * RT_STRIDE + lane * RT_STRIDE;
            int len = min(RT_TJ, d - t * RT_TJ);
#pragma unroll 16
            for (int jj = 0; jj < len; jj++) acc = __fadd_rn(acc, row[jj]);
        }
        __syncthreads();
    }
    if (warp == 0 && lane < nloc) logits[e0 + lane] = acc;

    // last CTA to arrive runs the top-k
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned prev = atomicAdd(counter, 1u);
        last_sh = (prev == gridDim.x - 1);
    }
    __syncthreads();
    if (!last_sh) return;
    __threadfence();
    if (tid == 0) {
        // insertion top-k, strict '>', so equal logits keep the lower expert index first
        int tp[8];
        float tv[8];
        for (int i = 0; i < 8; i++) { tp[i] = 0; tv[i] = -3.402823466e+38f; }
        for (int e = 0; e < ne; e++) {
            float v = __ldcg(logits + e);
            if (v > tv[topk - 1]) {
                int p = topk - 1;
                while (p > 0 && tv[p - 1] < v) { tv[p] = tv[p - 1]; tp[p] = tp[p - 1]; p--; }
                tv[p] = v; tp[p] = e;
            }
        }
        float ex[8], wsum = 0.0f;
        for (int i = 0; i < topk; i++) { ex[i] = brrr_expf_dev(__fsub_rn(tv[i], tv[0])); wsum = __fadd_rn(wsum, ex[i]); }
        for (int i = 0; i < topk; i++) { wts[i] = __fdiv_rn(ex[i], wsum); top[i] = tp[i]; }
        *counter = 0u;
    }
}

static size_t ffn_in_smem(int d) { return (size_t)d * sizeof(float) + (size_t)2 * 32 * RT_STRIDE * sizeof(float); }

int ffn_in_init() {
    return (int)cudaFuncSetAttribute(ffn_in_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ffn_in_smem(8192));
}

void launch_ffn_in(const float *x_in, const float *norm_w, float eps, int d, int8_t *xq_out, float *xs_out,
                   const float *W, const float *b, int ne, int topk, float *logits, int32_t *top, float *wts,
                   unsigned int *counter, cudaStream_t st) {
    unsigned grid = (ne + 31) / 32;
    ffn_in_kernel<<<grid, RT_THREADS, ffn_in_smem(d), st>>>(x_in, norm_w, eps, d, xq_out, xs_out, W, b, ne, topk, logits, top, wts, counter);
}

}  // namespace brrr
