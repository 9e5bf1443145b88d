// Stage-level K-quant kernels of the qwen3moe decode path: the Q8_K activation quantiser and the
// Q4_K / Q6_K x Q8_K matrix-vector products, on weights in the GGUF byte layout.  One warp per
// superblock (quantiser) or per row (products); the arithmetic is in brrr_kq.cuh.
#include "brrr_kernels.h"
#include "brrr_kq.cuh"

namespace brrr {

namespace {

__global__ void __launch_bounds__(256) quant_q8k_kernel(const float *__restrict__ x, int nsb, int8_t *__restrict__ q,
                                                        float *__restrict__ s, int32_t *__restrict__ bsum) {
    int sb = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (sb >= nsb) return;
    const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)sb * 256 + lane * 8);
    float4 a = src[0], b = src[1];
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    warp_quant_q8k(v, lane, q + (size_t)sb * 256, s + sb, bsum + sb * 8);
}

__global__ void __launch_bounds__(256) q4k_matvec_kernel(const uint8_t *__restrict__ w, int rows, int nsb, const int8_t *__restrict__ xq,
                                                         const float *__restrict__ ys, const int32_t *__restrict__ bsum,
                                                         float *__restrict__ y, int32_t *__restrict__ dbg) {
    int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= rows) return;
    float v = q4k_row_dot(w + (size_t)row * nsb * 144, nsb, xq, ys, bsum, lane, dbg ? dbg + (size_t)row * nsb * 2 : nullptr);
    if (lane == 0) y[row] = v;
}

__global__ void __launch_bounds__(256) q6k_matvec_kernel(const uint8_t *__restrict__ w, int rows, int nsb, const int8_t *__restrict__ xq,
                                                         const float *__restrict__ ys, float *__restrict__ y, int32_t *__restrict__ dbg) {
    int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= rows) return;
    float v = q6k_row_dot(w + (size_t)row * nsb * 210, nsb, xq, ys, lane, dbg ? dbg + (size_t)row * nsb : nullptr);
    if (lane == 0) y[row] = v;
}

}  // namespace

void launch_quant_q8k(const float *x, int n, int8_t *q, float *s, int32_t *bsum, cudaStream_t st) {
    int nsb = n / 256;
    quant_q8k_kernel<<<(nsb + 7) / 8, 256, 0, st>>>(x, nsb, q, s, bsum);
}

void launch_q4k_matvec(const uint8_t *w, int rows, int cols, const int8_t *xq, const float *ys, const int32_t *bsum, float *y,
                       int32_t *dbg, cudaStream_t st) {
    q4k_matvec_kernel<<<(rows + 7) / 8, 256, 0, st>>>(w, rows, cols / 256, xq, ys, bsum, y, dbg);
}

void launch_q6k_matvec(const uint8_t *w, int rows, int cols, const int8_t *xq, const float *ys, float *y, int32_t *dbg, cudaStream_t st) {
    q6k_matvec_kernel<<<(rows + 7) / 8, 256, 0, st>>>(w, rows, cols / 256, xq, ys, y, dbg);
}

}  // namespace brrr
