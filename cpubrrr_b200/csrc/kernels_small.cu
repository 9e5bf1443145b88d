// Small stages of the decode step: activation quantiser, RMSNorm, embedding gather, clamped
// SwiGLU, token hand-over, and the synthetic tensor fill.
#include "brrr_kernels.h"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"
#include "brrr_synth.h"

namespace brrr {

// ---------------------------------------------------------------- Q8 activation quantiser
// One warp per 32-block: lane i owns element i; amax by butterfly max (order-free), one true
// division for the scale, one per element for the quotient.
__global__ void quant_q8_kernel(const float *__restrict__ x, int nblocks, int8_t *__restrict__ q, float *__restrict__ s) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= nblocks) return;
    float v = x[warp * 32 + lane];
    warp_quant_block(v, lane, q + warp * 32, s + warp);
}

void launch_quant_q8(const float *x, int n, int8_t *q, float *s, cudaStream_t st) {
    int nb = n / 32;
    if (nb <= 0) return;
    quant_q8_kernel<<<(nb + 7) / 8, 256, 0, st>>>(x, nb, q, s);
}

// ---------------------------------------------------------------- RMSNorm + quantiser
// Single CTA.  The sum of squares follows the 16-chain order (block_rms_inv); the scaling is
// (x * inv) * w with two separately rounded multiplies.
__global__ void __launch_bounds__(512) rmsnorm_quant_kernel(const float *__restrict__ x, const float *__restrict__ w, float eps, int n,
                                                            float *__restrict__ xn, int8_t *__restrict__ q, float *__restrict__ s) {
    extern __shared__ __align__(16) float sm[];      // n floats of x, then n floats of norm weights
    __shared__ float inv_sh;
    float *wn = sm + n;
    // one CTA per row (token): rows are n floats apart in x and xn, n quants and n / 32 scales apart in q and s
    x += (size_t)blockIdx.x * n;
    if (xn) xn += (size_t)blockIdx.x * n;
    if (q) q += (size_t)blockIdx.x * n;
    if (s) s += (size_t)blockIdx.x * (n / 32);
    stage_vec4(w, wn, n, threadIdx.x, blockDim.x);   // static: fetched before the wait
    float4 wreg[4];
    norm_prefetch<4>(w, n, wreg, threadIdx.x, blockDim.x);
    pdl_wait();
    pdl_trigger();
    block_norm_quant<NQ_NATURAL, 4>(x, w, wreg, eps, n, sm, reinterpret_cast<int2 *>(q), s, &inv_sh, threadIdx.x, blockDim.x);
    if (xn) {
        float inv = inv_sh;
        for (int i = threadIdx.x; i < n; i += blockDim.x) xn[i] = __fmul_rn(__fmul_rn(sm[i], inv), wn[i]);
    }
}

cudaError_t launch_rmsnorm_quant(const float *x, const float *w, float eps, int n, float *xn, int8_t *q, float *s, bool pdl, cudaStream_t st,
                                 int rows) {
    return launch_k(rmsnorm_quant_kernel, dim3(rows), dim3(512), (size_t)n * 2 * sizeof(float), st, pdl, x, w, eps, n, xn, q, s);
}

// ---------------------------------------------------------------- embedding gather
__global__ void embed_kernel(const uint16_t *__restrict__ embd, int d, const DevState *__restrict__ state, float *__restrict__ x) {
    size_t tok = state->tok;
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < d; j += gridDim.x * blockDim.x)
        x[j] = brrr_bf16_to_f32(embd[tok * d + j]);
}

// the same for a token id given by the host (token tiles)
__global__ void embed_tok_kernel(const uint16_t *__restrict__ embd, int d, uint32_t tok, float *__restrict__ x) {
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < d; j += gridDim.x * blockDim.x)
        x[j] = brrr_bf16_to_f32(embd[(size_t)tok * d + j]);
}

void launch_embed_tok(const uint16_t *embd, int d, uint32_t tok, float *x, cudaStream_t st) {
    embed_tok_kernel<<<(d + 255) / 256, 256, 0, st>>>(embd, d, tok, x);
}

__global__ void embed_tile_kernel(const uint16_t *__restrict__ embd, int d, const uint32_t *__restrict__ toks, float *__restrict__ x) {
    const size_t tok = toks[blockIdx.y];
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < d; j += gridDim.x * blockDim.x)
        x[(size_t)blockIdx.y * d + j] = brrr_bf16_to_f32(embd[tok * d + j]);
}

void launch_embed_tile(const uint16_t *embd, int d, const uint32_t *toks_dev, int ntok, float *x, cudaStream_t st) {
    embed_tile_kernel<<<dim3((d + 255) / 256, ntok), 256, 0, st>>>(embd, d, toks_dev, x);
}

void launch_embed(const uint16_t *embd, int d, const DevState *state, float *x, cudaStream_t st) {
    embed_kernel<<<(d + 255) / 256, 256, 0, st>>>(embd, d, state, x);
}

// ---------------------------------------------------------------- clamped SwiGLU + quantiser
// gu[ei][2d] = gate | up.  One warp per (expert slot, 32-block).
__global__ void swiglu_quant_kernel(const float *__restrict__ gu, int topk, int d, int8_t *__restrict__ hq, float *__restrict__ hs) {
    int nb = d / 32;
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= topk * nb) return;
    int ei = warp / nb, blk = warp % nb;
    float g = gu[(size_t)ei * 2 * d + blk * 32 + lane];
    float u = gu[(size_t)ei * 2 * d + d + blk * 32 + lane];
    float v = swiglu_oai(g, u);
    warp_quant_block(v, lane, hq + (size_t)ei * d + blk * 32, hs + ei * nb + blk);
}

void launch_swiglu_quant(const float *gu, int topk, int d, int8_t *hq, float *hs, cudaStream_t st) {
    int nw = topk * (d / 32);
    swiglu_quant_kernel<<<(nw + 7) / 8, 256, 0, st>>>(gu, topk, d, hq, hs);
}

// ---------------------------------------------------------------- token hand-over
// Decodes the running argmax of the vocabulary projection, publishes it as the next step's
// input token, appends it to the output ring and advances the position.
__global__ void finish_token_kernel(DevState *state) {
    unsigned long long key = state->best;
    uint32_t tok = 0xFFFFFFFFu - (uint32_t)(key & 0xFFFFFFFFull);
    state->tok = tok;
    state->out[state->n_out % BRRR_MAXSEQ] = tok;
    state->n_out += 1;
    state->pos += 1;
    state->best = 0ull;
}

void launch_finish_token(DevState *state, cudaStream_t st) { finish_token_kernel<<<1, 1, 0, st>>>(state); }

// ---------------------------------------------------------------- exp (test hook)
__global__ void expf_kernel(const float *x, int n, float *y) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = brrr_expf_dev(x[i]);
}
void launch_expf(const float *x, int n, float *y, cudaStream_t st) { expf_kernel<<<(n + 255) / 256, 256, 0, st>>>(x, n, y); }

// ---------------------------------------------------------------- synthetic tensors
__global__ void synth_f32_kernel(uint64_t key, uint64_t n, float mean, float sigma, float *out) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        out[i] = brrr_synth_f32(key, i, mean, sigma);
}
__global__ void synth_bf16_kernel(uint64_t key, uint64_t n, float sigma, uint16_t *out) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        out[i] = brrr_synth_bf16(key, i, sigma);
}
__global__ void synth_mxfp4_kernel(uint64_t key, uint64_t first, uint64_t nblocks, uint8_t *out) {
    for (uint64_t b = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; b < nblocks; b += (uint64_t)gridDim.x * blockDim.x) {
        uint8_t tmp[17];
        brrr_synth_mxfp4_block(key, first + b, tmp);
        for (int i = 0; i < 17; i++) out[b * 17 + i] = tmp[i];
    }
}

__global__ void synth_q4k_kernel(uint64_t key, uint64_t nblocks, uint8_t *out) {
    for (uint64_t b = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; b < nblocks; b += (uint64_t)gridDim.x * blockDim.x) {
        uint8_t tmp[144];
        brrr_synth_q4k_block(key, b, tmp);
        uint32_t *dst = reinterpret_cast<uint32_t *>(out + b * 144);
        for (int i = 0; i < 36; i++) dst[i] = tmp[4 * i] | (tmp[4 * i + 1] << 8) | (tmp[4 * i + 2] << 16) | ((uint32_t)tmp[4 * i + 3] << 24);
    }
}
__global__ void synth_q6k_kernel(uint64_t key, uint64_t nblocks, uint8_t *out) {
    for (uint64_t b = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; b < nblocks; b += (uint64_t)gridDim.x * blockDim.x) {
        uint8_t tmp[210];
        brrr_synth_q6k_block(key, b, tmp);
        unsigned short *dst = reinterpret_cast<unsigned short *>(out + b * 210);
        for (int i = 0; i < 105; i++) dst[i] = (unsigned short)(tmp[2 * i] | (tmp[2 * i + 1] << 8));
    }
}

void launch_synth(uint64_t seed, uint32_t layer, uint32_t kind, uint32_t type, uint64_t nelems, void *out, cudaStream_t st, uint64_t first_elem) {
    uint64_t key = brrr_tensor_key(seed, layer, kind);
    float mean = (kind == BRRR_T_ATTN_NORM || kind == BRRR_T_FFN_NORM || kind == BRRR_T_OUT_NORM || kind == BRRR_T_Q_NORM ||
                  kind == BRRR_T_K_NORM) ? 1.0f : 0.0f;
    float sigma = kind == BRRR_T_SINKS ? 1.0f : 0.02f;
    uint64_t units = type == 39 ? nelems / 32 : (type == 12 || type == 14) ? nelems / 256 : nelems;
    if (units == 0) return;
    unsigned grid = (unsigned)((units + 255) / 256 < 148 * 16 ? (units + 255) / 256 : 148 * 16);
    if (type == 0) synth_f32_kernel<<<grid, 256, 0, st>>>(key, nelems, mean, sigma, (float *)out);
    else if (type == 30) synth_bf16_kernel<<<grid, 256, 0, st>>>(key, nelems, sigma, (uint16_t *)out);
    else if (type == 39) synth_mxfp4_kernel<<<grid, 256, 0, st>>>(key, first_elem / 32, units, (uint8_t *)out);
    else if (type == 12) synth_q4k_kernel<<<grid, 256, 0, st>>>(key, units, (uint8_t *)out);
    else if (type == 14) synth_q6k_kernel<<<grid, 256, 0, st>>>(key, units, (uint8_t *)out);
}

}  // namespace brrr
