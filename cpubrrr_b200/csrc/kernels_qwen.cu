// Decode kernels of the qwen3moe engine (src/bin/engine_qwen2.rs:302-451): Q4_K embedding row,
// RMS norm with the reference's 12 partial sums + Q8_K quantisation, K-quant matrix-vector
// products with their epilogues, per-head QK norm + RoPE + cache append, full causal GQA
// attention (head_dim 128), SiLU-GLU experts, weighted down-projection and the vocabulary argmax.
//
// Float order: every sum the reference forms serially is formed serially by one thread here
// (norm partials, head mean square, softmax denominator, probability-weighted values, the
// expert combine); integer sums are exact and split across lanes.  All kernels start with the
// programmatic-dependent-launch wait, so they can be chained in one stream or graph.
#include "brrr_kernels.h"
#include "brrr_kq.cuh"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"

namespace brrr {

namespace {

constexpr int QW_NT = 12;          // the reference's worker count fixes the norm's summation tree (engine_qwen2.rs:15)
constexpr int QW_HD = 128;

// worker w's contiguous slice of n items (engine_qwen2.rs:246-252)
__device__ __forceinline__ void qw_slice(int w, int n, int &a, int &b) {
    int base = n / QW_NT, rem = n % QW_NT;
    a = w * base + min(w, rem);
    b = a + base + (w < rem ? 1 : 0);
}

// ---------------------------------------------------------------- embedding (engine_qwen2.rs:310-330)
__global__ void __launch_bounds__(256) qw_embed_kernel(const uint8_t *__restrict__ embd, int d, const DevState *__restrict__ state,
                                                       float *__restrict__ x) {
    pdl_wait();
    pdl_trigger();
    const size_t tok = state->tok;
    const int sb = blockIdx.x, i = threadIdx.x;
    const uint32_t *b32 = reinterpret_cast<const uint32_t *>(embd + (tok * (size_t)(d / 256) + sb) * 144);
    uint32_t dd = b32[0], s0 = b32[1], s1 = b32[2], s2 = b32[3];
    int j = i >> 5, l = i & 31, sc, mn;
    k4_scale_min(s0, s1, s2, j, sc, mn);
    uint32_t byte = reinterpret_cast<const uint8_t *>(b32 + 4)[(j >> 1) * 32 + l];
    uint32_t q = (j & 1) ? (byte >> 4) : (byte & 0xFu);
    float dv = half_bits_to_f32(dd & 0xffffu), dmin = half_bits_to_f32(dd >> 16);
    x[sb * 256 + i] = __fsub_rn(__fmul_rn(__fmul_rn(dv, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
}

// ---------------------------------------------------------------- RMS norm + Q8_K (engine_qwen2.rs:453-465, 287-300)
// One CTA.  12 threads walk the 12 slices serially, the partials are added in worker order.
__global__ void __launch_bounds__(256) qw_norm_quant_kernel(const float *__restrict__ x, const float *__restrict__ w, float eps, int d,
                                                            float *__restrict__ xn_out, int8_t *__restrict__ q, float *__restrict__ s,
                                                            int32_t *__restrict__ bsum) {
    extern __shared__ __align__(16) float xs_sh[];
    __shared__ float part[QW_NT];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    pdl_trigger();
    for (int i = tid; i < d / 4; i += 256) reinterpret_cast<float4 *>(xs_sh)[i] = reinterpret_cast<const float4 *>(x)[i];
    __syncthreads();
    if (tid < QW_NT) {
        int a, b;
        qw_slice(tid, d, a, b);
        float ps = 0.0f;
#pragma unroll 8
        for (int i = a; i < b; i++) { float v = xs_sh[i]; ps = __fadd_rn(ps, __fmul_rn(v, v)); }
        part[tid] = ps;
    }
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int k = 0; k < QW_NT; k++) tot = __fadd_rn(tot, part[k]);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)d), eps)));
    for (int sb = warp; sb < d / 256; sb += 8) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int idx = sb * 256 + lane * 8 + i;
            v[i] = __fmul_rn(__fmul_rn(xs_sh[idx], inv), w[idx]);
        }
        if (xn_out) {
            float4 *dst = reinterpret_cast<float4 *>(xn_out + sb * 256 + lane * 8);
            dst[0] = make_float4(v[0], v[1], v[2], v[3]);
            dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
        warp_quant_q8k(v, lane, q + sb * 256, s + sb, bsum + sb * 8);
    }
}

// Q8_K quantisation of n floats (one warp per superblock), chainable like the other kernels
__global__ void __launch_bounds__(256) qw_quant_kernel(const float *__restrict__ x, int nsb, int8_t *__restrict__ q, float *__restrict__ s,
                                                       int32_t *__restrict__ bsum) {
    const int sb = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    pdl_trigger();
    if (sb >= nsb) return;
    const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)sb * 256 + lane * 8);
    float4 a = src[0], b = src[1];
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    warp_quant_q8k(v, lane, q + (size_t)sb * 256, s + sb, bsum + sb * 8);
}

// ---------------------------------------------------------------- K-quant matvec over up to three stacked matrices
struct KStack {
    KMatDev m[3];
    float *y[3];
    int n;
};
enum { KEPI_PLAIN = 0, KEPI_RESID = 1 };

template <int EPI>
__global__ void __launch_bounds__(256) qw_matvec_kernel(KStack a, const int8_t *__restrict__ xq, const float *__restrict__ ys,
                                                        const int32_t *__restrict__ bsum) {
    int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    pdl_wait();
    pdl_trigger();
    int mi = 0;
    while (mi < a.n && row >= a.m[mi].rows) { row -= a.m[mi].rows; mi++; }
    if (mi >= a.n) return;
    float v = kq_row_dot(a.m[mi], (size_t)row, xq, ys, bsum, lane);
    if (lane == 0) {
        float *y = a.y[mi] + row;
        *y = EPI == KEPI_RESID ? __fadd_rn(*y, v) : v;
    }
}

// ---------------------------------------------------------------- QK norm + RoPE + cache append (engine_qwen2.rs:353-362, 466-482)
// One CTA of head_dim threads per q or k head.  Cache layout [kv head][position][head_dim].
__global__ void __launch_bounds__(QW_HD) qw_qknorm_rope_kernel(float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                                               const float *__restrict__ q_norm, const float *__restrict__ k_norm,
                                                               const float *__restrict__ rope, float eps, int nh, int nkv,
                                                               const DevState *__restrict__ state, int pos_val, float *__restrict__ kc,
                                                               float *__restrict__ vc) {
    __shared__ float raw[QW_HD], nv[QW_HD];
    const int h = blockIdx.x, tid = threadIdx.x, hd = QW_HD, half = QW_HD / 2;
    const int pos = state ? (int)state->pos : pos_val;
    const bool is_q = h < nh;
    const float *src = is_q ? q + h * hd : k + (h - nh) * hd;
    const float wv = (is_q ? q_norm : k_norm)[tid];
    const float co = rope[((size_t)pos * half + (tid % half)) * 2], si = rope[((size_t)pos * half + (tid % half)) * 2 + 1];
    pdl_wait();
    pdl_trigger();
    raw[tid] = src[tid];
    __syncthreads();
    float ms = 0.0f;
#pragma unroll 16
    for (int i = 0; i < hd; i++) { float t = raw[i]; ms = __fadd_rn(ms, __fmul_rn(t, t)); }
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ms, (float)hd), eps)));
    nv[tid] = __fmul_rn(__fmul_rn(raw[tid], inv), wv);
    __syncthreads();
    const float aa = nv[tid % half], bb = nv[half + tid % half];
    const float out = tid < half ? __fsub_rn(__fmul_rn(aa, co), __fmul_rn(bb, si)) : __fadd_rn(__fmul_rn(bb, co), __fmul_rn(aa, si));
    if (is_q) q[h * hd + tid] = out;
    else {
        const int hh = h - nh;
        const size_t o = ((size_t)hh * BRRR_MAXSEQ + pos) * hd + tid;
        kc[o] = out;
        vc[o] = v[hh * hd + tid];
    }
}

// ---------------------------------------------------------------- attention (engine_qwen2.rs:365-389)
// One CTA per q head.  score(t): 8 chains (chain c covers dims c, c+8, ..., fused), combined as
// (c + c+4) per lane then (l0+l1)+(l2+l3), times 1/sqrt(128); softmax with the running maximum
// taken over all keys; denominator and the 128 output sums serial over t.
__global__ void __launch_bounds__(256) qw_attn_kernel(const float *__restrict__ q, const float *__restrict__ kc, const float *__restrict__ vc,
                                                      int nh, int nkv, const DevState *__restrict__ state, int pos_val, float *__restrict__ ao) {
    __shared__ float sc[BRRR_MAXSEQ];
    __shared__ float qs[QW_HD];
    __shared__ float red[8];
    __shared__ float den_sh;
    const int h = blockIdx.x, tid = threadIdx.x, kvh = h / (nh / nkv);
    const int pos = state ? (int)state->pos : pos_val;
    const int n = pos + 1;
    const float *kbase = kc + (size_t)kvh * BRRR_MAXSEQ * QW_HD, *vbase = vc + (size_t)kvh * BRRR_MAXSEQ * QW_HD;
    pdl_wait();
    pdl_trigger();
    if (tid < QW_HD) qs[tid] = q[h * QW_HD + tid];
    __syncthreads();
    {
        const int g = tid >> 3, c = tid & 7;
        float qr[16];
#pragma unroll
        for (int i = 0; i < 16; i++) qr[i] = qs[8 * i + c];
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)QW_HD));
        for (int t0 = 0; t0 < n; t0 += 32) {
            const int t = t0 + g;
            const bool live = t < n;
            float s = 0.0f;
            if (live) {
                const float *kp = kbase + (size_t)t * QW_HD + c;
#pragma unroll
                for (int i = 0; i < 16; i++) s = __fmaf_rn(kp[8 * i], qr[i], s);
            }
            s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 4));
            s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
            s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 2));
            if (live && c == 0) sc[t] = __fmul_rn(s, scale);
        }
    }
    __syncthreads();
    float mx = -3.402823466e+38f;
    for (int t = tid; t < n; t += 256) mx = fmaxf(mx, sc[t]);
    mx = warp_max(mx);
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < 8; w++) mx = fmaxf(mx, red[w]);
    for (int t = tid; t < n; t += 256) sc[t] = brrr_expf_dev(__fsub_rn(sc[t], mx));
    __syncthreads();
    float acc = 0.0f;
    if (tid == QW_HD) {
        float den = 0.0f;
#pragma unroll 8
        for (int t = 0; t < n; t++) den = __fadd_rn(den, sc[t]);
        den_sh = den;
    } else if (tid < QW_HD) {
        const float *vp = vbase + tid;
#pragma unroll 8
        for (int t = 0; t < n; t++) acc = __fmaf_rn(vp[(size_t)t * QW_HD], sc[t], acc);
    }
    __syncthreads();
    if (tid < QW_HD) ao[h * QW_HD + tid] = __fmul_rn(acc, __fdiv_rn(1.0f, den_sh));
}

// ---------------------------------------------------------------- experts
// gate/up rows of the selected experts and SiLU-GLU (engine_qwen2.rs:419-426): one warp per (slot, row).
__global__ void __launch_bounds__(256) qw_gate_up_kernel(KMatDev gate, KMatDev up, const int32_t *__restrict__ top, int topk, int ff,
                                                         const int8_t *__restrict__ xq, const float *__restrict__ ys,
                                                         const int32_t *__restrict__ bsum, float *__restrict__ hbuf) {
    const int it = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    pdl_trigger();
    if (it >= topk * ff) return;
    const int ei = it / ff, r = it % ff;
    const size_t gr = (size_t)top[ei] * ff + r;
    const float g = kq_row_dot(gate, gr, xq, ys, bsum, lane), u = kq_row_dot(up, gr, xq, ys, bsum, lane);
    if (lane == 0) hbuf[it] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, brrr_expf_dev(-g))), u);
}

// down-projection and weighted accumulate in slot order (engine_qwen2.rs:432-441): one warp per output row.
__global__ void __launch_bounds__(256) qw_down_kernel(KMatDev down, const int32_t *__restrict__ top, const float *__restrict__ wts, int topk,
                                                      int d, int ff, const int8_t *__restrict__ hq, const float *__restrict__ hs,
                                                      const int32_t *__restrict__ hsum, float *__restrict__ x) {
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    pdl_trigger();
    if (r >= d) return;
    float acc = x[r];
    for (int ei = 0; ei < topk; ei++) {
        float dot = kq_row_dot(down, (size_t)top[ei] * d + r, hq + (size_t)ei * ff, hs + ei * (ff / 256), hsum + ei * (ff / 32), lane);
        acc = __fadd_rn(acc, __fmul_rn(wts[ei], dot));
    }
    if (lane == 0) x[r] = acc;
}

// ---------------------------------------------------------------- vocabulary projection + argmax (engine_qwen2.rs:436-448)
__global__ void __launch_bounds__(256) qw_head_kernel(KMatDev head, const int8_t *__restrict__ xq, const float *__restrict__ ys,
                                                      const int32_t *__restrict__ bsum, float *__restrict__ logits, DevState *state) {
    __shared__ unsigned long long wbest[8];
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    pdl_trigger();
    unsigned long long key = 0ull;
    if (row < head.rows) {
        float v = kq_row_dot(head, (size_t)row, xq, ys, bsum, lane);
        if (lane == 0) logits[row] = v;
        key = ((unsigned long long)float_orderable(v) << 32) | (0xFFFFFFFFu - (uint32_t)row);
    }
    if (lane == 0) wbest[warp] = key;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long best = wbest[0];
#pragma unroll
        for (int w = 1; w < 8; w++) best = wbest[w] > best ? wbest[w] : best;
        if (best) atomicMax(&state->best, best);
    }
}

}  // namespace

// ---------------------------------------------------------------- launchers
cudaError_t launch_qw_embed(const uint8_t *embd, int d, const DevState *state, float *x, bool pdl, cudaStream_t st) {
    return launch_k(qw_embed_kernel, dim3(d / 256), dim3(256), 0, st, pdl, embd, d, state, x);
}

cudaError_t launch_qw_norm_quant(const float *x, const float *w, float eps, int d, float *xn, int8_t *q, float *s, int32_t *bsum,
                                 bool pdl, cudaStream_t st) {
    return launch_k(qw_norm_quant_kernel, dim3(1), dim3(256), (size_t)d * 4, st, pdl, x, w, eps, d, xn, q, s, bsum);
}

cudaError_t launch_qw_quant(const float *x, int n, int8_t *q, float *s, int32_t *bsum, bool pdl, cudaStream_t st) {
    int nsb = n / 256;
    return launch_k(qw_quant_kernel, dim3((nsb + 7) / 8), dim3(256), 0, st, pdl, x, nsb, q, s, bsum);
}

cudaError_t launch_qw_matvec(const KMatDev *mats, float *const *ys_out, int n, bool resid, const int8_t *xq, const float *ys,
                             const int32_t *bsum, bool pdl, cudaStream_t st) {
    KStack a{};
    int rows = 0;
    a.n = n;
    for (int i = 0; i < n; i++) { a.m[i] = mats[i]; a.y[i] = ys_out[i]; rows += mats[i].rows; }
    dim3 grid((rows + 7) / 8), block(256);
    return resid ? launch_k(qw_matvec_kernel<KEPI_RESID>, grid, block, 0, st, pdl, a, xq, ys, bsum)
                 : launch_k(qw_matvec_kernel<KEPI_PLAIN>, grid, block, 0, st, pdl, a, xq, ys, bsum);
}

cudaError_t launch_qw_qknorm_rope(float *q, const float *k, const float *v, const float *q_norm, const float *k_norm, const float *rope,
                                  float eps, int nh, int nkv, const DevState *state, int pos_val, float *kc, float *vc, bool pdl,
                                  cudaStream_t st) {
    return launch_k(qw_qknorm_rope_kernel, dim3(nh + nkv), dim3(QW_HD), 0, st, pdl, q, k, v, q_norm, k_norm, rope, eps, nh, nkv, state,
                    pos_val, kc, vc);
}

cudaError_t launch_qw_attn(const float *q, const float *kc, const float *vc, int nh, int nkv, const DevState *state, int pos_val, float *ao,
                           bool pdl, cudaStream_t st) {
    return launch_k(qw_attn_kernel, dim3(nh), dim3(256), 0, st, pdl, q, kc, vc, nh, nkv, state, pos_val, ao);
}

cudaError_t launch_qw_gate_up(const KMatDev &gate, const KMatDev &up, const int32_t *top, int topk, int ff, const int8_t *xq, const float *ys,
                              const int32_t *bsum, float *hbuf, bool pdl, cudaStream_t st) {
    return launch_k(qw_gate_up_kernel, dim3((topk * ff + 7) / 8), dim3(256), 0, st, pdl, gate, up, top, topk, ff, xq, ys, bsum, hbuf);
}

cudaError_t launch_qw_down(const KMatDev &down, const int32_t *top, const float *wts, int topk, int d, int ff, const int8_t *hq, const float *hs,
                           const int32_t *hsum, float *x, bool pdl, cudaStream_t st) {
    return launch_k(qw_down_kernel, dim3((d + 7) / 8), dim3(256), 0, st, pdl, down, top, wts, topk, d, ff, hq, hs, hsum, x);
}

cudaError_t launch_qw_head(const KMatDev &head, const int8_t *xq, const float *ys, const int32_t *bsum, float *logits, DevState *state, bool pdl,
                           cudaStream_t st) {
    return launch_k(qw_head_kernel, dim3((head.rows + 7) / 8), dim3(256), 0, st, pdl, head, xq, ys, bsum, logits, state);
}

}  // namespace brrr
