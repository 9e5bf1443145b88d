// Decode kernels of the qwen3moe engine (src/bin/engine_qwen2.rs:302-451): Q4_K embedding row,
// RMS norm with the reference's 12 partial sums + Q8_K quantisation, K-quant matrix-vector
// products with their epilogues, per-head QK norm + RoPE + cache append, full causal GQA
// attention (head_dim 128), SiLU-GLU experts, weighted down-projection and the vocabulary argmax.
//
// Float order: every sum the reference forms serially is formed serially by one thread here
// (norm partials, head mean square, softmax denominator, probability-weighted values, the
// expert combine); integer sums are exact and split across lanes.
//
// One layer is seven launches chained by programmatic dependent launch:
//   q|k|v matvec -> QK norm + RoPE + cache append -> attention (+ Q8_K of its output) -> o-proj (+ residual)
//   -> router (FFN norm + Q8_K of the normalised token in its prologue) -> gate/up + SiLU-GLU
//   -> down (Q8_K of h in its prologue, weighted accumulate, and - by the last CTA to finish - the
//      next layer's attention norm + Q8_K, or the output norm after the last layer).
// Matrix rows are read in the lane-group form of brrr_kq.cuh (16 bytes per lane and load); kernels
// whose matrices are known before their predecessor ends (q|k|v, o-proj, down) fetch every weight
// byte into registers ahead of the dependency wait.
#include "brrr_kernels.h"
#include "brrr_kq.cuh"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"

namespace brrr {

namespace {

constexpr int QW_HD = 128;
constexpr int QW_HEAD_ROWS = 64;   // vocabulary rows per CTA of the head kernel

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


// ---------------------------------------------------------------- lane-group rows
// A warp owns a row; lane group g = lane / 8 owns superblocks g, g + 4, ... (UPL per lane).
template <int UPL>
__device__ __forceinline__ void qw_row_load(const KMatDev &m, const uint8_t *row, int nsb, int lane, KUnit (&u)[UPL]) {
    const int g = lane >> 3, l8 = lane & 7;
#pragma unroll
    for (int i = 0; i < UPL; i++)
        if (g + 4 * i < nsb) kq_unit_load(m, row, g + 4 * i, l8, u[i]);
}

// Row sum from units in registers and the Q8_K activation in shared memory: superblock terms are
// added in superblock order, one unfused add each (q4k_dot / q6k_dot of the reference); the result
// is valid in every lane.
template <int UPL>
__device__ __forceinline__ float qw_row_sum(int type, const KUnit (&u)[UPL], int nsb, int lane, const int8_t *xq, const float *ys,
                                            const int32_t *bsum) {
    const int g = lane >> 3, l8 = lane & 7;
    const unsigned gmask = 0xFFu << (8 * g);
    float sumf = 0.0f;
#pragma unroll
    for (int i = 0; i < UPL; i++) {
        const int sb = g + 4 * i;
        float term = 0.0f;
        if (sb < nsb) term = kq_unit_term(type, u[i], l8, xq + sb * 256, ys[sb], bsum + sb * 8, gmask);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float t = __shfl_sync(0xffffffffu, term, 8 * k);
            if (4 * i + k < nsb) sumf = __fadd_rn(sumf, t);
        }
    }
    return sumf;
}

// Q8_K activation (n values) from global memory into shared memory: quants, scales, 32-sums.
__device__ __forceinline__ void qw_stage_q8k(const int8_t *q, const float *s, const int32_t *bsum, int n, int8_t *sq, float *ss, int32_t *sb,
                                             int tid, int nthreads) {
    for (int i = tid; i < n / 16; i += nthreads) reinterpret_cast<int4 *>(sq)[i] = reinterpret_cast<const int4 *>(q)[i];
    for (int i = tid; i < n / 256; i += nthreads) ss[i] = s[i];
    for (int i = tid; i < n / 32; i += nthreads) sb[i] = bsum[i];
}

// ---------------------------------------------------------------- matvec over up to three stacked matrices (q|k|v, o-proj)
struct KStack {
    KMatDev m[3];
    float *y[3];
    int n;
    const int8_t *xq;          // Q8_K activation of the previous stage
    const float *ys;
    const int32_t *bsum;
    // optional: K/V cache of the attention kernel that follows ([nkv][MAXSEQ][128] each): positions
    // 0 .. pos-1 are requested into L2 ahead of time (last touched a whole step ago)
    const float *pf_k, *pf_v;
    int pf_nkv;
    const DevState *state;
};
enum { KEPI_PLAIN = 0, KEPI_RESID = 1 };

__device__ __forceinline__ void qw_l2_prefetch(const void *p, uint32_t n) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(n) : "memory");
}

template <int EPI, int UPL>
__global__ void __launch_bounds__(256) qw_matvec_kernel(KStack a) {
    extern __shared__ __align__(16) unsigned char qsm[];
    const int tid = threadIdx.x, lane = tid & 31;
    int row = (blockIdx.x * 256 + tid) >> 5;
    int mi = 0;
    while (mi < a.n && row >= a.m[mi].rows) { row -= a.m[mi].rows; mi++; }
    const bool live = mi < a.n;
    const KMatDev &m = a.m[live ? mi : 0];
    const int K = a.m[0].cols, nsb = K / 256;
    KUnit u[UPL];
    if (live) qw_row_load<UPL>(m, m.p + (size_t)row * m.bpr(), nsb, lane, u);          // static weights: before the wait
    float resid = 0.0f;
    if (EPI == KEPI_RESID && live && lane == 0) resid = a.y[mi][row];                      // written several kernels back
    if (a.pf_k && a.state && tid == 0 && blockIdx.x < 2 * a.pf_nkv) {
        const int pos = (int)a.state->pos;
        const float *base = ((blockIdx.x & 1) ? a.pf_v : a.pf_k) + (size_t)(blockIdx.x >> 1) * BRRR_MAXSEQ * QW_HD;
        for (int k = 0; k < pos; k += 64) qw_l2_prefetch(base + (size_t)k * QW_HD, (uint32_t)min(64, pos - k) * QW_HD * 4u);
    }
    pdl_wait();
    pdl_trigger();
    int8_t *sq = reinterpret_cast<int8_t *>(qsm);
    float *ss = reinterpret_cast<float *>(qsm + K);
    int32_t *sbs = reinterpret_cast<int32_t *>(ss + nsb);
    qw_stage_q8k(a.xq, a.ys, a.bsum, K, sq, ss, sbs, tid, 256);
    __syncthreads();
    if (!live) return;
    const float v = qw_row_sum<UPL>(m.type, u, nsb, lane, sq, ss, sbs);
    if (lane == 0) a.y[mi][row] = EPI == KEPI_RESID ? __fadd_rn(resid, v) : v;
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
// One CTA per pair of q heads (256 threads each).  score(t): 8 chains (chain c covers dims c, c+8,
// ..., fused), combined as (c + c+4) per lane then (l0+l1)+(l2+l3), times 1/sqrt(128); softmax with
// the running maximum taken over all keys; denominator and the 128 output sums serial over t.  The
// two heads' outputs are one 256-value superblock of the o-proj's activation, quantised here
// (Q8_K, engine_qwen2.rs:390).
__global__ void __launch_bounds__(512) qw_attn_kernel(const float *__restrict__ q, const float *__restrict__ kc, const float *__restrict__ vc,
                                                      int nh, int nkv, const DevState *__restrict__ state, int pos_val,
                                                      int8_t *__restrict__ aq, float *__restrict__ as, int32_t *__restrict__ asum) {
    extern __shared__ __align__(16) float asm_[];       // sc[2][MAXSEQ]
    __shared__ float qs[2][QW_HD];
    __shared__ float red[2][8];
    __shared__ float den_sh[2];
    __shared__ __align__(16) float outv[2 * QW_HD];
    const int hh = threadIdx.x >> 8, tid = threadIdx.x & 255;
    const int h = 2 * blockIdx.x + hh, kvh = h / (nh / nkv);
    const int pos = state ? (int)state->pos : pos_val;
    const int n = pos + 1;
    float *sc = asm_ + hh * BRRR_MAXSEQ;
    const float *kbase = kc + (size_t)kvh * BRRR_MAXSEQ * QW_HD, *vbase = vc + (size_t)kvh * BRRR_MAXSEQ * QW_HD;
    auto bar_half = [&]() { asm volatile("bar.sync %0, 256;" ::"r"(1 + hh) : "memory"); };
    pdl_wait();
    pdl_trigger();
    if (tid < QW_HD) qs[hh][tid] = q[h * QW_HD + tid];
    bar_half();
    {
        const int g = tid >> 3, c = tid & 7;
        float qr[16];
#pragma unroll
        for (int i = 0; i < 16; i++) qr[i] = qs[hh][8 * i + c];
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
    bar_half();
    float mx = -3.402823466e+38f;
    for (int t = tid; t < n; t += 256) mx = fmaxf(mx, sc[t]);
    mx = warp_max(mx);
    if ((tid & 31) == 0) red[hh][tid >> 5] = mx;
    bar_half();
    mx = red[hh][0];
#pragma unroll
    for (int w = 1; w < 8; w++) mx = fmaxf(mx, red[hh][w]);
    for (int t = tid; t < n; t += 256) sc[t] = brrr_expf_dev(__fsub_rn(sc[t], mx));
    bar_half();
    float acc = 0.0f;
    if (tid == QW_HD) {
        float den = 0.0f;
#pragma unroll 8
        for (int t = 0; t < n; t++) den = __fadd_rn(den, sc[t]);
        den_sh[hh] = den;
    } else if (tid < QW_HD) {
        const float *vp = vbase + tid;
#pragma unroll 8
        for (int t = 0; t < n; t++) acc = __fmaf_rn(vp[(size_t)t * QW_HD], sc[t], acc);
    }
    bar_half();
    if (tid < QW_HD) outv[hh * QW_HD + tid] = __fmul_rn(acc, __fdiv_rn(1.0f, den_sh[hh]));
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const float4 a0 = reinterpret_cast<const float4 *>(outv)[lane * 2], a1 = reinterpret_cast<const float4 *>(outv)[lane * 2 + 1];
        const float v[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        warp_quant_q8k(v, lane, aq + (size_t)blockIdx.x * 256, as + blockIdx.x, asum + blockIdx.x * 8);
    }
}

// ---------------------------------------------------------------- experts
// gate/up rows of the selected experts and SiLU-GLU (engine_qwen2.rs:419-426): one warp per (slot, row).
template <int UPL>
__global__ void __launch_bounds__(256) qw_gate_up_kernel(KMatDev gate, KMatDev up, const int32_t *__restrict__ top, int topk, int ff,
                                                         const int8_t *__restrict__ xq, const float *__restrict__ ys,
                                                         const int32_t *__restrict__ bsum, float *__restrict__ hbuf) {
    extern __shared__ __align__(16) unsigned char qsm[];
    const int tid = threadIdx.x, lane = tid & 31;
    const int it = (blockIdx.x * 256 + tid) >> 5;
    const int K = gate.cols, nsb = K / 256;
    const bool live = it < topk * ff;
    pdl_wait();          // the routing comes from the kernel before this one
    pdl_trigger();
    KUnit ug[UPL], uu[UPL];
    int ei = 0, r = 0;
    if (live) {
        ei = it / ff; r = it % ff;
        const size_t gr = (size_t)top[ei] * ff + r;
        qw_row_load<UPL>(gate, gate.p + gr * gate.bpr(), nsb, lane, ug);
        qw_row_load<UPL>(up, up.p + gr * up.bpr(), nsb, lane, uu);
    }
    int8_t *sq = reinterpret_cast<int8_t *>(qsm);
    float *ss = reinterpret_cast<float *>(qsm + K);
    int32_t *sbs = reinterpret_cast<int32_t *>(ss + nsb);
    qw_stage_q8k(xq, ys, bsum, K, sq, ss, sbs, tid, 256);
    __syncthreads();
    if (!live) return;
    const float g = qw_row_sum<UPL>(gate.type, ug, nsb, lane, sq, ss, sbs), u = qw_row_sum<UPL>(up.type, uu, nsb, lane, sq, ss, sbs);
    if (lane == 0) hbuf[it] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, brrr_expf_dev(-g))), u);
}

// down-projection and weighted accumulate in slot order (engine_qwen2.rs:432-441): one warp per
// output row, all (slot, superblock) units of the row in registers before the dependency wait (the
// routing is two kernels old by then).  Prologue: Q8_K of h (every CTA quantises all of it: 24 KB
// from L2).  Epilogue: the last CTA to finish normalises and quantises the finished residual for
// the next consumer (next layer's q|k|v, or the vocabulary head).
struct QDownArgs {
    KMatDev down;
    const int32_t *top;
    const float *wts;
    int topk, d, ff;
    const float *hbuf;
    float *x;
    unsigned int *counter;           // arrival counter, zero between launches
    const float *next_norm_w;        // nullable: no norm epilogue
    float eps;
    int8_t *nq; float *ns; int32_t *nsum;
};

template <int NSBF>
__global__ void __launch_bounds__(256) qw_down_kernel(QDownArgs a) {
    extern __shared__ __align__(16) unsigned char qsm[];
    constexpr int UPL = 2 * NSBF;                    // units per lane: up to 8 slots x NSBF superblocks over 4 lane groups
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 3, l8 = lane & 7;
    const int r = blockIdx.x * 8 + warp;
    const int nun = a.topk * NSBF, hn = a.topk * a.ff;
    __shared__ int last_sh;
    __shared__ float part[QW_NT];
    KUnit u[UPL];
    float w[8];
    if (r < a.d) {
#pragma unroll
        for (int i = 0; i < UPL; i++) {
            const int ui = g + 4 * i;
            if (ui < nun) {
                const int ei = ui / NSBF, sb = ui % NSBF;
                kq_unit_load(a.down, a.down.p + ((size_t)a.top[ei] * a.d + r) * a.down.bpr(), sb, l8, u[i]);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 8; k++) w[k] = k < a.topk ? a.wts[k] : 0.0f;
    float acc = r < a.d ? a.x[r] : 0.0f;
    pdl_wait();          // h is complete
    pdl_trigger();
    int8_t *sq = reinterpret_cast<int8_t *>(qsm);
    float *ss = reinterpret_cast<float *>(qsm + hn);
    int32_t *sbs = reinterpret_cast<int32_t *>(ss + hn / 256);
    for (int sb = warp; sb < hn / 256; sb += 8) {
        const float4 *src = reinterpret_cast<const float4 *>(a.hbuf + (size_t)sb * 256 + lane * 8);
        const float4 p0 = src[0], p1 = src[1];
        const float v[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        warp_quant_q8k(v, lane, sq + sb * 256, ss + sb, sbs + sb * 8);
    }
    __syncthreads();
    if (r < a.d) {
        const unsigned gmask = 0xFFu << (8 * g);
        float tv[UPL];
#pragma unroll
        for (int i = 0; i < UPL; i++) {
            const int ui = g + 4 * i;
            tv[i] = 0.0f;
            if (ui < nun) {
                const int ei = ui / NSBF, sb = ui % NSBF, hsb = ei * NSBF + sb;
                tv[i] = kq_unit_term(a.down.type, u[i], l8, sq + hsb * 256, ss[hsb], sbs + hsb * 8, gmask);
            }
        }
        // slot ei: dot = ((0 + t0) + t1) + ...; x += w[ei] * dot, slots in order
        float dot = 0.0f;
#pragma unroll
        for (int ui = 0; ui < 4 * UPL; ui++) {
            const float t = __shfl_sync(0xffffffffu, tv[ui / 4], 8 * (ui % 4));
            if (ui < nun) {
                dot = __fadd_rn(dot, t);
                if (ui % NSBF == NSBF - 1) { acc = __fadd_rn(acc, __fmul_rn(w[ui / NSBF], dot)); dot = 0.0f; }
            }
        }
        if (lane == 0) a.x[r] = acc;
    }
    if (!a.next_norm_w) return;
    // ---- the last CTA to finish: RMS norm (12 slices, engine_qwen2.rs:453-465) + Q8_K of the whole residual
    __threadfence();
    __syncthreads();
    if (tid == 0) last_sh = atomicAdd(a.counter, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!last_sh) return;
    __threadfence();
    float *xs_sh = reinterpret_cast<float *>(qsm);          // d floats (the Q8_K image of h is no longer needed)
    for (int i = tid; i < a.d / 4; i += 256) reinterpret_cast<float4 *>(xs_sh)[i] = __ldcg(reinterpret_cast<const float4 *>(a.x) + i);
    __syncthreads();
    if (tid < QW_NT) {
        int lo, hi;
        qw_slice(tid, a.d, lo, hi);
        float ps = 0.0f;
#pragma unroll 8
        for (int i = lo; i < hi; i++) { const float v = xs_sh[i]; ps = __fadd_rn(ps, __fmul_rn(v, v)); }
        part[tid] = ps;
    }
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int k = 0; k < QW_NT; k++) tot = __fadd_rn(tot, part[k]);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)a.d), a.eps)));
    for (int sb = warp; sb < a.d / 256; sb += 8) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int idx = sb * 256 + lane * 8 + i;
            v[i] = __fmul_rn(__fmul_rn(xs_sh[idx], inv), a.next_norm_w[idx]);
        }
        warp_quant_q8k(v, lane, a.nq + sb * 256, a.ns + sb, a.nsum + sb * 8);
    }
    if (tid == 0) *a.counter = 0u;
}

// ---------------------------------------------------------------- vocabulary projection + argmax (engine_qwen2.rs:436-448)
template <int UPL>
__global__ void __launch_bounds__(256) qw_head_kernel(KMatDev head, const int8_t *__restrict__ xq, const float *__restrict__ ys,
                                                      const int32_t *__restrict__ bsum, float *__restrict__ logits, DevState *state) {
    extern __shared__ __align__(16) unsigned char qsm[];
    __shared__ unsigned long long wbest[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = head.cols, nsb = K / 256;
    int8_t *sq = reinterpret_cast<int8_t *>(qsm);
    float *ss = reinterpret_cast<float *>(qsm + K);
    int32_t *sbs = reinterpret_cast<int32_t *>(ss + nsb);
    // a CTA walks QW_HEAD_ROWS rows, eight at a time, the next eight rows' units in flight while the current ones are summed
    const int row0 = blockIdx.x * QW_HEAD_ROWS;
    KUnit u[UPL], un[UPL];
    int row = row0 + warp;
    if (row < head.rows) qw_row_load<UPL>(head, head.p + (size_t)row * head.bpr(), nsb, lane, u);
    pdl_wait();
    pdl_trigger();
    qw_stage_q8k(xq, ys, bsum, K, sq, ss, sbs, tid, 256);
    __syncthreads();
    unsigned long long best = 0ull;
    for (int i = 0; i < QW_HEAD_ROWS; i += 8) {
        const int nrow = row + 8;
        const bool more = i + 8 < QW_HEAD_ROWS && nrow < head.rows;
        if (more) qw_row_load<UPL>(head, head.p + (size_t)nrow * head.bpr(), nsb, lane, un);
        if (row < head.rows) {
            const float v = qw_row_sum<UPL>(head.type, u, nsb, lane, sq, ss, sbs);
            if (lane == 0) logits[row] = v;
            const unsigned long long key = ((unsigned long long)float_orderable(v) << 32) | (0xFFFFFFFFu - (uint32_t)row);
            best = key > best ? key : best;
        }
        if (more) {
#pragma unroll
            for (int k = 0; k < UPL; k++) u[k] = un[k];
        }
        row = nrow;
    }
    if (lane == 0) wbest[warp] = best;
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int w = 1; w < 8; w++) best = wbest[w] > best ? wbest[w] : best;
        if (best) atomicMax(&state->best, best);
    }
}

// ---------------------------------------------------------------- load-time re-layout of Q6_K rows into aligned planes
__global__ void q6k_planes_kernel(const uint8_t *__restrict__ src, size_t rows, int nsb, uint8_t *__restrict__ dst) {
    const size_t rb = q6k_plane_row_bytes(nsb), total = rows * rb;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / rb;
        const int o = (int)(i % rb);
        const uint8_t *r = src + row * (size_t)nsb * 210;
        uint8_t v = 0;
        if (o < nsb * 128) v = r[(o / 128) * 210 + o % 128];
        else if (o < nsb * 192) { const int k = o - nsb * 128; v = r[(k / 64) * 210 + 128 + k % 64]; }
        else if (o < nsb * 208) { const int k = o - nsb * 192; v = r[(k / 16) * 210 + 192 + k % 16]; }
        else if (o < nsb * 210) { const int k = o - nsb * 208; v = r[(k / 2) * 210 + 208 + k % 2]; }
        dst[i] = v;
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

// units per lane for rows of nsb superblocks: 1, 2 or 4 (nsb <= 16)
static int qw_upl(int nsb) { return nsb <= 4 ? 1 : nsb <= 8 ? 2 : nsb <= 16 ? 4 : 0; }
static size_t qw_act_smem(int K) { return (size_t)K + (size_t)(K / 256) * 4 + (size_t)(K / 32) * 4; }

template <int EPI>
static cudaError_t qw_matvec_launch(const KStack &a, int upl, dim3 grid, size_t smem, bool pdl, cudaStream_t st) {
    switch (upl) {
    case 1: return launch_k(qw_matvec_kernel<EPI, 1>, grid, dim3(256), smem, st, pdl, a);
    case 2: return launch_k(qw_matvec_kernel<EPI, 2>, grid, dim3(256), smem, st, pdl, a);
    case 4: return launch_k(qw_matvec_kernel<EPI, 4>, grid, dim3(256), smem, st, pdl, a);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_qw_matvec(const KMatDev *mats, float *const *ys_out, int n, bool resid, const int8_t *xq, const float *ys,
                             const int32_t *bsum, bool pdl, cudaStream_t st, const float *pf_k, const float *pf_v, int pf_nkv,
                             const DevState *state) {
    KStack a{};
    int rows = 0;
    a.n = n;
    for (int i = 0; i < n; i++) {
        a.m[i] = mats[i]; a.y[i] = ys_out[i]; rows += mats[i].rows;
        if (mats[i].cols != mats[0].cols || (mats[i].type == 14 && !mats[i].planes)) return cudaErrorInvalidValue;
    }
    a.xq = xq; a.ys = ys; a.bsum = bsum; a.pf_k = pf_k; a.pf_v = pf_v; a.pf_nkv = pf_nkv; a.state = state;
    const int K = mats[0].cols, upl = qw_upl(K / 256);
    dim3 grid((rows + 7) / 8);
    return resid ? qw_matvec_launch<KEPI_RESID>(a, upl, grid, qw_act_smem(K), pdl, st) : qw_matvec_launch<KEPI_PLAIN>(a, upl, grid, qw_act_smem(K), pdl, st);
}

cudaError_t launch_qw_qknorm_rope(float *q, const float *k, const float *v, const float *q_norm, const float *k_norm, const float *rope,
                                  float eps, int nh, int nkv, const DevState *state, int pos_val, float *kc, float *vc, bool pdl,
                                  cudaStream_t st) {
    return launch_k(qw_qknorm_rope_kernel, dim3(nh + nkv), dim3(QW_HD), 0, st, pdl, q, k, v, q_norm, k_norm, rope, eps, nh, nkv, state,
                    pos_val, kc, vc);
}

cudaError_t launch_qw_attn(const float *q, const float *kc, const float *vc, int nh, int nkv, const DevState *state, int pos_val, int8_t *aq,
                           float *as, int32_t *asum, bool pdl, cudaStream_t st) {
    if (nh % 2) return cudaErrorInvalidValue;
    static unsigned long long configured = 0;      // one bit per device
    const size_t smem = (size_t)2 * BRRR_MAXSEQ * sizeof(float);
    cudaError_t e = smem_optin(qw_attn_kernel, (int)smem, configured);
    if (e != cudaSuccess) return e;
    return launch_k(qw_attn_kernel, dim3(nh / 2), dim3(512), smem, st, pdl, q, kc, vc, nh, nkv, state, pos_val, aq, as, asum);
}

cudaError_t launch_qw_gate_up(const KMatDev &gate, const KMatDev &up, const int32_t *top, int topk, int ff, const int8_t *xq, const float *ys,
                              const int32_t *bsum, float *hbuf, bool pdl, cudaStream_t st) {
    if (gate.cols != up.cols || (gate.type == 14 && !gate.planes) || (up.type == 14 && !up.planes)) return cudaErrorInvalidValue;
    const int K = gate.cols;
    dim3 grid((topk * ff + 7) / 8);
    switch (qw_upl(K / 256)) {
    case 1: return launch_k(qw_gate_up_kernel<1>, grid, dim3(256), qw_act_smem(K), st, pdl, gate, up, top, topk, ff, xq, ys, bsum, hbuf);
    case 2: return launch_k(qw_gate_up_kernel<2>, grid, dim3(256), qw_act_smem(K), st, pdl, gate, up, top, topk, ff, xq, ys, bsum, hbuf);
    case 4: return launch_k(qw_gate_up_kernel<4>, grid, dim3(256), qw_act_smem(K), st, pdl, gate, up, top, topk, ff, xq, ys, bsum, hbuf);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_qw_down(const KMatDev &down, const int32_t *top, const float *wts, int topk, int d, int ff, const float *hbuf, float *x,
                           unsigned int *counter, const float *next_norm_w, float eps, int8_t *nq, float *ns, int32_t *nsum, bool pdl,
                           cudaStream_t st) {
    if ((down.type == 14 && !down.planes) || ff % 256 || ff > 1024 || topk > 8) return cudaErrorInvalidValue;
    QDownArgs a{down, top, wts, topk, d, ff, hbuf, x, counter, next_norm_w, eps, nq, ns, nsum};
    const size_t act = qw_act_smem(topk * ff), smem = act > (size_t)d * 4 ? act : (size_t)d * 4;
    dim3 grid((d + 7) / 8);
    switch (ff / 256) {
    case 1: return launch_k(qw_down_kernel<1>, grid, dim3(256), smem, st, pdl, a);
    case 2: return launch_k(qw_down_kernel<2>, grid, dim3(256), smem, st, pdl, a);
    case 3: return launch_k(qw_down_kernel<3>, grid, dim3(256), smem, st, pdl, a);
    case 4: return launch_k(qw_down_kernel<4>, grid, dim3(256), smem, st, pdl, a);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_qw_head(const KMatDev &head, const int8_t *xq, const float *ys, const int32_t *bsum, float *logits, DevState *state, bool pdl,
                           cudaStream_t st) {
    if (head.type == 14 && !head.planes) return cudaErrorInvalidValue;
    const int K = head.cols;
    dim3 grid((head.rows + QW_HEAD_ROWS - 1) / QW_HEAD_ROWS);
    switch (qw_upl(K / 256)) {
    case 1: return launch_k(qw_head_kernel<1>, grid, dim3(256), qw_act_smem(K), st, pdl, head, xq, ys, bsum, logits, state);
    case 2: return launch_k(qw_head_kernel<2>, grid, dim3(256), qw_act_smem(K), st, pdl, head, xq, ys, bsum, logits, state);
    case 4: return launch_k(qw_head_kernel<4>, grid, dim3(256), qw_act_smem(K), st, pdl, head, xq, ys, bsum, logits, state);
    }
    return cudaErrorInvalidValue;
}

void launch_q6k_planes(const uint8_t *src, size_t rows, int cols, uint8_t *dst, cudaStream_t st) {
    if (rows) q6k_planes_kernel<<<1184, 256, 0, st>>>(src, rows, cols / 256, dst);
}

}  // namespace brrr
