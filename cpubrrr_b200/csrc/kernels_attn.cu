// Decode attention for one token: RoPE of q and k, KV-cache append, GQA attention with an
// attention sink and an optional sliding window, and the Q8 quantisation of the output.
//
// One CTA per query head (head_dim = 64).  Fixed float order:
//   score(t): 16 chains (chain c covers dims c, c+16, c+32, c+48, fused), combined
//             ((a0+a1)+(a2+a3)) per lane then (l0+l1)+(l2+l3), times 1/sqrt(64)
//   mx = max(sink, scores); den = exp(sink-mx) + sum_t exp(s_t-mx), t ascending, serial
//   out[u] = (sum_t fma(v[t][u], p_t, .), t ascending, serial) * (1/den)
// The serial sums are one thread each (64 output dims + 1 denominator).
#include "brrr_kernels.h"
#include "brrr_block.cuh"

namespace brrr {

constexpr int HD = 64;
constexpr int AT_THREADS = 256;

__global__ void __launch_bounds__(AT_THREADS) attn_decode_kernel(const float *__restrict__ qkv, float *__restrict__ kc, float *__restrict__ vc,
                                                                 const float *__restrict__ rope, const float *__restrict__ sinks, int nh, int nkv,
                                                                 const DevState *__restrict__ state, int pos_val, int window,
                                                                 float *__restrict__ ao, int8_t *__restrict__ aq, float *__restrict__ as) {
    __shared__ float q[HD], kcur[HD], vcur[HD];
    __shared__ float sc[BRRR_MAXSEQ];
    __shared__ float red[AT_THREADS / 32];
    __shared__ float den_sh;
    const int h = blockIdx.x, tid = threadIdx.x;
    const int group = nh / nkv, kvh = h / group;
    const int pos = state ? (int)state->pos : pos_val;
    const int start = window > 0 ? max(pos - (window - 1), 0) : 0;
    const int n = pos - start + 1;
    const float sink = sinks[h];

    // ---- RoPE (NeoX halves, table holds cos*mscale / sin*mscale) on q and k; v passes through
    if (tid < 64) {
        const float *src = tid < 32 ? qkv + h * HD : qkv + (nh + kvh) * HD;
        float *dst = tid < 32 ? q : kcur;
        int i = tid & 31;
        float c = rope[((size_t)pos * 32 + i) * 2], s = rope[((size_t)pos * 32 + i) * 2 + 1];
        float a = src[i], b = src[32 + i];
        dst[i] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
        dst[32 + i] = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
    } else if (tid < 128) {
        vcur[tid - 64] = qkv[(nh + nkv + kvh) * HD + (tid - 64)];
    }
    __syncthreads();
    // the first head of each KV group appends this position to the cache
    if (h % group == 0 && tid < 128) {
        size_t o = ((size_t)pos * nkv + kvh) * HD + (tid & 63);
        if (tid < 64) kc[o] = kcur[tid]; else vc[o] = vcur[tid - 64];
    }

    // ---- scores: 16 threads per key
    {
        const int g = tid >> 4, c = tid & 15;
        const float q0 = q[c], q1 = q[16 + c], q2 = q[32 + c], q3 = q[48 + c];
        for (int t0 = 0; t0 < n; t0 += AT_THREADS / 16) {
            int t = t0 + g;
            bool live = t < n;
            float a = 0.0f;
            if (live) {
                int tp = start + t;
                const float *kp = tp == pos ? kcur : kc + ((size_t)tp * nkv + kvh) * HD;
                a = __fmaf_rn(kp[c], q0, a);
                a = __fmaf_rn(kp[16 + c], q1, a);
                a = __fmaf_rn(kp[32 + c], q2, a);
                a = __fmaf_rn(kp[48 + c], q3, a);
            }
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 4));
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 8));
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 1));
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 2));
            if (live && c == 0) sc[t] = __fmul_rn(a, 0.125f);
        }
    }
    __syncthreads();

    // ---- max (order-free), then exponentials in place
    float mx = sink;
    for (int t = tid; t < n; t += AT_THREADS) mx = fmaxf(mx, sc[t]);
    mx = warp_max(mx);
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < AT_THREADS / 32; w++) mx = fmaxf(mx, red[w]);
    for (int t = tid; t < n; t += AT_THREADS) sc[t] = brrr_expf_dev(__fsub_rn(sc[t], mx));
    __syncthreads();

    // ---- serial sums: thread u < 64 owns output dim u, thread 64 the denominator
    float acc = 0.0f;
    if (tid < 64) {
        const float *vbase = vc + ((size_t)start * nkv + kvh) * HD + tid;
        const size_t vstride = (size_t)nkv * HD;
#pragma unroll 8
        for (int t = 0; t < n - 1; t++) acc = __fmaf_rn(__ldcg(vbase + (size_t)t * vstride), sc[t], acc);
        acc = __fmaf_rn(vcur[tid], sc[n - 1], acc);          // t = pos: this token's own v
    } else if (tid == 64) {
        float den = brrr_expf_dev(__fsub_rn(sink, mx));
#pragma unroll 8
        for (int t = 0; t < n; t++) den = __fadd_rn(den, sc[t]);
        den_sh = den;
    }
    __syncthreads();
    if (tid < 64) {
        float inv = __fdiv_rn(1.0f, den_sh);
        float o = __fmul_rn(acc, inv);
        ao[h * HD + tid] = o;
        // this head owns Q8 blocks 2h and 2h+1 of the attention output
        warp_quant_block(o, tid & 31, aq + h * HD + (tid >> 5) * 32, as + h * 2 + (tid >> 5));
    }
}

void launch_attn_decode(const float *qkv, float *kc, float *vc, const float *rope, const float *sinks, int nh, int nkv,
                        const DevState *state, int pos_val, int window, float *ao, int8_t *aq, float *as, cudaStream_t st) {
    attn_decode_kernel<<<nh, AT_THREADS, 0, st>>>(qkv, kc, vc, rope, sinks, nh, nkv, state, pos_val, window, ao, aq, as);
}

}  // namespace brrr
