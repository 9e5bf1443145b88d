// Decode attention for one token: RoPE of q and k, KV-cache append, GQA attention with an
// attention sink and an optional sliding window, and the Q8 quantisation of the output.
//
// One CTA per query head (head_dim = 64).  Fixed float order:
//   score(t): 16 chains (chain c covers dims c, c+16, c+32, c+48, fused), combined
//             ((a0+a1)+(a2+a3)) per lane then (l0+l1)+(l2+l3), times 1/sqrt(64)
//   mx = max(sink, scores); den = exp(sink-mx) + sum_t exp(s_t-mx), t ascending, serial
//   out[u] = (sum_t fma(v[t][u], p_t, .), t ascending, serial) * (1/den)
// The serial sums are one thread each (64 output dims + 1 denominator).
//
// The cache is laid out [kv head][position][64] so the window of one head is one contiguous
// range; it is brought into shared memory in tiles of 128 positions (32 for token rows) by bulk asynchronous copies
// issued before the kernel waits on its predecessor (the cached positions are older than this
// token).  The current position's k and v never come from the cache: every head recomputes them.
#include "brrr_kernels.h"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"

namespace brrr {

constexpr int HD = 64;
constexpr int AT_THREADS = 256;
constexpr int AT_TILE_ONE = 128;                   // positions per tile: one token per launch (one CTA per SM streams its head's window)
constexpr int AT_TILE_ROWS = 32;                   // token rows: many (head, row) CTAs share an SM, so each holds less
constexpr int AT_SLOTS = 2;                        // ring depth per tensor

struct AttnArgs {
    const float *qkv;
    float *kc, *vc;          // [nkv][MAXSEQ][64]
    const float *rope, *sinks;
    int nh, nkv;
    const DevState *state;
    int pos_val, window;
    int pos_off;             // added to the device-side position (token t of a prompt tile: t)
    float *ao;
    int8_t *aq;
    float *as;
    DevState *err_state;
    // token rows (grid.y = rows; nullptr: one token): row t attends at position row_pos[t] of sequence
    // row_seq[t] (caches seq_stride floats apart); its q | k | v are ldq floats after the previous row's,
    // its outputs nh * 64 values after it.  The cached positions may then have been written by the kernel
    // just before this one (earlier rows of the same sequence), so they are fetched after the dependency wait.
    const int *row_pos, *row_seq;
    size_t seq_stride;
    int ldq;
};

#ifndef AT_SCORE_UNROLL
#define AT_SCORE_UNROLL 8
#endif
constexpr int kScoreUnroll = AT_SCORE_UNROLL;      // keys of the score loop in flight per thread group (their shuffle chains overlap)

template <int AT_TILE>
__global__ void __launch_bounds__(AT_THREADS) attn_decode_kernel(AttnArgs a) {
    constexpr size_t AT_TILE_BYTES = (size_t)AT_TILE * HD * sizeof(float);
    extern __shared__ __align__(128) unsigned char smraw[];
    float *ktiles = reinterpret_cast<float *>(smraw);                                   // [AT_SLOTS][128][64]
    float *vtiles = reinterpret_cast<float *>(smraw + AT_TILE_BYTES * AT_SLOTS);
    float *sc = reinterpret_cast<float *>(smraw + AT_TILE_BYTES * AT_SLOTS * 2);         // [MAXSEQ]
    uint64_t *kbar = reinterpret_cast<uint64_t *>(sc + BRRR_MAXSEQ);
    uint64_t *vbar = kbar + AT_SLOTS;
    __shared__ float q[HD], kcur[HD], vcur[HD];
    __shared__ float red[AT_THREADS / 32];
    __shared__ float den_sh;
    const int h = blockIdx.x, tid = threadIdx.x;
    const int group = a.nh / a.nkv, kvh = h / group;
    uint32_t *err = a.err_state ? &a.err_state->err : nullptr;
    Waiter waiter(err);
    const bool rows = a.row_pos != nullptr;
    if (rows) {
        const int t = blockIdx.y;
        a.qkv += (size_t)t * a.ldq;
        a.kc += (size_t)a.row_seq[t] * a.seq_stride;
        a.vc += (size_t)a.row_seq[t] * a.seq_stride;
        a.ao += (size_t)t * a.nh * HD;
        a.aq += (size_t)t * a.nh * HD;
        a.as += (size_t)t * a.nh * 2;
    }

    // The position is an input of this step (written before the graph launch or by the previous
    // step's last kernel), never by the immediate predecessor, so it may be read before the wait.
    const int pos = rows ? a.row_pos[blockIdx.y] : (a.state ? (int)a.state->pos + a.pos_off : a.pos_val);
    const int start = a.window > 0 ? max(pos - (a.window - 1), 0) : 0;
    const int n = pos - start + 1;                  // keys including the current one
    const int ncached = n - 1;                      // keys that come from the cache
    const int ntiles = (ncached + AT_TILE - 1) / AT_TILE;
    const float *kbase = a.kc + ((size_t)kvh * BRRR_MAXSEQ + start) * HD;
    const float *vbase = a.vc + ((size_t)kvh * BRRR_MAXSEQ + start) * HD;

    auto issue = [&](const float *base, float *tiles, uint64_t *bars, int t) {     // thread 0 only
        int slot = t % AT_SLOTS, cnt = min(AT_TILE, ncached - t * AT_TILE);
        mbar_expect_tx(&bars[slot], (uint32_t)cnt * HD * 4);
        bulk_g2s(tiles + (size_t)slot * AT_TILE * HD, base + (size_t)t * AT_TILE * HD, (uint32_t)cnt * HD * 4, &bars[slot]);
    };
    BRRR_STAMP(a.err_state, 160);
    BRRR_GT_START(a.err_state, 233);
    if (tid == 0) {
        for (int s = 0; s < AT_SLOTS; s++) { mbar_init(&kbar[s], 1); mbar_init(&vbar[s], 1); }
        mbar_fence_init();
    }
    __syncwarp();
    // one lane per copy (K and V of the first tiles): their address translations overlap
    if (!rows && tid < 2 * min(AT_SLOTS, ntiles)) {
        if (tid & 1) issue(vbase, vtiles, vbar, tid >> 1);
        else issue(kbase, ktiles, kbar, tid >> 1);
    }
    // static / step-constant operands: the sink and this position's rotation
    const float sink = a.sinks[h];
    float rc = 0.0f, rs = 0.0f;
    if (tid < 64) { rc = a.rope[((size_t)pos * 32 + (tid & 31)) * 2]; rs = a.rope[((size_t)pos * 32 + (tid & 31)) * 2 + 1]; }
    BRRR_STAMP(a.err_state, 161);
    pdl_wait();          // qkv projection done
    BRRR_STAMP(a.err_state, 162);
    BRRR_GT_GO(a.err_state, 190);
    pdl_trigger();
    waiter.poison_if_failed();
    if (rows && tid < 2 * min(AT_SLOTS, ntiles)) {
        if (tid & 1) issue(vbase, vtiles, vbar, tid >> 1);
        else issue(kbase, ktiles, kbar, tid >> 1);
    }

    // ---- RoPE (NeoX halves, table holds cos*mscale / sin*mscale) on q and k; v passes through
    if (tid < 64) {
        const float *src = tid < 32 ? a.qkv + h * HD : a.qkv + (a.nh + kvh) * HD;
        float *dst = tid < 32 ? q : kcur;
        int i = tid & 31;
        const float c = rc, s = rs;
        float x0 = src[i], x1 = src[32 + i];
        dst[i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        dst[32 + i] = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
    } else if (tid < 128) {
        vcur[tid - 64] = a.qkv[(a.nh + a.nkv + kvh) * HD + (tid - 64)];
    }
    __syncthreads();
    // the first head of each KV group appends this position to the cache
    if (!rows && h % group == 0 && tid < 128) {        // (token rows: kv_append_rows_kernel has done it for every row)
        size_t o = ((size_t)kvh * BRRR_MAXSEQ + pos) * HD + (tid & 63);
        if (tid < 64) a.kc[o] = kcur[tid]; else a.vc[o] = vcur[tid - 64];
    }

    // ---- scores: 16 threads per key
    {
        const int g = tid >> 4, c = tid & 15;
        const float q0 = q[c], q1 = q[16 + c], q2 = q[32 + c], q3 = q[48 + c];
        for (int t = 0; t < ntiles; t++) {
            const int slot = t % AT_SLOTS, cnt = min(AT_TILE, ncached - t * AT_TILE);
            waiter.wait(&kbar[slot], (uint32_t)(t / AT_SLOTS) & 1u);
            const float *kt = ktiles + (size_t)slot * AT_TILE * HD;
#pragma unroll kScoreUnroll
            for (int k0 = 0; k0 < cnt; k0 += AT_THREADS / 16) {
                int kk = k0 + g;
                bool live = kk < cnt;
                float s = 0.0f;
                if (live) {
                    const float *kp = kt + kk * HD;
                    s = __fmaf_rn(kp[c], q0, s);
                    s = __fmaf_rn(kp[16 + c], q1, s);
                    s = __fmaf_rn(kp[32 + c], q2, s);
                    s = __fmaf_rn(kp[48 + c], q3, s);
                }
                s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 4));
                s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 8));
                s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
                s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 2));
                if (live && c == 0) sc[t * AT_TILE + kk] = __fmul_rn(s, 0.125f);
            }
            if (t + AT_SLOTS < ntiles) {
                __syncthreads();
                if (tid == 0) { fence_proxy_async(); issue(kbase, ktiles, kbar, t + AT_SLOTS); }
            }
        }
        // the current position, from this CTA's own rotated k
        if (g == 0) {
            float s = 0.0f;
            s = __fmaf_rn(kcur[c], q0, s);
            s = __fmaf_rn(kcur[16 + c], q1, s);
            s = __fmaf_rn(kcur[32 + c], q2, s);
            s = __fmaf_rn(kcur[48 + c], q3, s);
            s = __fadd_rn(s, __shfl_xor_sync(0xffffu, s, 4));
            s = __fadd_rn(s, __shfl_xor_sync(0xffffu, s, 8));
            s = __fadd_rn(s, __shfl_xor_sync(0xffffu, s, 1));
            s = __fadd_rn(s, __shfl_xor_sync(0xffffu, s, 2));
            if (c == 0) sc[ncached] = __fmul_rn(s, 0.125f);
        }
    }
    __syncthreads();

    BRRR_STAMP(a.err_state, 163);
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

    BRRR_STAMP(a.err_state, 164);
    // ---- serial sums: thread u < 64 owns output dim u, thread 64 the denominator
    float acc = 0.0f;
    if (tid == 64) {
        float den = brrr_expf_dev(__fsub_rn(sink, mx));
#pragma unroll 8
        for (int t = 0; t < n; t++) den = __fadd_rn(den, sc[t]);
        den_sh = den;
    }
    for (int t = 0; t < ntiles; t++) {
        const int slot = t % AT_SLOTS, cnt = min(AT_TILE, ncached - t * AT_TILE);
        if (tid < 64) {
            waiter.wait(&vbar[slot], (uint32_t)(t / AT_SLOTS) & 1u);
            const float *vt = vtiles + (size_t)slot * AT_TILE * HD + tid;
            const float *pt = sc + t * AT_TILE;
#pragma unroll 8
            for (int kk = 0; kk < cnt; kk++) acc = __fmaf_rn(vt[kk * HD], pt[kk], acc);
        }
        if (t + AT_SLOTS < ntiles) {
            __syncthreads();
            if (tid == 0) { fence_proxy_async(); issue(vbase, vtiles, vbar, t + AT_SLOTS); }
        }
    }
    if (tid < 64) acc = __fmaf_rn(vcur[tid], sc[ncached], acc);          // t = pos: this token's own v
    __syncthreads();
    if (tid < 64) {
        float inv = __fdiv_rn(1.0f, den_sh);
        float o = __fmul_rn(acc, inv);
        a.ao[h * HD + tid] = o;
        // this head owns Q8 blocks 2h and 2h+1 of the attention output
        warp_quant_block(o, tid & 31, a.aq + h * HD + (tid >> 5) * 32, a.as + h * 2 + (tid >> 5));
    }
    BRRR_STAMP(a.err_state, 165);
    BRRR_GT_END(a.err_state, 191);
}

static size_t attn_smem(int tile) { return (size_t)tile * HD * sizeof(float) * AT_SLOTS * 2 + (size_t)BRRR_MAXSEQ * 4 + AT_SLOTS * 2 * 8; }

cudaError_t launch_attn_decode(const float *qkv, float *kc, float *vc, const float *rope, const float *sinks, int nh, int nkv,
                               const DevState *state, int pos_val, int window, float *ao, int8_t *aq, float *as,
                               DevState *err_state, bool pdl, cudaStream_t st, int pos_off, const int *row_pos, const int *row_seq, size_t seq_stride,
                               int ldq, int rows) {
    AttnArgs a{qkv, kc, vc, rope, sinks, nh, nkv, state, pos_val, window, pos_off, ao, aq, as, err_state, row_pos, row_seq, seq_stride, ldq};
    static unsigned long long configured = 0, configured_rows = 0;      // one bit per device
    if (row_pos) {
        cudaError_t e = smem_optin(attn_decode_kernel<AT_TILE_ROWS>, (int)attn_smem(AT_TILE_ROWS), configured_rows);
        if (e != cudaSuccess) return e;
        return launch_k(attn_decode_kernel<AT_TILE_ROWS>, dim3(nh, rows), dim3(AT_THREADS), attn_smem(AT_TILE_ROWS), st, pdl, a);
    }
    cudaError_t e = smem_optin(attn_decode_kernel<AT_TILE_ONE>, (int)attn_smem(AT_TILE_ONE), configured);
    if (e != cudaSuccess) return e;
    return launch_k(attn_decode_kernel<AT_TILE_ONE>, dim3(nh, 1), dim3(AT_THREADS), attn_smem(AT_TILE_ONE), st, pdl, a);
}

}  // namespace brrr
