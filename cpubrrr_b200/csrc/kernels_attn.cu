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

// ---------------------------------------------------------------- prompt tiles: rows of one sequence share their keys
// attn_decode_kernel per (head, row) streams the row's whole window from L2 for every one of the 64 heads: a tile of
// R rows at position p costs 64 R p key reads.  Here one CTA serves one KV head and a block of consecutive rows of one
// sequence: 32 (query head, row) pairs = group x (32 / group) rows share every K and V tile it brings into shared
// memory.  Same operations in the same order per pair as attn_decode_kernel (the row's own key comes from the cache,
// where kv_append_rows_kernel wrote the same bits):
//   score(t)  one thread: the 16 four-term chains, then the pairwise combine of the shuffle butterfly (xor 4, 8, 1, 2)
//   pass 1    scores of every key -> the pair's maximum;  pass 2  scores again -> p = exp(s - mx) into shared memory,
//             then, tile by tile in ascending key order, the serial denominator (one thread per pair) and the serial
//             p.V sums (one thread per (dim, 8 pairs)).  Keys outside a pair's range carry p = +0: x + 0 = x exactly
//             (no accumulator is ever -0: the sums start at +0 and round to nearest), so they need no branch.
// Scores are computed twice instead of being kept: 32 pairs x 4096 keys would not fit shared memory.
constexpr int AR_THREADS = 256;
constexpr int AR_TILE = 128;
constexpr int AR_PAIRS = 32;
constexpr size_t AR_TILE_BYTES = (size_t)AR_TILE * HD * sizeof(float);
constexpr size_t AR_SMEM = 4 * AR_TILE_BYTES + (size_t)AR_TILE * AR_PAIRS * 4 + (size_t)AR_PAIRS * HD * 4;

struct AttnRowsArgs {
    const float *qkv;        // [rows][ldq]: q | k | v of every row, bias added, not rotated
    const float *kc, *vc;    // [sequence][nkv][MAXSEQ][64]
    const float *rope, *sinks;
    int nh, nkv, window, rows, ldq;
    const int *row_pos, *row_seq;
    size_t seq_stride;
    float *ao;
    int8_t *aq;
    float *as;
    DevState *err_state;
};

// one score: q in registers, the key's 64 floats at kp (shared memory, the same address in every lane)
__device__ __forceinline__ float ar_score(const float (&q)[HD], const float *kp) {
    float a[16];
#pragma unroll
    for (int c4 = 0; c4 < 4; c4++) {
        const float4 k0 = *reinterpret_cast<const float4 *>(kp + 4 * c4), k1 = *reinterpret_cast<const float4 *>(kp + 16 + 4 * c4);
        const float4 k2 = *reinterpret_cast<const float4 *>(kp + 32 + 4 * c4), k3 = *reinterpret_cast<const float4 *>(kp + 48 + 4 * c4);
        const float kk0[4] = {k0.x, k0.y, k0.z, k0.w}, kk1[4] = {k1.x, k1.y, k1.z, k1.w}, kk2[4] = {k2.x, k2.y, k2.z, k2.w}, kk3[4] = {k3.x, k3.y, k3.z, k3.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int c = 4 * c4 + i;
            float v = __fmaf_rn(kk0[i], q[c], 0.0f);
            v = __fmaf_rn(kk1[i], q[16 + c], v);
            v = __fmaf_rn(kk2[i], q[32 + c], v);
            a[c] = __fmaf_rn(kk3[i], q[48 + c], v);
        }
    }
    // butterfly xor 4, 8, 1, 2 of the 16-thread group, as one thread
    const float b0 = __fadd_rn(a[0], a[4]), b1 = __fadd_rn(a[1], a[5]), b2 = __fadd_rn(a[2], a[6]), b3 = __fadd_rn(a[3], a[7]);
    const float b8 = __fadd_rn(a[8], a[12]), b9 = __fadd_rn(a[9], a[13]), b10 = __fadd_rn(a[10], a[14]), b11 = __fadd_rn(a[11], a[15]);
    const float c0 = __fadd_rn(b0, b8), c1 = __fadd_rn(b1, b9), c2 = __fadd_rn(b2, b10), c3 = __fadd_rn(b3, b11);
    return __fmul_rn(__fadd_rn(__fadd_rn(c0, c1), __fadd_rn(c2, c3)), 0.125f);
}

__global__ void __launch_bounds__(AR_THREADS) attn_rows_kernel(AttnRowsArgs a) {
    extern __shared__ __align__(128) unsigned char smraw[];
    float *ktile = reinterpret_cast<float *>(smraw);                                    // [2][128][64]
    float *vtile = reinterpret_cast<float *>(smraw + 2 * AR_TILE_BYTES);                // [2][128][64]
    float *psm = reinterpret_cast<float *>(smraw + 4 * AR_TILE_BYTES);                  // [128 keys][32 pairs]
    float *qsm = psm + AR_TILE * AR_PAIRS;                                              // [32 pairs][64]
    __shared__ __align__(8) uint64_t kbar[2], vbar[2];
    __shared__ float red[AR_THREADS / 32][AR_PAIRS];
    __shared__ float mx_sm[AR_PAIRS], den_sm[AR_PAIRS];
    __shared__ int pos_sm[AR_PAIRS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = a.nh / a.nkv, rb = AR_PAIRS / group;        // rows per CTA
    const int kvh = blockIdx.x, r0 = blockIdx.y * rb;
    const int nrows = min(rb, a.rows - r0);
    uint32_t *err = a.err_state ? &a.err_state->err : nullptr;
    Waiter waiter(err);
    if (tid == 0) {
        mbar_init(&kbar[0], 1); mbar_init(&kbar[1], 1); mbar_init(&vbar[0], 1); mbar_init(&vbar[1], 1);
        mbar_fence_init();
    }
    pdl_wait();          // q/k/v projection and the cache append of every row are done
    pdl_trigger();
    waiter.poison_if_failed();
    // ---- the pairs: pair = row-in-block * group + head-in-group
    const int pr = lane;                                           // this thread's pair in the score phases
    const int pr_row = pr / group, pr_h = kvh * group + pr % group;
    const bool pr_live = pr_row < nrows;
    if (tid < AR_PAIRS) pos_sm[tid] = (tid / group) < nrows ? a.row_pos[r0 + tid / group] : -1;
    // RoPE of q (NeoX halves), 1024 rotations over 256 threads
    for (int idx = tid; idx < AR_PAIRS * 32; idx += AR_THREADS) {
        const int p2 = idx >> 5, i = idx & 31, rr = p2 / group;
        if (rr < nrows) {
            const int pos = a.row_pos[r0 + rr];
            const float *src = a.qkv + (size_t)(r0 + rr) * a.ldq + (size_t)(kvh * group + p2 % group) * HD;
            const float c = a.rope[((size_t)pos * 32 + i) * 2], sn = a.rope[((size_t)pos * 32 + i) * 2 + 1];
            const float x0 = src[i], x1 = src[32 + i];
            qsm[p2 * HD + i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
            qsm[p2 * HD + 32 + i] = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, sn));
        } else { qsm[p2 * HD + i] = 0.0f; qsm[p2 * HD + 32 + i] = 0.0f; }
    }
    __syncthreads();
    float q[HD];
#pragma unroll
    for (int i = 0; i < HD; i++) q[i] = qsm[pr * HD + i];
    const int my_pos = pos_sm[pr];
    const int my_start = a.window > 0 ? max(my_pos - (a.window - 1), 0) : 0;
    // key range of the block: from the first row's window start to the last row's position
    const int pos_first = pos_sm[0], pos_last = pos_sm[(nrows - 1) * group];
    const int t_lo = a.window > 0 ? max(pos_first - (a.window - 1), 0) : 0;
    const int nkeys = pos_last - t_lo + 1, ntiles = (nkeys + AR_TILE - 1) / AR_TILE;
    const size_t seq_off = (size_t)a.row_seq[r0] * a.seq_stride;
    const float *kbase = a.kc + seq_off + ((size_t)kvh * BRRR_MAXSEQ + t_lo) * HD;
    const float *vbase = a.vc + seq_off + ((size_t)kvh * BRRR_MAXSEQ + t_lo) * HD;
    int k_issued = 0, v_issued = 0, k_used = 0, v_used = 0;       // tiles issued / consumed so far (buffer = count & 1, parity = count >> 1 & 1)
    auto issue_k = [&](int t) {       // thread 0
        const int buf = k_issued & 1, cnt = min(AR_TILE, nkeys - t * AR_TILE);
        mbar_expect_tx(&kbar[buf], (uint32_t)cnt * HD * 4);
        bulk_g2s(ktile + (size_t)buf * AR_TILE * HD, kbase + (size_t)t * AR_TILE * HD, (uint32_t)cnt * HD * 4, &kbar[buf]);
    };
    auto issue_v = [&](int t) {
        const int buf = v_issued & 1, cnt = min(AR_TILE, nkeys - t * AR_TILE);
        mbar_expect_tx(&vbar[buf], (uint32_t)cnt * HD * 4);
        bulk_g2s(vtile + (size_t)buf * AR_TILE * HD, vbase + (size_t)t * AR_TILE * HD, (uint32_t)cnt * HD * 4, &vbar[buf]);
    };

    // ---- pass 1: the maximum of every pair's scores
    float mx = -3.4028234663852886e38f;
    if (tid == 0) issue_k(0);
    k_issued++;
    for (int t = 0; t < ntiles; t++) {
        if (t + 1 < ntiles) { if (tid == 0) issue_k(t + 1); k_issued++; }        // the other buffer: free since the barrier that ended tile t - 1
        const int buf = k_used & 1;
        waiter.wait(&kbar[buf], (uint32_t)(k_used >> 1) & 1u);
        k_used++;
        const float *kt = ktile + (size_t)buf * AR_TILE * HD;
        const int cnt = min(AR_TILE, nkeys - t * AR_TILE), tb = t_lo + t * AR_TILE;
        for (int kk = warp; kk < cnt; kk += AR_THREADS / 32) {
            const float sc = ar_score(q, kt + kk * HD);
            const int key = tb + kk;
            if (pr_live && key >= my_start && key <= my_pos) mx = fmaxf(mx, sc);
        }
        __syncthreads();              // everyone is done with this buffer
        if (tid == 0) fence_proxy_async();
    }
    red[warp][lane] = mx;
    __syncthreads();
    if (tid < AR_PAIRS) {
        float m = a.sinks[kvh * group + tid % group];
#pragma unroll
        for (int w = 0; w < AR_THREADS / 32; w++) m = fmaxf(m, red[w][tid]);
        mx_sm[tid] = m;
        den_sm[tid] = brrr_expf_dev(__fsub_rn(a.sinks[kvh * group + tid % group], m));      // the sink's term opens the denominator
    }
    __syncthreads();
    mx = mx_sm[pr];

    // ---- pass 2: probabilities tile by tile; denominator and p.V sums in ascending key order
    const int u = tid & 63, grp = tid >> 6;                        // this thread in the p.V phase: dim u of pairs grp * 8 .. + 7
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] = 0.0f;
    float den = tid < AR_PAIRS ? den_sm[tid] : 0.0f;
    if (tid == 0) { issue_k(0); issue_v(0); }
    k_issued++; v_issued++;
    for (int t = 0; t < ntiles; t++) {
        if (t + 1 < ntiles) { if (tid == 0) { issue_k(t + 1); issue_v(t + 1); } k_issued++; v_issued++; }
        const int kb = k_used & 1, vb = v_used & 1;
        waiter.wait(&kbar[kb], (uint32_t)(k_used >> 1) & 1u);
        k_used++;
        const float *kt = ktile + (size_t)kb * AR_TILE * HD;
        const int cnt = min(AR_TILE, nkeys - t * AR_TILE), tb = t_lo + t * AR_TILE;
        for (int kk = warp; kk < cnt; kk += AR_THREADS / 32) {
            const float sc = ar_score(q, kt + kk * HD);
            const int key = tb + kk;
            const bool valid = pr_live && key >= my_start && key <= my_pos;
            psm[kk * AR_PAIRS + pr] = valid ? brrr_expf_dev(__fsub_rn(sc, mx)) : 0.0f;
        }
        __syncthreads();
        if (tid < AR_PAIRS) {
#pragma unroll 8
            for (int kk = 0; kk < cnt; kk++) den = __fadd_rn(den, psm[kk * AR_PAIRS + tid]);
        }
        waiter.wait(&vbar[vb], (uint32_t)(v_used >> 1) & 1u);
        v_used++;
        const float *vt = vtile + (size_t)vb * AR_TILE * HD + u;
        const float *pt = psm + grp * 8;
#pragma unroll 4
        for (int kk = 0; kk < cnt; kk++) {
            const float v = vt[kk * HD];
            const float4 p0 = *reinterpret_cast<const float4 *>(pt + kk * AR_PAIRS), p1 = *reinterpret_cast<const float4 *>(pt + kk * AR_PAIRS + 4);
            acc[0] = __fmaf_rn(v, p0.x, acc[0]); acc[1] = __fmaf_rn(v, p0.y, acc[1]); acc[2] = __fmaf_rn(v, p0.z, acc[2]); acc[3] = __fmaf_rn(v, p0.w, acc[3]);
            acc[4] = __fmaf_rn(v, p1.x, acc[4]); acc[5] = __fmaf_rn(v, p1.y, acc[5]); acc[6] = __fmaf_rn(v, p1.z, acc[6]); acc[7] = __fmaf_rn(v, p1.w, acc[7]);
        }
        __syncthreads();              // the tile's buffers and the probabilities are free
        if (tid == 0) fence_proxy_async();
    }
    if (tid < AR_PAIRS) den_sm[tid] = den;
    __syncthreads();
    // ---- outputs: o = acc / den, and the Q8 image of every pair's two 32-blocks (a warp = one 32-block of a pair)
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int p2 = grp * 8 + j, rr = p2 / group, h = kvh * group + p2 % group;
        if (rr < nrows) {             // uniform over the warp
            const float inv = __fdiv_rn(1.0f, den_sm[p2]);
            const float o = __fmul_rn(acc[j], inv);
            const size_t row = (size_t)(r0 + rr);
            a.ao[row * a.nh * HD + h * HD + u] = o;
            warp_quant_block(o, lane, a.aq + row * a.nh * HD + h * HD + (u >> 5) * 32, a.as + row * a.nh * 2 + h * 2 + (u >> 5));
        }
    }
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

// Attention for token rows of ONE sequence with ascending positions (a prompt tile): rows share the K / V tiles.
// Needs the rows' keys in the cache already (launch_kv_append_rows) and nh / nkv a power of two <= 32.
cudaError_t launch_attn_rows(const float *qkv, int ldq, const float *kc, const float *vc, size_t seq_stride, const float *rope, const float *sinks,
                             int nh, int nkv, int window, const int *row_pos, const int *row_seq, int rows, float *ao, int8_t *aq, float *as,
                             DevState *err_state, bool pdl, cudaStream_t st) {
    const int group = nkv > 0 ? nh / nkv : 0;
    if (group < 1 || group > 32 || (group & (group - 1)) || nh % nkv || rows < 1) return cudaErrorInvalidValue;
    AttnRowsArgs a{qkv, kc, vc, rope, sinks, nh, nkv, window, rows, ldq, row_pos, row_seq, seq_stride, ao, aq, as, err_state};
    static unsigned long long configured = 0;      // one bit per device
    cudaError_t e = smem_optin(attn_rows_kernel, (int)AR_SMEM, configured);
    if (e != cudaSuccess) return e;
    const int rb = AR_PAIRS / group;
    return launch_k(attn_rows_kernel, dim3(nkv, (rows + rb - 1) / rb), dim3(AR_THREADS), AR_SMEM, st, pdl, a);
}

}  // namespace brrr
