// Q8 weight matrices: load-time quantisation from bf16 and the streaming row . Q8-activation GEMV
// (qkv projection, output projection, vocabulary projection).
//
// Float order of one row (fixed): 8 chains = 2 block parities x 4 lanes.  Chain (p, j) walks the
// blocks b = p, p+2, ... accumulating fma(float(t_j(b)), ws[b]*xs[b], acc) where t_j(b) is the
// exact int32 dot of bytes 4j..4j+3 of both 16-byte halves of the block.  The row result is
// hsum4(acc_even + acc_odd).  One thread owns one chain, so the order never depends on the grid.
//
// Data movement: a CTA (128 threads = 16 rows x 8 chains) owns a run of consecutive 16-row unit
// rows, i.e. one contiguous byte range of the matrix.  Thread 0 streams it into a shared-memory
// ring with bulk asynchronous copies (one mbarrier per stage); the copies are issued before the
// kernel waits on its predecessor (programmatic dependent launch), so weight traffic overlaps
// the previous kernel's tail.  Compute threads read quants and scales from shared memory.
#include "brrr_kernels.h"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"

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
    uint8_t *unit = m.data + q8_unit_off(row >> 4, pair, np);
    int rl = row & 15;
    unit[rl * 64 + p * 32 + j * 8 + byte] = (uint8_t)(int8_t)brrr_q8_round(v, sc);
    if (lane == 0) reinterpret_cast<float *>(unit + Q8_UNIT_SCALES)[rl * 2 + p] = sc;
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
    const uint8_t *unit = m.data + q8_unit_off(r >> 4, pair, np);
    int rl = r & 15;
    q[(size_t)r * m.cols + b * 32 + lane] = (int8_t)unit[rl * 64 + p * 32 + j * 8 + byte];
    if (lane == 0) s[(size_t)r * nb + b] = reinterpret_cast<const float *>(unit + Q8_UNIT_SCALES)[rl * 2 + p];
}

void launch_q8_export(Q8Dev m, int8_t *q, float *s, cudaStream_t st) {
    size_t warps = (size_t)m.rows * (m.cols / 32);
    q8_export_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(m, q, s);
}

// N consecutive block pairs of one chain, from units resident in shared memory: all operands are
// fetched and all integer dots formed first, then the N fused multiply-adds run in order.
template <int N>
__device__ __forceinline__ float q8_pairs(const unsigned char *unit, int rl, int c8, int p, const int2 *xp8, const float *xsc2, float acc) {
    int2 w[N], xv[N];
    float s[N], xs[N];
#pragma unroll
    for (int i = 0; i < N; i++) {
        const unsigned char *u = unit + (size_t)i * Q8_UNIT;
        w[i] = *reinterpret_cast<const int2 *>(u + rl * 64 + c8 * 8);
        s[i] = *reinterpret_cast<const float *>(u + Q8_UNIT_SCALES + rl * 8 + p * 4);
        xv[i] = xp8[i * 8];
        xs[i] = xsc2[i * 2];
    }
    float tf[N], sv[N];
#pragma unroll
    for (int i = 0; i < N; i++) {
        tf[i] = (float)__dp4a(w[i].y, xv[i].y, __dp4a(w[i].x, xv[i].x, 0));
        sv[i] = __fmul_rn(s[i], xs[i]);
    }
#pragma unroll
    for (int i = 0; i < N; i++) acc = __fmaf_rn(tf[i], sv[i], acc);
    return acc;
}

// cnt block pairs of one chain from a ring stage
__device__ __forceinline__ float q8_chunk(const unsigned char *base, int cnt, int rl, int c8, int p, const int2 *xp8, const float *xsc2, float acc) {
    int i = 0;
#ifndef Q8_UNROLL
#define Q8_UNROLL 8
#endif
#if Q8_UNROLL == 8
    for (; i + 8 <= cnt; i += 8) acc = q8_pairs<8>(base + (size_t)i * Q8_UNIT, rl, c8, p, xp8 + i * 8, xsc2 + i * 2, acc);
    if (i + 4 <= cnt) { acc = q8_pairs<4>(base + (size_t)i * Q8_UNIT, rl, c8, p, xp8 + i * 8, xsc2 + i * 2, acc); i += 4; }
    if (i + 2 <= cnt) { acc = q8_pairs<2>(base + (size_t)i * Q8_UNIT, rl, c8, p, xp8 + i * 8, xsc2 + i * 2, acc); i += 2; }
    if (i < cnt) acc = q8_pairs<1>(base + (size_t)i * Q8_UNIT, rl, c8, p, xp8 + i * 8, xsc2 + i * 2, acc);
#else
    for (; i + Q8_UNROLL <= cnt; i += Q8_UNROLL) acc = q8_pairs<Q8_UNROLL>(base + (size_t)i * Q8_UNIT, rl, c8, p, xp8 + i * 8, xsc2 + i * 2, acc);
    for (; i < cnt; i++) acc = q8_pairs<1>(base + (size_t)i * Q8_UNIT, rl, c8, p, xp8 + i * 8, xsc2 + i * 2, acc);
#endif
    return acc;
}

// ---------------------------------------------------------------- streaming GEMV
struct Q8Args {
    Q8Dev m;
    const float *x_f32;     // NORM: residual stream (RMSNorm + quantise in the prologue)
    const float *norm_w;
    float eps;
    const int8_t *xq;       // !NORM: already quantised activation
    const float *xs;
    const float *bias;
    float *y;
    DevState *state;
    int ch;                 // pairs per chunk
    int stages;             // ring depth
    // optional: K/V cache of the attention kernel that follows ([nkv][MAXSEQ][64] each); the window
    // it will read is requested into L2 ahead of time (it was last touched a whole step ago)
    const float *pf_k, *pf_v;
    int pf_nkv, pf_window;
};

constexpr int Q8_THREADS = 128;

// Ask for bytes [p, p + n) to be brought into L2 (n a multiple of 16); no completion is awaited.
__device__ __forceinline__ void l2_prefetch(const void *p, uint32_t n) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(n) : "memory");
}

template <int EPI, bool NORM>
__global__ void __launch_bounds__(Q8_THREADS) q8_stream_kernel(Q8Args a) {
    extern __shared__ __align__(128) unsigned char smraw[];
    const int nb = a.m.cols / 32, np = a.m.cols / 64;
    const int tid = threadIdx.x;
    const size_t stage_bytes = (size_t)a.ch * Q8_UNIT;
    unsigned char *ring = smraw;
    float *xf = reinterpret_cast<float *>(smraw + stage_bytes * a.stages);   // NORM only: cols floats (16-byte aligned)
    int2 *xp = reinterpret_cast<int2 *>(xf + (NORM ? a.m.cols : 0));
    float *xsc = reinterpret_cast<float *>(xp + nb * 4);
    uint64_t *bars = reinterpret_cast<uint64_t *>(xsc + nb + (nb & 1));
    __shared__ float inv_sh;
    __shared__ unsigned long long wbest[Q8_THREADS / 32];
    uint32_t *err = a.state ? &a.state->err : nullptr;
    Waiter waiter(err);

    // unit rows [u0, u1) of this CTA, balanced over the grid
    const int urows = q8_urows(a.m.rows);
    const int u0 = (int)((long long)urows * blockIdx.x / gridDim.x);
    const int u1 = (int)((long long)urows * (blockIdx.x + 1) / gridDim.x);
    const int cpr = (np + a.ch - 1) / a.ch;                          // chunks per unit row
    const int nchunks = (u1 - u0) * cpr;

    auto issue = [&](int c) {                                        // one thread per chunk
        int u = u0 + c / cpr, k = c % cpr;
        int cnt = min(a.ch, np - k * a.ch);
        int slot = c % a.stages;
        mbar_expect_tx(&bars[slot], (uint32_t)cnt * Q8_UNIT);
        bulk_g2s(ring + stage_bytes * slot, a.m.data + q8_unit_off(u, k * a.ch, np), (uint32_t)cnt * Q8_UNIT, &bars[slot]);
    };

    const int sb = (NORM || EPI == Q8_EPI_BIAS) ? 32 : 64;      // timeline slots of this kernel flavour (q/k/v, o-proj)
    (void)sb;
    BRRR_STAMP(a.state, sb);
    BRRR_GT_START(a.state, (NORM || EPI == Q8_EPI_BIAS) ? 232 : 234);
    if (tid == 0) {
        for (int s = 0; s < a.stages; s++) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    __syncthreads();
    // one lane per stage: the copies' address translations overlap instead of queueing behind one thread
    if (tid < min(a.stages, nchunks)) issue(tid);
    // static operands (norm weights, bias) and the residual written several kernels back are
    // fetched now, while the predecessor is still running
    const int rl = tid >> 3, c8 = tid & 7, p = c8 >> 2;
    float4 wreg[6];
    if (NORM) norm_prefetch<6>(a.norm_w, a.m.cols, wreg, tid, Q8_THREADS);
    float bias_pre = 0.0f, resid_pre = 0.0f;
    const bool one_row = (u1 - u0) == 1;
    if (one_row && c8 == 0 && u0 * 16 + rl < a.m.rows) {
        if (EPI == Q8_EPI_BIAS || EPI == Q8_EPI_RESID_BIAS) bias_pre = a.bias[u0 * 16 + rl];
        if (EPI == Q8_EPI_RESID_BIAS) resid_pre = a.y[u0 * 16 + rl];
    }
    BRRR_STAMP(a.state, sb + 1);
    pdl_wait();          // predecessor's outputs (activation, residual) are now visible
    BRRR_STAMP(a.state, sb + 2);
    BRRR_GT_GO(a.state, sb + 30);
    pdl_trigger();
    waiter.poison_if_failed();

    // ---- activation: normalise + quantise, or stage the given Q8 vector
    if (NORM) {
        block_norm_quant<NQ_Q8, 6>(a.x_f32, a.norm_w, wreg, a.eps, a.m.cols, xf, xp, xsc, &inv_sh, tid, Q8_THREADS);
    } else {
        // every load before the first store to shared memory: a store in between would order the
        // loads behind it (possible aliasing), and each is a round trip to L2 on the critical path
        const int nidx = nb * 4;
        float sv[2];
#pragma unroll
        for (int k = 0; k < 2; k++) sv[k] = tid + k * Q8_THREADS < nb ? a.xs[tid + k * Q8_THREADS] : 0.0f;
        for (int i0 = tid; i0 < nidx; i0 += 8 * Q8_THREADS) {
            int2 v[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int idx = i0 + k * Q8_THREADS;
                if (idx < nidx) {
                    const int *xw = reinterpret_cast<const int *>(a.xq + (idx >> 2) * 32);
                    v[k] = make_int2(xw[idx & 3], xw[4 + (idx & 3)]);
                }
            }
#pragma unroll
            for (int k = 0; k < 8; k++) if (i0 + k * Q8_THREADS < nidx) xp[i0 + k * Q8_THREADS] = v[k];
        }
#pragma unroll
        for (int k = 0; k < 2; k++) if (tid + k * Q8_THREADS < nb) xsc[tid + k * Q8_THREADS] = sv[k];
        for (int b = tid + 2 * Q8_THREADS; b < nb; b += Q8_THREADS) xsc[b] = a.xs[b];
    }
    __syncthreads();

    BRRR_STAMP(a.state, sb + 3);
    float acc = 0.0f;
    unsigned long long best = 0ull;
    for (int c = 0; c < nchunks; c++) {
        if (c < 12) BRRR_STAMP(a.state, sb + 8 + c);
        const int u = u0 + c / cpr, k = c % cpr;
        const int cnt = min(a.ch, np - k * a.ch);
        const int slot = c % a.stages;
        waiter.wait(&bars[slot], (uint32_t)(c / a.stages) & 1u);
        if (c < 12) BRRR_STAMP(a.state, sb + 20 + c);
        const unsigned char *base = ring + stage_bytes * slot;
        const int pair0 = k * a.ch;
        acc = q8_chunk(base, cnt, rl, c8, p, xp + (size_t)pair0 * 8 + c8, xsc + pair0 * 2 + p, acc);
        if (k == cpr - 1) {
            BRRR_STAMP(a.state, sb + 4);
            // row finished: acc_even + acc_odd per lane, then (l0+l1)+(l2+l3)
            float r = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
            r = brrr_hsum4(r);
            const int row = u * 16 + rl;
            if (c8 == 0 && row < a.m.rows) {
                if (EPI == Q8_EPI_PLAIN) a.y[row] = r;
                else if (EPI == Q8_EPI_BIAS) a.y[row] = __fadd_rn(r, one_row ? bias_pre : a.bias[row]);
                else if (EPI == Q8_EPI_RESID_BIAS)                                                               // x += dot + bias
                    a.y[row] = __fadd_rn(one_row ? resid_pre : a.y[row], __fadd_rn(r, one_row ? bias_pre : a.bias[row]));
                else {
                    a.y[row] = r;
                    unsigned long long key = ((unsigned long long)float_orderable(r) << 32) | (0xFFFFFFFFu - (uint32_t)row);
                    best = key > best ? key : best;
                }
            }
            acc = 0.0f;
        }
        if (c + a.stages < nchunks) {
            __syncthreads();                       // everyone is done with this slot
            if (tid == 0) { fence_proxy_async(); issue(c + a.stages); }
        }
    }
    BRRR_STAMP(a.state, sb + 5);
    BRRR_GT_END(a.state, sb + 31);
    if (EPI == Q8_EPI_HEAD) {
        // running argmax: first strict maximum = lowest index among equal values
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if ((tid & 31) == 0) wbest[tid >> 5] = best;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < Q8_THREADS / 32; w++) best = wbest[w] > best ? wbest[w] : best;
            if (best) atomicMax(&a.state->best, best);
        }
    }
}

// ---------------------------------------------------------------- direct-load GEMV (vocabulary head)
// For a matrix far larger than what the SMs can hold in flight, staging through shared memory
// only adds traffic: 32 rows per CTA, 8 chains per row, weights read straight from global memory
// (a warp's step is one contiguous 256-byte read of a unit), thousands of CTAs in flight.
template <int EPI>
__global__ void __launch_bounds__(256) q8_direct_kernel(Q8Dev m, const int8_t *__restrict__ xq, const float *__restrict__ xs,
                                                        const float *__restrict__ bias, float *__restrict__ y, DevState *state) {
    extern __shared__ __align__(128) unsigned char smraw[];
    const int nb = m.cols / 32, np = m.cols / 64;
    int2 *xp = reinterpret_cast<int2 *>(smraw);
    float *xsc = reinterpret_cast<float *>(smraw + (size_t)nb * 4 * sizeof(int2));
    __shared__ unsigned long long wbest[8];
    pdl_wait();
    pdl_trigger();
    for (int idx = threadIdx.x; idx < nb * 4; idx += 256) {
        int b = idx >> 2, j = idx & 3;
        const int *xw = reinterpret_cast<const int *>(xq + b * 32);
        xp[idx] = make_int2(xw[j], xw[4 + j]);
    }
    for (int b = threadIdx.x; b < nb; b += 256) xsc[b] = xs[b];
    __syncthreads();
    const int row = blockIdx.x * 32 + (threadIdx.x >> 3);
    const int c8 = threadIdx.x & 7, p = c8 >> 2;
    const bool live = row < q8_urows(m.rows) * 16;            // padding rows exist in storage (zeros)
    float acc = 0.0f;
    if (live) {
        const uint8_t *u0 = m.data + q8_unit_off(row >> 4, 0, np);
        const int2 *wp = reinterpret_cast<const int2 *>(u0 + (row & 15) * 64 + c8 * 8);
        const float *sp = reinterpret_cast<const float *>(u0 + Q8_UNIT_SCALES + (row & 15) * 8 + p * 4);
#pragma unroll 8
        for (int i = 0; i < np; i++) {
            int2 w = __ldg(wp + (size_t)i * (Q8_UNIT / 8));
            float s = __ldg(sp + (size_t)i * (Q8_UNIT / 4));
            int2 xv = xp[i * 8 + c8];
            int t = __dp4a(w.y, xv.y, __dp4a(w.x, xv.x, 0));
            acc = __fmaf_rn((float)t, __fmul_rn(s, xsc[i * 2 + p]), acc);
        }
    }
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));   // acc_even + acc_odd, per lane
    acc = brrr_hsum4(acc);
    const bool out = live && c8 == 0 && row < m.rows;
    if (EPI == Q8_EPI_HEAD) {
        unsigned long long key = 0ull;
        if (out) {
            y[row] = acc;
            key = ((unsigned long long)float_orderable(acc) << 32) | (0xFFFFFFFFu - (uint32_t)row);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
            key = other > key ? other : key;
        }
        if ((threadIdx.x & 31) == 0) wbest[threadIdx.x >> 5] = key;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < 8; w++) key = wbest[w] > key ? wbest[w] : key;
            if (key) atomicMax(&state->best, key);
        }
    } else if (out) {
        if (EPI == Q8_EPI_PLAIN) y[row] = acc;
        else if (EPI == Q8_EPI_BIAS) y[row] = __fadd_rn(acc, bias[row]);
        else y[row] = __fadd_rn(y[row], __fadd_rn(acc, bias[row]));
    }
}

// ---------------------------------------------------------------- register-resident GEMV (q/k/v, o-proj)
// For the layer projections one CTA owns one unit row (16 rows) and the whole grid is resident at
// once, so every thread can fetch ALL the weights of its chain (NP block pairs: 8 weight bytes and one
// scale each) straight into registers before the dependency wait, while the kernel before it is
// still running.  After the wait only the activation goes through shared memory: no ring, no
// barrier per chunk, a third of the shared-memory reads of the ring kernel.  Same chain order.
template <int EPI, int NP>
__global__ void __launch_bounds__(Q8_THREADS) q8_reg_kernel(Q8Args a) {
    __shared__ __align__(16) int2 xp[NP * 8];
    __shared__ float xsc[NP * 2];
    const int tid = threadIdx.x, rl = tid >> 3, c8 = tid & 7, p = c8 >> 2;
    const int u = blockIdx.x, row = u * 16 + rl;
    const uint8_t *unit0 = a.m.data + q8_unit_off(u, 0, NP);
    const int2 *wp = reinterpret_cast<const int2 *>(unit0 + rl * 64 + c8 * 8);
    const float *sp = reinterpret_cast<const float *>(unit0 + Q8_UNIT_SCALES + rl * 8 + p * 4);
    int2 w[NP];
    float s[NP];
#pragma unroll
    for (int i = 0; i < NP; i++) {
        w[i] = __ldg(wp + (size_t)i * (Q8_UNIT / 8));
        s[i] = __ldg(sp + (size_t)i * (Q8_UNIT / 4));
    }
    float bias_pre = 0.0f, resid_pre = 0.0f;
    if (c8 == 0 && row < a.m.rows) {
        if (EPI == Q8_EPI_BIAS || EPI == Q8_EPI_RESID_BIAS) bias_pre = a.bias[row];
        if (EPI == Q8_EPI_RESID_BIAS) resid_pre = a.y[row];          // written several kernels back
    }
#ifndef BRRR_NO_KV_PREFETCH
    if (a.pf_k && tid == 0 && u < 2 * a.pf_nkv && a.state) {
        // CTA 2h / 2h+1: the K / V window of KV head h that the attention kernel after this one reads
        // (positions start .. pos-1; the position is an input of the step, written long before)
        const int pos = (int)a.state->pos, start = a.pf_window > 0 ? max(pos - (a.pf_window - 1), 0) : 0;
        const float *base = ((u & 1) ? a.pf_v : a.pf_k) + ((size_t)(u >> 1) * BRRR_MAXSEQ + start) * 64;
        for (int k = 0; k < pos - start; k += 128) l2_prefetch(base + (size_t)k * 64, (uint32_t)min(128, pos - start - k) * 256u);
    }
#endif
    BRRR_GT_START(a.state, EPI == Q8_EPI_BIAS ? 232 : 234);
    pdl_wait();          // the activation is now visible
    BRRR_GT_GO(a.state, (EPI == Q8_EPI_BIAS ? 32 : 64) + 30);
    pdl_trigger();
    {
        // every global load before the first shared-memory store (a store in between would order the loads behind it)
        constexpr int NIDX = NP * 8, PASSES = (NIDX + Q8_THREADS - 1) / Q8_THREADS;
        int2 v[PASSES];
#pragma unroll
        for (int k = 0; k < PASSES; k++) {
            const int idx = tid + k * Q8_THREADS;
            if (idx < NIDX) {
                const int *xw = reinterpret_cast<const int *>(a.xq + (idx >> 2) * 32);
                v[k] = make_int2(xw[idx & 3], xw[4 + (idx & 3)]);
            }
        }
        const float sv = tid < NP * 2 ? a.xs[tid] : 0.0f;
#pragma unroll
        for (int k = 0; k < PASSES; k++) if (tid + k * Q8_THREADS < NIDX) xp[tid + k * Q8_THREADS] = v[k];
        if (tid < NP * 2) xsc[tid] = sv;
    }
    __syncthreads();
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < NP; i++) {
        const int2 xv = xp[i * 8 + c8];
        const int t = __dp4a(w[i].y, xv.y, __dp4a(w[i].x, xv.x, 0));
        acc = __fmaf_rn((float)t, __fmul_rn(s[i], xsc[i * 2 + p]), acc);
    }
    float r = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));      // acc_even + acc_odd per lane, then (l0+l1)+(l2+l3)
    r = brrr_hsum4(r);
    if (c8 == 0 && row < a.m.rows) {
        if (EPI == Q8_EPI_PLAIN) a.y[row] = r;
        else if (EPI == Q8_EPI_BIAS) a.y[row] = __fadd_rn(r, bias_pre);
        else a.y[row] = __fadd_rn(resid_pre, __fadd_rn(r, bias_pre));     // x += dot + bias
    }
    BRRR_GT_END(a.state, (EPI == Q8_EPI_BIAS ? 32 : 64) + 31);
}

template <int NP>
static cudaError_t q8_reg_launch(const Q8Args &a, int epi, unsigned grid, bool pdl, cudaStream_t st) {
    switch (epi) {
    case Q8_EPI_PLAIN: return launch_k(q8_reg_kernel<Q8_EPI_PLAIN, NP>, dim3(grid), dim3(Q8_THREADS), 0, st, pdl, a);
    case Q8_EPI_BIAS: return launch_k(q8_reg_kernel<Q8_EPI_BIAS, NP>, dim3(grid), dim3(Q8_THREADS), 0, st, pdl, a);
    case Q8_EPI_RESID_BIAS: return launch_k(q8_reg_kernel<Q8_EPI_RESID_BIAS, NP>, dim3(grid), dim3(Q8_THREADS), 0, st, pdl, a);
    }
    return cudaErrorInvalidValue;
}

// ---------------------------------------------------------------- vocabulary head: persistent ring
// The head is one long contiguous stream, so it runs as persistent CTAs (two per SM), each owning a
// run of consecutive unit rows: a producer thread keeps a ring of chunks (ch units, about 17 KB, one
// bulk copy each) in flight; the four consumer warps (16 rows x 8 chains) walk the chunks in order
// and hand each stage back through an mbarrier, so the loop has no block-wide barrier.  Every
// barrier has one waiting side that consumes in order (a waiter is never more than one phase
// behind).  Same chain order as every other Q8 row dot.
constexpr int QH_THREADS = 128 + 32;

struct QHeadArgs {
    Q8Dev m;
    const int8_t *xq;
    const float *xs;
    float *y;
    DevState *state;
    int ch;                 // pairs per chunk
    int stages;             // ring depth
};

__global__ void __launch_bounds__(QH_THREADS) q8_head_ring_kernel(QHeadArgs a) {
    extern __shared__ __align__(128) unsigned char smraw[];
    const int nb = a.m.cols / 32, np = a.m.cols / 64;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const size_t stage_bytes = (size_t)a.ch * Q8_UNIT;
    unsigned char *ring = smraw;
    int2 *xp = reinterpret_cast<int2 *>(smraw + stage_bytes * a.stages);
    float *xsc = reinterpret_cast<float *>(xp + nb * 4);
    uint64_t *full = reinterpret_cast<uint64_t *>(xsc + nb + (nb & 1));
    uint64_t *empty = full + a.stages;
    __shared__ unsigned long long wbest[4];
    uint32_t *err = a.state ? &a.state->err : nullptr;
    Waiter waiter(err);
    const int urows = q8_urows(a.m.rows);
    const int u0 = (int)((long long)urows * blockIdx.x / gridDim.x);
    const int u1 = (int)((long long)urows * (blockIdx.x + 1) / gridDim.x);
    const int cpr = (np + a.ch - 1) / a.ch;                          // chunks per unit row
    const int nchunks = (u1 - u0) * cpr;
    if (tid == 0) {
        for (int s = 0; s < a.stages; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 4); }
        mbar_fence_init();
    }
    __syncthreads();
    auto issue = [&](int c) {
        const int u = u0 + c / cpr, k = c % cpr, slot = c % a.stages;
        const uint32_t bytes = (uint32_t)min(a.ch, np - k * a.ch) * Q8_UNIT;
        mbar_expect_tx(&full[slot], bytes);
        bulk_g2s(ring + stage_bytes * slot, a.m.data + q8_unit_off(u, k * a.ch, np), bytes, &full[slot]);
    };
    // the weights do not depend on the step: the first ring goes out before the dependency wait
    const bool producer = warp == 4;
    if (producer && lane < min(a.stages, nchunks)) issue(lane);
    pdl_wait();
    pdl_trigger();
    waiter.poison_if_failed();
    if (producer) {
        if (lane == 0) {
            for (int c = a.stages; c < nchunks; c++) {
                waiter.wait_relaxed(&empty[c % a.stages], (uint32_t)(c / a.stages - 1) & 1u);
                fence_proxy_async();
                issue(c);
            }
        }
        return;
    }
    const int nidx = nb * 4;
    for (int idx = tid; idx < nidx; idx += 128) {
        const int *xw = reinterpret_cast<const int *>(a.xq + (idx >> 2) * 32);
        xp[idx] = make_int2(xw[idx & 3], xw[4 + (idx & 3)]);
    }
    for (int b = tid; b < nb; b += 128) xsc[b] = a.xs[b];
    asm volatile("bar.sync 1, 128;" ::: "memory");                   // the consumer warps only
    const int rl = tid >> 3, c8 = tid & 7, p = c8 >> 2;
    unsigned long long best = 0ull;
    float acc = 0.0f;
    for (int c = 0; c < nchunks; c++) {
        const int k = c % cpr, slot = c % a.stages, pair0 = k * a.ch;
        waiter.wait(&full[slot], (uint32_t)(c / a.stages) & 1u);
        acc = q8_chunk(ring + stage_bytes * slot, min(a.ch, np - pair0), rl, c8, p, xp + (size_t)pair0 * 8 + c8, xsc + pair0 * 2 + p, acc);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);             // this warp has read its four rows of the stage
        if (k == cpr - 1) {
            float r = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
            r = brrr_hsum4(r);
            const int row = (u0 + c / cpr) * 16 + rl;
            if (c8 == 0 && row < a.m.rows) {
                a.y[row] = r;
                const unsigned long long key = ((unsigned long long)float_orderable(r) << 32) | (0xFFFFFFFFu - (uint32_t)row);
                best = key > best ? key : best;
            }
            acc = 0.0f;
        }
    }
    // running argmax: first strict maximum = lowest index among equal values
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if (lane == 0) wbest[warp] = best;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (tid == 0) {
        for (int w = 1; w < 4; w++) best = wbest[w] > best ? wbest[w] : best;
        if (best) atomicMax(&a.state->best, best);
    }
}

cudaError_t launch_q8_direct(Q8Dev m, const int8_t *xq, const float *xs, const float *bias, float *y, int epi, DevState *state, bool pdl, cudaStream_t st) {
    const int nb = m.cols / 32;
    size_t smem = (size_t)nb * 4 * sizeof(int2) + (size_t)nb * sizeof(float);
    dim3 grid((q8_urows(m.rows) * 16 + 31) / 32), block(256);
    switch (epi) {
    case Q8_EPI_PLAIN: return launch_k(q8_direct_kernel<Q8_EPI_PLAIN>, grid, block, smem, st, pdl, m, xq, xs, bias, y, state);
    case Q8_EPI_BIAS: return launch_k(q8_direct_kernel<Q8_EPI_BIAS>, grid, block, smem, st, pdl, m, xq, xs, bias, y, state);
    case Q8_EPI_RESID_BIAS: return launch_k(q8_direct_kernel<Q8_EPI_RESID_BIAS>, grid, block, smem, st, pdl, m, xq, xs, bias, y, state);
    case Q8_EPI_HEAD: return launch_k(q8_direct_kernel<Q8_EPI_HEAD>, grid, block, smem, st, pdl, m, xq, xs, bias, y, state);
    }
    return cudaErrorInvalidValue;
}

// chunk size: bulk copies of 16-23 KB move fastest and every chunk costs one barrier wait, so
// prefer a divisor of np between 14 and 20 pairs (no ragged tail), else 16
static int pick_chunk(int np) {
    for (int c = 16; c >= 14; c--) if (np % c == 0) return c;
    for (int c = 17; c <= 20; c++) if (np % c == 0) return c;
    return np < 16 ? np : 16;
}

// The vocabulary projection with its running argmax (logits to y, best (value, lowest row) to
// state->best): two persistent CTAs per SM.
cudaError_t launch_q8_head(Q8Dev m, const int8_t *xq, const float *xs, float *y, DevState *state, bool pdl, cudaStream_t st) {
    const int nb = m.cols / 32, np = m.cols / 64;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        return cudaErrorInvalidDevice;
    QHeadArgs a{m, xq, xs, y, state, pick_chunk(np), 0};
    const size_t stage = (size_t)a.ch * Q8_UNIT, fixed = (size_t)nb * 4 * 8 + (size_t)(nb + (nb & 1)) * 4 + 256;
    a.stages = (int)((100 * 1024 - fixed) / stage);
    if (a.stages > 8) a.stages = 8;
    if (a.stages < 2) return launch_q8_direct(m, xq, xs, nullptr, y, Q8_EPI_HEAD, state, pdl, st);
    const int urows = q8_urows(m.rows);
    const unsigned grid = (unsigned)(urows < 2 * sms ? urows : 2 * sms);
    const size_t smem = stage * a.stages + fixed;
    static unsigned long long configured = 0;      // one bit per device
    cudaError_t e = smem_optin(q8_head_ring_kernel, 100 * 1024, configured);
    if (e != cudaSuccess) return e;
    return launch_k(q8_head_ring_kernel, dim3(grid), dim3(QH_THREADS), smem, st, pdl, a);
}

static size_t q8_smem(const Q8Args &a, bool norm) {
    int nb = a.m.cols / 32;
    size_t s = (size_t)a.ch * Q8_UNIT * a.stages + (size_t)nb * 4 * 8 + (size_t)nb * 4 + (norm ? (size_t)a.m.cols * 4 : 0) + 8 + (size_t)a.stages * 8;
    return s;
}

template <int EPI, bool NORM>
static cudaError_t q8_launch_t(const Q8Args &a, unsigned grid, bool pdl, cudaStream_t st) {
    static unsigned long long configured = 0;      // one bit per device
    size_t smem = q8_smem(a, NORM);
    {
        cudaError_t e = smem_optin(q8_stream_kernel<EPI, NORM>, 200 * 1024, configured);
        if (e != cudaSuccess) return e;
    }
    return launch_k(q8_stream_kernel<EPI, NORM>, dim3(grid), dim3(Q8_THREADS), smem, st, pdl, a);
}

cudaError_t launch_q8_stream(Q8Dev m, const float *x_f32, const float *norm_w, float eps, const int8_t *xq, const float *xs,
                             const float *bias, float *y, int epi, DevState *state, bool pdl, cudaStream_t st,
                             const float *pf_k, const float *pf_v, int pf_nkv, int pf_window) {
    Q8Args a{};
    a.m = m; a.x_f32 = x_f32; a.norm_w = norm_w; a.eps = eps; a.xq = xq; a.xs = xs; a.bias = bias; a.y = y; a.state = state;
    a.pf_k = pf_k; a.pf_v = pf_v; a.pf_nkv = pf_nkv; a.pf_window = pf_window;
    const int np = m.cols / 64, urows = q8_urows(m.rows);
#ifndef BRRR_NO_Q8_REG
    // layer projections of the gpt-oss shapes (d 2880, 64 heads x 64): every weight in registers
    // before the dependency wait; the grid (one CTA per unit row) is resident as a whole
    // (about 160 registers per thread at 45 pairs: three CTAs per SM; about 220 at 64 pairs: two)
    if (!x_f32 && epi != Q8_EPI_HEAD) {
        if (np == 45 && urows <= 148 * 3) return q8_reg_launch<45>(a, epi, (unsigned)urows, pdl, st);
        if (np == 64 && urows <= 148 * 2) return q8_reg_launch<64>(a, epi, (unsigned)urows, pdl, st);
    }
#endif
    a.ch = pick_chunk(np);
    const int cpr = (np + a.ch - 1) / a.ch;
    // Small matrices: one unit row per CTA, whole row resident.  Large ones: a persistent grid.
    unsigned grid = urows <= 148 * 4 ? urows : 148 * 4;
    int per_cta = (urows + grid - 1) / grid * cpr;
    int max_stages = (int)((96 * 1024) / ((size_t)a.ch * Q8_UNIT));
    if (max_stages < 2) max_stages = 2;
    a.stages = per_cta < max_stages ? per_cta : max_stages;
    if (epi == Q8_EPI_HEAD && a.stages > 5) a.stages = 5;
    const bool norm = x_f32 != nullptr;
    switch (epi) {
    case Q8_EPI_PLAIN: return norm ? q8_launch_t<Q8_EPI_PLAIN, true>(a, grid, pdl, st) : q8_launch_t<Q8_EPI_PLAIN, false>(a, grid, pdl, st);
    case Q8_EPI_BIAS: return norm ? q8_launch_t<Q8_EPI_BIAS, true>(a, grid, pdl, st) : q8_launch_t<Q8_EPI_BIAS, false>(a, grid, pdl, st);
    case Q8_EPI_RESID_BIAS: return norm ? q8_launch_t<Q8_EPI_RESID_BIAS, true>(a, grid, pdl, st) : q8_launch_t<Q8_EPI_RESID_BIAS, false>(a, grid, pdl, st);
    case Q8_EPI_HEAD: return norm ? q8_launch_t<Q8_EPI_HEAD, true>(a, grid, pdl, st) : q8_launch_t<Q8_EPI_HEAD, false>(a, grid, pdl, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace brrr
