// FFN entry stage: RMSNorm of the residual stream, router GEMV and top-k softmax.
//
// The router logit of expert e is the *serial* f32 sum  acc = b[e]; acc += W[e][j] * xn[j]
// for j ascending, multiply and add rounded separately.  That chain cannot be split without
// changing bits, so one lane owns one expert and walks the whole row: 4 cycles of dependent
// FADD latency per element is the floor of this stage.  The lane is kept fed from a ring of
// shared-memory tiles; each tile is ONE bulk asynchronous copy, because the router matrix is
// re-laid at load time as [32-expert group][tile][32 experts][128 + 4 floats] (the 4-float row
// padding makes a 128-bit read per lane bank-conflict free).  Experts are split 32 per CTA; with
// several CTAs the last one to finish runs the top-k.
#include "brrr_kernels.h"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"
#include "brrr_mxt.cuh"
#include "brrr_kq.cuh"

namespace brrr {

constexpr int RT_STAGES = 5;
constexpr int RT_THREADS = 256;

// ---------------------------------------------------------------- pack: W[ne][d] -> tiled layout
__global__ void router_pack_kernel(const float *__restrict__ W, int ne, int d, float *__restrict__ out) {
    const int ntiles = (d + RT_TJ - 1) / RT_TJ;
    const size_t total = (size_t)((ne + 31) / 32) * ntiles * RT_TILE_FLOATS;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        int jj = (int)(i % RT_STRIDE);
        size_t r = i / RT_STRIDE;
        int el = (int)(r % 32);
        size_t gt = r / 32;
        int t = (int)(gt % ntiles), g = (int)(gt / ntiles);
        int e = g * 32 + el, j = t * RT_TJ + jj;
        out[i] = (jj < RT_TJ && e < ne && j < d) ? W[(size_t)e * d + j] : 0.0f;
    }
}

void launch_router_pack(const float *W, int ne, int d, float *out, cudaStream_t st) {
    router_pack_kernel<<<148, 256, 0, st>>>(W, ne, d, out);
}

// acc += w[j] * x[j] for j = 0..LEN-1, strictly in order, product and sum rounded separately.
// Products are formed 32 at a time from 128-bit shared-memory reads so that only the adds sit
// on the dependent chain.
template <int LEN>
__device__ __forceinline__ float chain_span(const float *__restrict__ w, const float *__restrict__ x, float acc) {
#pragma unroll
    for (int j0 = 0; j0 < LEN; j0 += 32) {
        float p[32];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            float4 a = *reinterpret_cast<const float4 *>(w + j0 + 4 * k);
            float4 b = *reinterpret_cast<const float4 *>(x + j0 + 4 * k);
            p[4 * k] = __fmul_rn(a.x, b.x); p[4 * k + 1] = __fmul_rn(a.y, b.y);
            p[4 * k + 2] = __fmul_rn(a.z, b.z); p[4 * k + 3] = __fmul_rn(a.w, b.w);
        }
#pragma unroll
        for (int k = 0; k < 32; k++) acc = __fadd_rn(acc, p[k]);
    }
    return acc;
}

struct RouterArgs {
    const float *x_in;       // residual stream (norm_w != null) or normalised vector
    const float *norm_w;
    float eps;
    int d;
    const float *Wt;         // tiled router matrix (router_pack_kernel)
    const float *b;
    int ne, topk;
    float *logits;
    int32_t *top;
    float *wts;
    unsigned int *counter;
    DevState *state;
    uint32_t *signal;        // nullable: sequence number of the published routing (see publish_route)
    unsigned long long *pub;
    // qwen3moe: the norm is the 12-slice one, and the first CTA also leaves the Q8_K image of the
    // normalised token (quants, scales per 256, sums per 32) for the gate/up kernel
    int qwen_norm;
    int8_t *q8k_q;
    float *q8k_s;
    int32_t *q8k_bsum;
};

// k rounds of warp arg-max over the logits (lane l holds experts l, l+32, ...): the largest value
// wins, the lower index among equals, which is the order the reference's strict-'>' insertion
// produces.  Then the softmax over the selected k in rank order.  Warp 0 only.
__device__ __forceinline__ void warp_topk(const RouterArgs &a, const float *lg, int lane) {
    float v[8];                                  // up to 256 experts
    const int per = (a.ne + 31) / 32;
    for (int i = 0; i < 8; i++) v[i] = (i < per && lane + 32 * i < a.ne) ? lg[lane + 32 * i] : 0.0f;
    unsigned taken = 0;
    float tv[8];
    int tp[8];
    for (int r = 0; r < a.topk; r++) {
        unsigned long long best = 0ull;
        for (int i = 0; i < per; i++) {
            int e = lane + 32 * i;
            if (e < a.ne && !(taken & (1u << i))) {
                unsigned long long key = ((unsigned long long)float_orderable(v[i]) << 32) | (0xFFFFFFFFu - (uint32_t)e);
                best = key > best ? key : best;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        int e = (int)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
        if ((e & 31) == lane) taken |= 1u << (e >> 5);
        tp[r] = e;
        tv[r] = lg[e];
    }
    if (lane == 0) {
        float ex[8], wsum = 0.0f;
        for (int i = 0; i < a.topk; i++) { ex[i] = brrr_expf_dev(__fsub_rn(tv[i], tv[0])); wsum = __fadd_rn(wsum, ex[i]); }
        for (int i = 0; i < a.topk; i++) { a.wts[i] = __fdiv_rn(ex[i], wsum); a.top[i] = tp[i]; }
    }
}

// Publication for a consumer that does not wait for this kernel to end (the fused fold of the
// speculative step): sequence-tagged 64-bit copies of the routing this thread has just written.
// Launches that publish are serialised on one stream, so the sequence word has a single writer.
__device__ __forceinline__ void publish_route(const RouterArgs &a) {
#ifdef BRRR_TEST_HOOKS
    if (a.state && (a.state->test_hooks & 2u)) return;      // test hook: stay silent, the consumer's bounded wait runs out
#endif
    const uint32_t seq = __ldcg(a.signal) + 1u;
    for (int i = 0; i < a.topk; i++) {
        __stcg(&a.pub[i], ((unsigned long long)seq << 32) | (uint32_t)a.top[i]);
        __stcg(&a.pub[8 + i], ((unsigned long long)seq << 32) | __float_as_uint(a.wts[i]));
    }
    __stcg(a.signal, seq);
}

__global__ void __launch_bounds__(RT_THREADS) ffn_in_kernel(RouterArgs a) {
    // blockIdx.y = token of a tile: inputs d apart, logits ne apart, routing 8 entries apart, one arrival counter each
    a.x_in += (size_t)blockIdx.y * a.d;
    a.logits += (size_t)blockIdx.y * a.ne;
    a.top += blockIdx.y * 8;
    a.wts += blockIdx.y * 8;
    a.counter += blockIdx.y;
    extern __shared__ __align__(128) unsigned char smraw[];
    float *tiles = reinterpret_cast<float *>(smraw);                                        // [RT_STAGES][32][RT_STRIDE]
    float *xn = reinterpret_cast<float *>(smraw + (size_t)RT_TILE_FLOATS * 4 * RT_STAGES);   // d floats
    float *lg = xn + a.d;                                                                   // ne floats (top-k staging)
    float *wn = lg + ((a.ne + 3) & ~3);                                        // d floats: norm weights (16-byte aligned: float4 stores)
    uint64_t *bars = reinterpret_cast<uint64_t *>(wn + a.d);                   // [RT_STAGES] tile landed
    uint64_t *empty = bars + RT_STAGES;                                        // [RT_STAGES] tile consumed
    __shared__ float inv_sh;
    __shared__ int last_sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, d = a.d;
    uint32_t *err = a.state ? &a.state->err : nullptr;
    Waiter waiter(err);
    const int e0 = blockIdx.x * 32;
    const int nloc = min(32, a.ne - e0);
    const int ntiles = (d + RT_TJ - 1) / RT_TJ;
    const float *wsrc = a.Wt + (size_t)blockIdx.x * ntiles * RT_TILE_FLOATS;

    auto issue = [&](int t) {                                       // one thread
        int slot = t % RT_STAGES;
        mbar_expect_tx(&bars[slot], (uint32_t)RT_TILE_FLOATS * 4);
        bulk_g2s(tiles + (size_t)slot * RT_TILE_FLOATS, wsrc + (size_t)t * RT_TILE_FLOATS, (uint32_t)RT_TILE_FLOATS * 4, &bars[slot]);
    };
    BRRR_STAMP(a.state, 0);
    if (tid == 0) {
        for (int s = 0; s < RT_STAGES; s++) { mbar_init(&bars[s], 1); mbar_init(&empty[s], 1); }
        mbar_fence_init();
    }
    __syncwarp();
    if (tid < min(RT_STAGES, ntiles)) issue(tid);        // one lane per stage: the copies' address translations overlap
    if (a.norm_w) stage_vec4(a.norm_w, wn, d, tid, RT_THREADS);             // static: fetched before the wait
    const float bias_pre = (warp == 0 && lane < nloc && a.b) ? a.b[e0 + lane] : 0.0f;
    BRRR_STAMP(a.state, 1);
    pdl_wait();          // residual stream complete
    BRRR_STAMP(a.state, 2);
    BRRR_GT_GO(a.state, 30);
    pdl_trigger();
    waiter.poison_if_failed();
    stage_vec4(a.x_in, xn, d, tid, RT_THREADS);
    __syncthreads();
    if (a.norm_w) {
        float inv;
        if (a.qwen_norm) {
            __shared__ float part[QW_NT];
            if (tid < QW_NT) {
                int lo, hi;
                qw_slice(tid, d, lo, hi);
                float ps = 0.0f;
#pragma unroll 8
                for (int i = lo; i < hi; i++) { const float v = xn[i]; ps = __fadd_rn(ps, __fmul_rn(v, v)); }
                part[tid] = ps;
            }
            __syncthreads();
            float tot = 0.0f;
#pragma unroll
            for (int k = 0; k < QW_NT; k++) tot = __fadd_rn(tot, part[k]);
            inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)d), a.eps)));
        } else inv = block_rms_inv(xn, d, a.eps, &inv_sh);
        for (int i = tid; i < d; i += RT_THREADS) xn[i] = __fmul_rn(__fmul_rn(xn[i], inv), wn[i]);
        __syncthreads();
    }
    if (a.q8k_q && blockIdx.x == 0 && blockIdx.y == 0 && warp >= 2) {
        // warps 2..7 of the first CTA, beside the chain warp: Q8_K of the normalised token
        for (int sb = warp - 2; sb < d / 256; sb += RT_THREADS / 32 - 2) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = xn[sb * 256 + lane * 8 + i];
            warp_quant_q8k(v, lane, a.q8k_q + sb * 256, a.q8k_s + sb, a.q8k_bsum + sb * 8);
        }
    }

    BRRR_STAMP(a.state, 3);
    if (warp == 1 && lane == 0) {
        // refill thread: as soon as the chain warp releases a slot, the tile RT_STAGES ahead goes in
        for (int t = RT_STAGES; t < ntiles; t++) {
            waiter.wait(&empty[t % RT_STAGES], (uint32_t)(t / RT_STAGES - 1) & 1u);
            fence_proxy_async();
            issue(t);
        }
    }
    if (warp == 0) {
        float acc = bias_pre;
        for (int t = 0; t < ntiles; t++) {
            if (t < 12) BRRR_STAMP(a.state, 8 + t);
            const int slot = t % RT_STAGES, j0 = t * RT_TJ, len = min(RT_TJ, d - j0);
            waiter.wait(&bars[slot], (uint32_t)(t / RT_STAGES) & 1u);
            const float *row = tiles + (size_t)slot * RT_TILE_FLOATS + lane * RT_STRIDE;
            const float *xr = xn + j0;
            if (len == RT_TJ) acc = chain_span<RT_TJ>(row, xr, acc);
            else
                for (int jj = 0; jj < len; jj += 32) acc = chain_span<32>(row + jj, xr + jj, acc);   // d % 64 == 0
            __syncwarp();                      // all lanes are done reading this slot
            if (lane == 0 && t + RT_STAGES < ntiles) mbar_arrive(&empty[slot]);
        }
        if (lane < nloc) {
            if (gridDim.x == 1) lg[lane] = acc;
            a.logits[e0 + lane] = acc;
        }
        BRRR_STAMP(a.state, 4);
        if (gridDim.x == 1) {                  // single CTA: top-k straight from shared memory
            __syncwarp();
            warp_topk(a, lg, lane);
        }
        BRRR_STAMP(a.state, 5);
        BRRR_GT_END(a.state, 31);
        if (gridDim.x == 1 && lane == 0 && a.signal) publish_route(a);      // routing written by this lane
    }
    if (gridDim.x == 1) return;

    // several CTAs: the last one to arrive runs the top-k over all logits
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned prev = atomicAdd(a.counter, 1u);
        last_sh = (prev == gridDim.x - 1);
    }
    __syncthreads();
    if (!last_sh) return;
    __threadfence();
    for (int e = tid; e < a.ne; e += RT_THREADS) lg[e] = __ldcg(a.logits + e);
    __syncthreads();
    if (warp == 0) warp_topk(a, lg, lane);
    if (tid == 0) {
        *a.counter = 0u;
        if (a.signal) publish_route(a);
    }
}

size_t router_packed_floats(int ne, int d) { return (size_t)((ne + 31) / 32) * ((d + RT_TJ - 1) / RT_TJ) * RT_TILE_FLOATS; }

cudaError_t launch_ffn_in(const float *x_in, const float *norm_w, float eps, int d, const float *Wt, const float *b, int ne, int topk,
                          float *logits, int32_t *top, float *wts, unsigned int *counter, DevState *state, bool pdl, cudaStream_t st, int ntok,
                          uint32_t *signal, int qwen_norm, int8_t *q8k_q, float *q8k_s, int32_t *q8k_bsum) {
    RouterArgs a{x_in, norm_w, eps, d, Wt, b, ne, topk, logits, top, wts, counter, state, signal, (signal && state) ? state->route_pub : nullptr,
                 qwen_norm, q8k_q, q8k_s, q8k_bsum};
    if (signal && !state) return cudaErrorInvalidValue;
    size_t smem = (size_t)RT_TILE_FLOATS * 4 * RT_STAGES + (size_t)d * 8 + (size_t)((ne + 3) & ~3) * 4 + RT_STAGES * 16;
    static unsigned long long configured = 0;      // one bit per device
    {
        cudaError_t e = smem_optin(ffn_in_kernel, 200 * 1024, configured);
        if (e != cudaSuccess) return e;
    }
    return launch_k(ffn_in_kernel, dim3((ne + 31) / 32, ntok), dim3(RT_THREADS), smem, st, pdl, a);
}

// ---------------------------------------------------------------- routing hint (speculation)
// A fast, order-free estimate of the router: one CTA per expert forms its logit with a parallel
// reduction (a few ulps away from the serial chain); consumers pick the k largest themselves
// (warp_spec_select).  The estimate only decides WHICH experts' gate/up weights start streaming while ffn_in_kernel walks
// the exact serial chains next to it; the exact top-k, its order and its weights still come from
// ffn_in_kernel, and down_combine_kernel refuses (spec_fail_step) any step whose exact expert set
// is not covered by the estimate, so results never depend on this kernel.
struct HintArgs {
    const float *x_in, *norm_w;
    float eps;
    int d;
    const float *Wt, *b;
    int ne, topk;
    float *est;              // [ne] estimated logits
    int8_t *xq_out;          // nullable: Q8 of the normalised vector, each CTA writes a share
    float *xs_out;
    DevState *state;
    uint8_t *bimg_out;       // nullable: digit-plane operand image of the same vector (brrr_mxt.cuh)
};

constexpr int HINT_THREADS = 128;
constexpr int HINT_MAXG = 8;         // float4 groups per thread kept in registers (d <= 4096)

__global__ void __launch_bounds__(HINT_THREADS) router_hint_kernel(HintArgs a) {
    extern __shared__ __align__(16) float hsm[];      // d floats of x, then ne floats
    float *xf = hsm, *lg = hsm + a.d;
    __shared__ float inv_sh, red[HINT_THREADS / 32];
    const int tid = threadIdx.x, e = blockIdx.x, d = a.d, groups = d >> 2;
    const int ntiles = (d + RT_TJ - 1) / RT_TJ;
    // static operands first: this expert's row of the tiled matrix and the norm weights
    const float *wrow = a.Wt + ((size_t)(e >> 5) * ntiles * 32 + (e & 31)) * RT_STRIDE;
    float4 w[HINT_MAXG], nw[HINT_MAXG];
#pragma unroll
    for (int p = 0; p < HINT_MAXG; p++) {
        const int g = tid + p * HINT_THREADS;
        if (g < groups) {
            const int j = g * 4, t = j / RT_TJ, jj = j % RT_TJ;
            w[p] = *reinterpret_cast<const float4 *>(wrow + (size_t)t * RT_TILE_FLOATS + jj);
            nw[p] = a.norm_w ? reinterpret_cast<const float4 *>(a.norm_w)[g] : make_float4(1.f, 1.f, 1.f, 1.f);
        } else { w[p] = make_float4(0.f, 0.f, 0.f, 0.f); nw[p] = w[p]; }
    }
    const float bias = a.b ? a.b[e] : 0.0f;
    BRRR_GT_START(a.state, 235);
    pdl_wait();
    BRRR_GT_GO(a.state, 224);
    pdl_trigger();
    stage_vec4(a.x_in, xf, d, tid, HINT_THREADS);
    __syncthreads();
    float inv = 1.0f;
    if (a.norm_w) inv = block_rms_inv(xf, d, a.eps, &inv_sh);
    float part = 0.0f;
#pragma unroll
    for (int p = 0; p < HINT_MAXG; p++) {
        const int g = tid + p * HINT_THREADS;
        if (g < groups) {
            float4 x = reinterpret_cast<const float4 *>(xf)[g];
            part += w[p].x * (x.x * inv * nw[p].x) + w[p].y * (x.y * inv * nw[p].y) + w[p].z * (x.z * inv * nw[p].z) + w[p].w * (x.w * inv * nw[p].w);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((tid & 31) == 0) red[tid >> 5] = part;
    __syncthreads();
    if (tid == 0) {
        float s = bias;
        for (int i = 0; i < HINT_THREADS / 32; i++) s += red[i];
        a.est[e] = s;
    }
    // This CTA's share of the Q8 quantisation of the normalised vector (exact, block-local):
    // gate/up then stages 3 KB instead of normalising and quantising in every CTA.
    if (a.xq_out) {
        const int nb = d / 32, warp = tid >> 5, lane = tid & 31;
        for (int blk = e * (HINT_THREADS / 32) + warp; blk < nb; blk += gridDim.x * (HINT_THREADS / 32)) {
            float v = xf[blk * 32 + lane];
            if (a.norm_w) v = __fmul_rn(__fmul_rn(v, inv), a.norm_w[blk * 32 + lane]);
            const float amax = fmaxf(warp_max(fabsf(v)), 1e-12f);
            const float sc = __fdiv_rn(amax, 127.0f);
            const int qv = brrr_q8_round(v, sc);
            if (lane == 0) a.xs_out[blk] = sc;
            a.xq_out[blk * 32 + lane] = (int8_t)qv;
            if (a.bimg_out) xt_emit_block(qv, lane, blk, a.bimg_out);
        }
    }
    BRRR_GT_END(a.state, 225);
}

cudaError_t launch_router_hint(const float *x_in, const float *norm_w, float eps, int d, const float *Wt, const float *b, int ne, int topk,
                               float *est, int8_t *xq_out, float *xs_out, DevState *state, bool pdl, cudaStream_t st, uint8_t *bimg_out) {
    HintArgs a{x_in, norm_w, eps, d, Wt, b, ne, topk, est, xq_out, xs_out, state, bimg_out};
    size_t smem = (size_t)(d + ne + 4) * sizeof(float);
    return launch_k(router_hint_kernel, dim3(ne), dim3(HINT_THREADS), smem, st, pdl, a);
}

}  // namespace brrr
