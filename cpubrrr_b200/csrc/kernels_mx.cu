// MXFP4 expert matrices: load-time re-layout of GGUF blocks and the expert matvecs.
//
// Float order of one row (fixed): 4 lane chains.  Chain j walks the blocks b = 0, 1, ...
// accumulating fma(float(t_j(b)), 2^(e_b - 128) * xs[b], acc), t_j(b) being the exact int32
// lane dot (brrr_mx_lane_dot); the row result is (a0+a1)+(a2+a3).  One thread owns one chain.
//
// Data movement: 64 threads (16 rows x 4 lanes) consume one 16-row unit row of one expert matrix,
// a contiguous byte stream; a CTA runs 4 (or top-k) such streams side by side.  Thread 0 feeds
// all of them through a shared-memory ring with bulk asynchronous copies, one mbarrier per stage.
#include "brrr_kernels.h"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"
#include "brrr_mx.cuh"

namespace brrr {

// ---------------------------------------------------------------- pack: GGUF rows -> MxDev
// raw: [rows][blocks][17] (e8m0 byte, then 16 nibble bytes).  One thread per (row, block, lane).
__global__ void mx_pack_kernel(const uint8_t *__restrict__ raw, MxDev m) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)m.rows * m.blocks * 4;
    if (idx >= total) return;
    int j = (int)(idx & 3);
    size_t rb = idx >> 2;
    int b = (int)(rb % m.blocks), row = (int)(rb / m.blocks);
    const uint8_t *src = raw + rb * 17;
    int np = m.blocks / 2;
    uint32_t w = (uint32_t)src[1 + 4 * j] | ((uint32_t)src[2 + 4 * j] << 8) | ((uint32_t)src[3 + 4 * j] << 16) | ((uint32_t)src[4 + 4 * j] << 24);
    uint8_t *unit = m.data + mx_unit_off(row >> 4, b >> 1, np);
    int rl = row & 15;
    *reinterpret_cast<uint32_t *>(unit + rl * 32 + j * 8 + (b & 1) * 4) = w;
    if (j == 0) unit[MX_UNIT_EXPS + rl * 2 + (b & 1)] = src[0];
}

void launch_mx_pack(const uint8_t *raw, MxDev m, cudaStream_t st) {
    size_t total = (size_t)m.rows * m.blocks * 4;
    if (!total) return;
    mx_pack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(raw, m);
}


// Two blocks (one pair) of one lane chain from a unit in shared memory.
template <bool DBG>
__device__ __forceinline__ float mx_pair_step(const unsigned char *unit, int rl, int j, const int2 *xpj, const float *xsc, int pair, float acc, int32_t *dbg) {
    uint2 w = *reinterpret_cast<const uint2 *>(unit + rl * 32 + j * 8);
    uint32_t e2 = *reinterpret_cast<const unsigned short *>(unit + MX_UNIT_EXPS + rl * 2);
    int2 x0 = xpj[pair * 8], x1 = xpj[pair * 8 + 4];
    int t0 = brrr_mx_lane_dot(w.x, x0.x, x0.y);
    int t1 = brrr_mx_lane_dot(w.y, x1.x, x1.y);
    if (DBG) { dbg[(2 * pair) * 4] = t0; dbg[(2 * pair + 1) * 4] = t1; }
    acc = __fmaf_rn((float)t0, __fmul_rn(brrr_e8m0_scale(e2 & 0xFFu), xsc[2 * pair]), acc);
    acc = __fmaf_rn((float)t1, __fmul_rn(brrr_e8m0_scale(e2 >> 8), xsc[2 * pair + 1]), acc);
    return acc;
}

// ---------------------------------------------------------------- plain matvec (stage-level / tests)
// Reads units straight from global memory; optionally dumps the int32 block accumulators.
template <bool DBG>
__global__ void __launch_bounds__(256) mx_gemv_kernel(MxDev m, int row0, int nrows, const int8_t *__restrict__ xq, const float *__restrict__ xs,
                                                      float *__restrict__ y, int32_t *__restrict__ blockdots) {
    extern __shared__ __align__(128) unsigned char smraw[];
    const int nb = m.blocks, np = nb / 2;
    int2 *xp = reinterpret_cast<int2 *>(smraw);
    float *xsc = reinterpret_cast<float *>(smraw + (size_t)nb * 4 * sizeof(int2));
    mx_stage_x(xq, xs, nb, xp, xsc, threadIdx.x, 256);
    __syncthreads();
    int rl_out = blockIdx.x * 64 + (threadIdx.x >> 2), j = threadIdx.x & 3;
    bool live = rl_out < nrows;
    float acc = 0.0f;
    if (live) {
        int row = row0 + rl_out;
        for (int i = 0; i < np; i++)
            acc = mx_pair_step<DBG>(m.data + mx_unit_off(row >> 4, i, np), row & 15, j, xp + j, xsc, i, acc,
                                    DBG ? blockdots + (size_t)rl_out * nb * 4 + j : nullptr);
    }
    acc = brrr_hsum4(acc);
    if (live && j == 0) y[rl_out] = acc;
}

void launch_mx_gemv(MxDev m, int row0, int nrows, const int8_t *xq, const float *xs, float *y, int32_t *blockdots, cudaStream_t st) {
    size_t smem = (size_t)m.blocks * 4 * sizeof(int2) + m.blocks * sizeof(float);
    unsigned grid = (nrows + 63) / 64;
    if (blockdots) mx_gemv_kernel<true><<<grid, 256, smem, st>>>(m, row0, nrows, xq, xs, y, blockdots);
    else mx_gemv_kernel<false><<<grid, 256, smem, st>>>(m, row0, nrows, xq, xs, y, blockdots);
}


// ---------------------------------------------------------------- gate / up + SwiGLU + quantiser
// One CTA per (expert slot ei, 32-row block): streams 0,1 = the two gate unit rows, 2,3 = the two
// up unit rows of expert top[ei].  The 32 gate and 32 up results (bias added) pass through the
// clamped SwiGLU and are quantised as one Q8 block of h.
struct GateUpArgs {
    MxDev gate, up;
    const float *gate_b, *up_b;
    const int32_t *top;
    int d;
    const float *x_f32;      // residual stream (norm_w != null) or normalised vector (norm_w == null); null: use xq/xs
    const float *norm_w;
    float eps;
    const int8_t *xq;
    const float *xs;
    int8_t *hq;
    float *hs;
    float *gu;               // nullable: [topk][2d] gate | up (bias added), for inspection
    DevState *state;
    int ch, stages;
    const float *est;        // nullable: router estimate; the expert set is its top-k instead of top[]
    int ne, topk;
    int e_lo, e_cnt;         // experts held by gate/up: [e_lo, e_lo + e_cnt)
};

__global__ void __launch_bounds__(256) gate_up_kernel(GateUpArgs a) {
    extern __shared__ __align__(128) unsigned char smraw[];
    const int nb = a.gate.blocks, np = nb / 2, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    MxRing r;
    r.ch = a.ch; r.stages = a.stages; r.np = np; r.ns = 4;
    r.stream_bytes = (size_t)a.ch * MX_UNIT; r.stage_bytes = r.stream_bytes * 4;
    r.ring = smraw;
    float *xf = reinterpret_cast<float *>(smraw + r.stage_bytes * a.stages);   // d floats when x_f32 is given (16-byte aligned)
    int2 *xp = reinterpret_cast<int2 *>(xf + (a.x_f32 ? a.d : 0));
    float *xsc = reinterpret_cast<float *>(xp + nb * 4);
    r.bars = reinterpret_cast<uint64_t *>(xsc + nb + (nb & 1));
    __shared__ float inv_sh;
    __shared__ float gu_s[2][32];
    __shared__ const uint8_t *src[4];
    uint32_t *err = a.state ? &a.state->err : nullptr;
    Waiter waiter(err);
    const int ei = blockIdx.y, blk32 = blockIdx.x;
    BRRR_STAMP(a.state, 96);
    __shared__ float tbl[256];
    mx_fill_scale_table(tbl, tid, 256);
    if (tid == 0) {
        for (int s = 0; s < a.stages; s++) mbar_init(&r.bars[s], 1);
        mbar_fence_init();
    }
    // The activation comes from two kernels back (complete by the launch protocol), so it is
    // normalised and quantised here, before waiting for the router that runs alongside.
    if (a.x_f32) {
        float4 wreg[3];
        norm_prefetch<3>(a.norm_w, a.d, wreg, tid, 256);
        block_norm_quant<NQ_MX, 3>(a.x_f32, a.norm_w, wreg, a.eps, a.d, xf, xp, xsc, &inv_sh, tid, 256);
    }
    BRRR_STAMP(a.state, 97);
    pdl_wait();          // router done: top[] valid
    BRRR_STAMP(a.state, 98);
    BRRR_GT_GO(a.state, 126);
    pdl_trigger();
    waiter.poison_if_failed();
    __shared__ int sel[8];
    __shared__ float lg[256];
    // all global reads of this phase are issued together: the activation words go to registers
    // first, the expert set is ranked, then the activation is staged
    uint32_t xlo[2], xhi[2];
    if (!a.x_f32) {
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int idx = tid + k * 256;
            if (idx < nb * 4) {
                const uint32_t *xw = reinterpret_cast<const uint32_t *>(a.xq + (idx >> 2) * 32);
                xlo[k] = xw[idx & 3]; xhi[k] = xw[4 + (idx & 3)];
            }
        }
    }
    if (a.est) {
        block_spec_select(a.est, a.ne, a.topk, a.state, lg, sel, tid, 256);
        __syncthreads();
    }
    BRRR_STAMP(a.state, 102);
    const int e = a.est ? sel[ei] : a.top[ei];
    const int el = e - a.e_lo;                       // index among the experts held here
    if (el < 0 || el >= a.e_cnt) return;             // this slot's expert lives on another rank
    const int nchunks = (np + a.ch - 1) / a.ch;
    if (warp == 0) {
        if (lane < 4) src[lane] = ((lane & 2) ? a.up.data : a.gate.data) + mx_unit_off(((el * a.d + blk32 * 32) >> 4) + (lane & 1), 0, np);
        __syncwarp();
        r.issue_warp(0, min(a.stages, nchunks), src, lane);
    }
    BRRR_STAMP(a.state, 103);
    if (!a.x_f32) {
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int idx = tid + k * 256;
            if (idx < nb * 4) xp[idx] = mx_interleave(xlo[k], xhi[k]);
        }
        for (int idx = tid + 512; idx < nb * 4; idx += 256) {          // d > 4096 only
            const uint32_t *xw = reinterpret_cast<const uint32_t *>(a.xq + (idx >> 2) * 32);
            xp[idx] = mx_interleave(xw[idx & 3], xw[4 + (idx & 3)]);
        }
        for (int b = tid; b < nb; b += 256) xsc[b] = a.xs[b];
    }
    __syncthreads();

    BRRR_STAMP(a.state, 99);
    const int sidx = tid >> 6, rl = (tid & 63) >> 2, j = tid & 3;
    const int isup = sidx >> 1, r32 = (sidx & 1) * 16 + rl;
    // the bias is fetched while the weight stream is in flight
    const float bias_pre = j == 0 ? (isup ? a.up_b : a.gate_b)[(size_t)e * a.d + blk32 * 32 + r32] : 0.0f;
    float acc = 0.0f;
    for (int c = 0; c < nchunks; c++) {
        if (c < 12) BRRR_STAMP(a.state, 104 + c);
        const int cnt = min(a.ch, np - c * a.ch), slot = c % a.stages;
        waiter.wait(&r.bars[slot], (uint32_t)(c / a.stages) & 1u);
        if (c < 12) BRRR_STAMP(a.state, 116 + c);
        const unsigned char *base = r.ring + r.stage_bytes * slot + r.stream_bytes * sidx;
        acc = mx_chunk(base, cnt, rl, j, xp + j, xsc, tbl, c * a.ch, acc);
        if (c + a.stages < nchunks) {
            __syncthreads();
            if (warp == 0) r.issue_warp(c + a.stages, 1, src, lane);
        }
    }
    BRRR_STAMP(a.state, 100);
    acc = brrr_hsum4(acc);
    if (j == 0) {
        float v = __fadd_rn(acc, bias_pre);
        gu_s[isup][r32] = v;
        if (a.gu) a.gu[(size_t)ei * 2 * a.d + (size_t)isup * a.d + blk32 * 32 + r32] = v;
    }
    __syncthreads();
    if (warp == 0) {
        float h = swiglu_oai(gu_s[0][lane], gu_s[1][lane]);
        warp_quant_block(h, lane, a.hq + (size_t)ei * a.d + blk32 * 32, a.hs + ei * nb + blk32);
    }
    BRRR_STAMP(a.state, 101);
    BRRR_GT_END(a.state, 127);
}

cudaError_t launch_gate_up(MxDev gate, MxDev up, const float *gate_b, const float *up_b, const int32_t *top, int topk, int d,
                           const float *x_f32, const float *norm_w, float eps, const int8_t *xq, const float *xs,
                           int8_t *hq, float *hs, float *gu, DevState *state, bool pdl, cudaStream_t st,
                           const float *est, int ne, int e_lo, int e_cnt) {
    GateUpArgs a{};
    a.e_lo = e_lo; a.e_cnt = e_cnt;
    a.est = est; a.ne = ne; a.topk = topk;
    a.gate = gate; a.up = up; a.gate_b = gate_b; a.up_b = up_b; a.top = top; a.d = d;
    a.x_f32 = x_f32; a.norm_w = norm_w; a.eps = eps; a.xq = xq; a.xs = xs; a.hq = hq; a.hs = hs; a.gu = gu; a.state = state;
    const int nb = gate.blocks, np = nb / 2;
    // Every CTA of the grid must be resident at once (3 per SM at the 20b shape), so the ring is
    // kept near 52 KB: chunks of 8 pairs (4 streams x 4.3 KB), 3 stages.
    MxLaunchShape s = mx_shape(np, 4, 56 * 1024);
    if (np > 8) { s.ch = 8; int nch = (np + 7) / 8; s.stages = nch < 3 ? nch : 3; }
    a.ch = s.ch; a.stages = s.stages;
    size_t smem = (size_t)4 * a.ch * MX_UNIT * a.stages + (size_t)nb * 4 * 8 + (size_t)nb * 4 + (x_f32 ? (size_t)d * 4 : 0) + 8 + (size_t)a.stages * 8;
    static unsigned long long configured = 0;      // one bit per device
    {
        cudaError_t e = smem_optin(gate_up_kernel, 200 * 1024, configured);
        if (e != cudaSuccess) return e;
    }
    return launch_k(gate_up_kernel, dim3(d / 32, topk), dim3(256), smem, st, pdl, a);
}

// ---------------------------------------------------------------- down + weighted combine
// One CTA per 16 output rows; stream ei = that unit row of expert top[ei]'s down matrix, consumed
// by 64 threads against the slot's own activation hq[ei].  One thread per row then folds
// s = x; s += wts[ei] * (acc_ei + bias) for ei ascending (multiply then add).
struct DownArgs {
    MxDev down;
    const float *down_b;
    const int32_t *top;
    const float *wts;
    const float *est;          // nullable: router estimate whose top-k the hq/hs slots were computed for
    int ne;
    int topk, d;
    const int8_t *hq;
    const float *hs;
    float *x;
    DevState *state;
    int ch, stages;
};

__global__ void __launch_bounds__(512) down_combine_kernel(DownArgs a) {
    extern __shared__ __align__(128) unsigned char smraw[];
    const int nb = a.down.blocks, np = nb / 2, tid = threadIdx.x, nthreads = a.topk * 64;
    MxRing r;
    r.ch = a.ch; r.stages = a.stages; r.np = np; r.ns = a.topk;
    r.stream_bytes = (size_t)a.ch * MX_UNIT; r.stage_bytes = r.stream_bytes * a.topk;
    r.ring = smraw;
    const size_t per = (size_t)nb * 4 * sizeof(int2) + (size_t)nb * sizeof(float);   // one slot's staged activation
    unsigned char *xbase = smraw + r.stage_bytes * a.stages;
    float *part = reinterpret_cast<float *>(xbase + per * a.topk);                    // [topk][16]
    r.bars = reinterpret_cast<uint64_t *>(part + a.topk * 16);
    __shared__ const uint8_t *src[8];
    uint32_t *err = a.state ? &a.state->err : nullptr;
    Waiter waiter(err);
    const int nchunks = (np + a.ch - 1) / a.ch;
    BRRR_STAMP(a.state, 128);
    __shared__ float tbl[256];
    mx_fill_scale_table(tbl, tid, nthreads);
    if (tid == 0) {
        for (int s = 0; s < a.stages; s++) mbar_init(&r.bars[s], 1);
        mbar_fence_init();
    }
    if (tid < 32) {
        // expert ids come from the router, two kernels back: complete by the launch protocol,
        // so the weight stream starts before this kernel waits for gate/up
        if (tid < a.topk) src[tid] = a.down.data + mx_unit_off(((a.top[tid] * a.d) >> 4) + blockIdx.x, 0, np);
        __syncwarp();
        r.issue_warp(0, min(min(a.stages, nchunks), 32 / a.topk), src, tid);
        for (int c = 32 / a.topk; c < min(a.stages, nchunks); c++) r.issue_warp(c, 1, src, tid);
    }
    // operands of the final fold: routing is two kernels old, the residual three
    float x_pre = 0.0f, b_pre[8], w_pre[8];
    if (tid < 16) {
        const int rr = blockIdx.x * 16 + tid;
        x_pre = a.x[rr];
#pragma unroll
        for (int k = 0; k < 8; k++)
            if (k < a.topk) { b_pre[k] = a.down_b[(size_t)a.top[k] * a.d + rr]; w_pre[k] = a.wts[k]; }
    }
    BRRR_STAMP(a.state, 129);
    pdl_wait();          // gate/up done: hq, hs valid
    BRRR_STAMP(a.state, 130);
    BRRR_GT_GO(a.state, 158);
    pdl_trigger();
    waiter.poison_if_failed();
    const int ei = tid >> 6, t64 = tid & 63;
    int2 *xp = reinterpret_cast<int2 *>(xbase + per * ei);
    float *xsc = reinterpret_cast<float *>(xbase + per * ei + (size_t)nb * 4 * sizeof(int2));
    // which slot of hq/hs holds this rank's expert (identity without speculation)
    int slot = ei;
    if (a.est) {
        __shared__ int sel[8];
        __shared__ float lg[256];
        block_spec_select(a.est, a.ne, a.topk, a.state, lg, sel, tid, nthreads);
        __syncthreads();
        slot = -1;
        const int want = a.top[ei];
        for (int s = 0; s < a.topk; s++) if (sel[s] == want) slot = s;
        if (slot < 0) {                       // the estimate missed this expert: flag the step, keep going
            slot = 0;
            if (t64 == 0 && blockIdx.x == 0 && a.state) atomicMin(&a.state->spec_fail_step, a.state->n_out);
        }
    }
    mx_stage_x(a.hq + (size_t)slot * a.d, a.hs + (size_t)slot * nb, nb, xp, xsc, t64, 64);
    __syncthreads();

    BRRR_STAMP(a.state, 131);
    const int rl = t64 >> 2, j = t64 & 3;
    float acc = 0.0f;
    for (int c = 0; c < nchunks; c++) {
        if (c < 12) BRRR_STAMP(a.state, 136 + c);
        const int cnt = min(a.ch, np - c * a.ch), slot = c % a.stages;
        waiter.wait(&r.bars[slot], (uint32_t)(c / a.stages) & 1u);
        if (c < 12) BRRR_STAMP(a.state, 148 + c);
        const unsigned char *base = r.ring + r.stage_bytes * slot + r.stream_bytes * ei;
        acc = mx_chunk(base, cnt, rl, j, xp + j, xsc, tbl, c * a.ch, acc);
        if (c + a.stages < nchunks) {
            __syncthreads();
            if (tid < 32) r.issue_warp(c + a.stages, 1, src, tid);
        }
    }
    BRRR_STAMP(a.state, 132);
    acc = brrr_hsum4(acc);
    if (j == 0) part[ei * 16 + rl] = acc;
    __syncthreads();
    if (tid < 16) {
        int rr = blockIdx.x * 16 + tid;
        float s = x_pre;
#pragma unroll
        for (int k = 0; k < 8; k++)
            if (k < a.topk) s = __fadd_rn(s, __fmul_rn(w_pre[k], __fadd_rn(part[k * 16 + tid], b_pre[k])));
        a.x[rr] = s;
    }
    BRRR_STAMP(a.state, 133);
    BRRR_GT_END(a.state, 159);
    (void)nthreads;
}

cudaError_t launch_down_combine(MxDev down, const float *down_b, const int32_t *top, const float *wts, const float *est, int ne,
                                int topk, int d, const int8_t *hq, const float *hs, float *x, DevState *state, bool pdl, cudaStream_t st) {
    DownArgs a{};
    a.down = down; a.down_b = down_b; a.top = top; a.wts = wts; a.est = est; a.ne = ne; a.topk = topk; a.d = d; a.hq = hq; a.hs = hs; a.x = x; a.state = state;
    const int nb = down.blocks, np = nb / 2;
    MxLaunchShape s = mx_shape(np, topk, 80 * 1024);
    a.ch = s.ch; a.stages = s.stages;
    size_t per = (size_t)nb * 4 * 8 + (size_t)nb * 4;
    size_t smem = (size_t)topk * a.ch * MX_UNIT * a.stages + per * topk + (size_t)topk * 16 * 4 + (size_t)a.stages * 8 + 8;
    static unsigned long long configured = 0;      // one bit per device
    {
        cudaError_t e = smem_optin(down_combine_kernel, 200 * 1024, configured);
        if (e != cudaSuccess) return e;
    }
    return launch_k(down_combine_kernel, dim3(d / 16), dim3(topk * 64), smem, st, pdl, a);
}

}  // namespace brrr
