// Expert-parallel decode across the GPUs of one node (gpt-oss): experts are sharded by index,
// everything else is replicated and computed redundantly (bit-identical on every rank), so the
// only exchange per layer is the down-projection output of the selected experts.
//
// down_ep_kernel fuses that exchange with the compute: the CTA that owns 16 output rows streams
// the local experts' rows, stores each finished 16-float slice straight into every rank's exchange
// buffer over NVLink peer memory, raises a per-slice flag, then waits (bounded) for the slices of
// the remote experts and folds all top-k slices in the fixed slot order
//   x += w_k * (slice_k + bias_k), k ascending
// which keeps the result bit-identical to the single-GPU path.  Plain peer stores and loads only:
// no multimem, no bulk copies from peer memory.
//
// Buffers are indexed by layer, flags carry the number of the step (epoch) that wrote them, and
// ep_begin_kernel lets a step start only after every rank has finished the previous one, so no
// slice is overwritten before it has been read.
#include "brrr_kernels.h"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"
#include "brrr_mx.cuh"

namespace brrr {

namespace {

// Start of a step: tell every rank that this rank has finished step `epoch`, wait until every
// rank has, then advance the epoch.  One warp.
__global__ void ep_begin_kernel(EpCtx c, DevState *state) {
    const int p = threadIdx.x;
    const uint32_t prev = *c.epoch;
    uint32_t *err = state ? &state->err : nullptr;
    if (p < c.world) {
        st_sys(c.done[p] + c.rank, prev);
        ep_wait(c.done[c.rank] + p, prev, err);
    }
    __syncwarp();
    if (p == 0) *c.epoch = prev + 1;
}

struct DownEpArgs {
    MxDev down;                // local experts only: rows = e_cnt * d
    const float *down_b;       // all experts (replicated)
    const int32_t *top;
    const float *wts;
    int topk, d, layer;
    const int8_t *hq;
    const float *hs;
    float *x;
    DevState *state;
    int ch, stages;
    EpCtx ep;
};

// The single-GPU down_combine_kernel with the top-k streams restricted to the local experts and
// the partial results exchanged before the fold.
__global__ void __launch_bounds__(512) down_ep_kernel(DownEpArgs a) {
    extern __shared__ __align__(128) unsigned char smraw[];
    const int nb = a.down.blocks, np = nb / 2, tid = threadIdx.x;
    const int ncta = a.d / 16;
    __shared__ int loc[8];               // slots whose expert lives here, ascending
    __shared__ int nloc_sh;
    __shared__ const uint8_t *src[8];
    __shared__ float tbl[256];
    uint32_t *err = a.state ? &a.state->err : nullptr;
    Waiter waiter(err);
    // routing comes from the router, two kernels back: complete by the launch protocol
    if (tid == 0) {
        int n = 0;
        for (int s = 0; s < a.topk; s++) {
            const int e = a.top[s] - a.ep.e_lo;
            if (e >= 0 && e < a.ep.e_cnt) { loc[n] = s; src[n] = a.down.data + mx_unit_off(((e * a.d) >> 4) + blockIdx.x, 0, np); n++; }
        }
        nloc_sh = n;
    }
    mx_fill_scale_table(tbl, tid, blockDim.x);
    __syncthreads();
    const int nloc = nloc_sh;
    MxRing r;
    r.ch = a.ch; r.stages = a.stages; r.np = np; r.ns = nloc > 0 ? nloc : 1;
    r.stream_bytes = (size_t)a.ch * MX_UNIT; r.stage_bytes = r.stream_bytes * a.topk;
    r.ring = smraw;
    const size_t per = (size_t)nb * 4 * sizeof(int2) + (size_t)nb * sizeof(float);
    unsigned char *xbase = smraw + r.stage_bytes * a.stages;
    float *part = reinterpret_cast<float *>(xbase + per * a.topk);                    // [topk][16]
    r.bars = reinterpret_cast<uint64_t *>(part + a.topk * 16);
    const int nchunks = (np + a.ch - 1) / a.ch;
    if (tid == 0) {
        for (int s = 0; s < a.stages; s++) mbar_init(&r.bars[s], 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (tid < 32 && nloc > 0)
        for (int c = 0; c < min(a.stages, nchunks); c++) r.issue_warp(c, 1, src, tid);
    // operands of the final fold
    float x_pre = 0.0f, b_pre[8], w_pre[8];
    if (tid < 16) {
        const int rr = blockIdx.x * 16 + tid;
        x_pre = a.x[rr];
#pragma unroll
        for (int k = 0; k < 8; k++)
            if (k < a.topk) { b_pre[k] = a.down_b[(size_t)a.top[k] * a.d + rr]; w_pre[k] = a.wts[k]; }
    }
    const uint32_t epoch = *a.ep.epoch;
    pdl_wait();          // gate/up done: hq, hs valid
    pdl_trigger();
    waiter.poison_if_failed();
    const int li = tid >> 6, t64 = tid & 63;          // local stream index of this 64-thread group
    const bool worker = li < nloc;
    int2 *xp = reinterpret_cast<int2 *>(xbase + per * li);
    float *xsc = reinterpret_cast<float *>(xbase + per * li + (size_t)nb * 4 * sizeof(int2));
    if (worker) {
        const int slot = loc[li];
        mx_stage_x(a.hq + (size_t)slot * a.d, a.hs + (size_t)slot * nb, nb, xp, xsc, t64, 64);
    }
    __syncthreads();
    const int rl = t64 >> 2, j = t64 & 3;
    float acc = 0.0f;
    for (int c = 0; c < nchunks && nloc > 0; c++) {
        const int cnt = min(a.ch, np - c * a.ch), slot = c % a.stages;
        if (worker) {
            waiter.wait(&r.bars[slot], (uint32_t)(c / a.stages) & 1u);
            const unsigned char *base = r.ring + r.stage_bytes * slot + r.stream_bytes * li;
            acc = mx_chunk(base, cnt, rl, j, xp + j, xsc, tbl, c * a.ch, acc);
        }
        if (c + a.stages < nchunks) {
            __syncthreads();
            if (tid < 32) r.issue_warp(c + a.stages, 1, src, tid);
        }
    }
    acc = brrr_hsum4(acc);
    // ---- publish the local slices to every rank, then raise their flags
    if (worker && j == 0) {
        const int slot = loc[li];
        const size_t off = ((size_t)a.layer * a.topk + slot) * a.d + blockIdx.x * 16 + rl;
        for (int p = 0; p < a.ep.world; p++) a.ep.xchg[p][off] = acc;
        __threadfence_system();
    }
    __syncthreads();
    if (tid < nloc * a.ep.world) {
        const int slot = loc[tid / a.ep.world], p = tid % a.ep.world;
        st_sys(a.ep.flags[p] + ((size_t)a.layer * a.topk + slot) * ncta + blockIdx.x, epoch);
    }
    // ---- fold in slot order once every slice of these 16 rows has arrived
    if (tid < 16) {
        const int rr = blockIdx.x * 16 + tid;
        float s = x_pre;
#pragma unroll
        for (int k = 0; k < 8; k++)
            if (k < a.topk) {
                const size_t base = (size_t)a.layer * a.topk + k;
                ep_wait(a.ep.flags[a.ep.rank] + base * ncta + blockIdx.x, epoch, err);
                const float v = ld_f32_sys(a.ep.xchg[a.ep.rank] + base * a.d + rr);
                s = __fadd_rn(s, __fmul_rn(w_pre[k], __fadd_rn(v, b_pre[k])));
            }
        a.x[rr] = s;
    }
}

}  // namespace

void launch_ep_begin(const EpCtx &c, DevState *state, cudaStream_t st) { ep_begin_kernel<<<1, 32, 0, st>>>(c, state); }

cudaError_t launch_down_ep(MxDev down, const float *down_b, const int32_t *top, const float *wts, int topk, int d, int layer, const int8_t *hq,
                           const float *hs, float *x, DevState *state, const EpCtx &ep, bool pdl, cudaStream_t st) {
    DownEpArgs a{};
    a.down = down; a.down_b = down_b; a.top = top; a.wts = wts; a.topk = topk; a.d = d; a.layer = layer; a.hq = hq; a.hs = hs; a.x = x;
    a.state = state; a.ep = ep;
    const int nb = down.blocks, np = nb / 2;
    MxLaunchShape sh = mx_shape(np, topk, 80 * 1024);
    a.ch = sh.ch; a.stages = sh.stages;
    size_t per = (size_t)nb * 4 * 8 + (size_t)nb * 4;
    size_t smem = (size_t)topk * a.ch * MX_UNIT * a.stages + per * topk + (size_t)topk * 16 * 4 + (size_t)a.stages * 8 + 8;
    static unsigned long long configured = 0;      // one bit per device
    {
        cudaError_t e = smem_optin(down_ep_kernel, 200 * 1024, configured);
        if (e != cudaSuccess) return e;
    }
    return launch_k(down_ep_kernel, dim3(d / 16), dim3(topk * 64), smem, st, pdl, a);
}

}  // namespace brrr
