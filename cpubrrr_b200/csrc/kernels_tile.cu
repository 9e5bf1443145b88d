// Token-tile MXFP4 matmul on the 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators in
// tensor memory): the batched counterpart of the per-token expert matvec, for prefill tiles and
// batched decode.  One pass over the weights serves up to 16 tokens, as the reference's tile path
// does on the CPU (src/bin/engine_gpt2.rs:1005-1010, TILE = 16), and every output equals the
// per-token result bit for bit.
//
// Arithmetic.  A row's value is four lane chains, each fma(float(t_lane(b)), 2^(e_b-128) * xs[b], acc)
// over the 32-blocks b, with t_lane(b) the exact int32 sum of the lane's 8 products.  The integer
// sums of 128 rows x 16 tokens x 4 lanes of one block are one 128 x 64 x 32 int8 matrix product:
//   A[row][k]           = the row's 32 codes decoded to signed bytes (k = 8*lane + i),
//   B[token*4+lane][k]  = the token's activation byte k if k belongs to `lane`, else 0,
// issued twice, once with the positive and once with the negative decode table (their sum is the
// signed value), accumulating in the same 128 x 64 int32 tile of tensor memory.  The four epilogue
// warps read their 32 lanes of tensor memory (tcgen05.ld) and run the float chains, one thread per
// row with 64 accumulators.
//
// This version is serialised per block pair inside a CTA (decode -> MMA -> epilogue; several CTAs
// per SM overlap each other, and the next pair's operands are fetched one pair ahead); operands are
// written to shared memory by the threads themselves in the canonical K-major no-swizzle layout
// (8-row x 16-byte core matrices).
#include "brrr_kernels.h"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"
#include "brrr_mx.cuh"

namespace brrr {

namespace {

constexpr int TL_ROWS = 128;           // rows per CTA = MMA M
constexpr int TL_N = 64;               // MMA N: 16 tokens x 4 chain lanes
constexpr int TL_MAXTOK = 16;
constexpr int TL_A_BYTES = TL_ROWS * 32;       // one decoded A tile (128 rows x 32 k bytes)
constexpr int TL_B_BYTES = TL_N * 32;
constexpr uint32_t TL_TMEM_COLS = 128;         // two 64-column accumulator tiles (the two blocks of a pair)

// shared-memory matrix descriptor: K-major, no swizzle; core matrix = 8 rows x 16 bytes, 128 bytes
// apart along M/N (stride byte offset), `lbo` bytes apart along K (leading byte offset)
__device__ __forceinline__ uint64_t tl_smem_desc(const void *p, uint32_t lbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(p) >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((128u >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;                      // descriptor version of this architecture
    return d;
}

// instruction descriptor, kind::i8: D = s32, A = B = signed 8-bit, both K-major, N = 64, M = 128
constexpr uint32_t TL_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((TL_N >> 3) << 17) | ((TL_ROWS >> 4) << 24);

__device__ __forceinline__ void tl_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(TL_IDESC), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tl_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tl_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tl_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 16 consecutive 32-bit columns of this warp's 32 lanes of tensor memory
__device__ __forceinline__ void tl_ld16(uint32_t taddr, int (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tl_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One launch serves blockIdx.y = expert (or a single matrix).  Each expert has a list of up to 16
// entries; entry i multiplies the activation row entry / src_div and writes output row entry.
struct TileArgs {
    MxDev w;
    int row0, nrows;         // rows [row0, row0 + nrows) of each expert's matrix
    int rows_per_expert;     // matrix row of (expert e, row r) = e * rows_per_expert + r
    const int *cnt;          // [experts] entries per expert; nullptr: one matrix, entries 0 .. ntok - 1
    const int *list;         // [experts][16]
    int src_div;
    const int8_t *xq;        // [activation rows][blocks * 32]
    const float *xs;         // [activation rows][blocks]
    int ntok;
    const float *bias;       // nullable: [experts][rows_per_expert], added to every output
    float *y;                // element [entry][col0 + row - row0], rows ldy apart
    int ldy, col0;
    DevState *state;
};

__global__ void __launch_bounds__(128) mx_tile_kernel(TileArgs a) {
    __shared__ __align__(128) unsigned char a_tiles[4][TL_A_BYTES];     // [block of the pair][P, N]
    __shared__ __align__(128) unsigned char b_tiles[2][TL_B_BYTES];
    __shared__ float tbl[256];
    __shared__ float xs_pair[2][TL_MAXTOK];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_base_sh;
    __shared__ int ent[TL_MAXTOK];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = a.w.blocks, np = nb / 2;
    const int e = blockIdx.y;
    const int n_ent = a.cnt ? a.cnt[e] : a.ntok;
    if (n_ent == 0) return;                      // no token routed to this expert (before anything is allocated)
    if (tid < TL_MAXTOK) ent[tid] = tid < n_ent ? (a.list ? a.list[e * TL_MAXTOK + tid] : tid) : 0;
    uint32_t *err = a.state ? &a.state->err : nullptr;
    Waiter waiter(err);
    const uint32_t P_LO = 0x04030200u, P_HI = 0x0D090705u, N_LO = 0xFDFEFF00u, N_HI = 0xF4F8FAFCu;

    mx_fill_scale_table(tbl, tid, 128);
    for (int i = tid; i < 2 * TL_B_BYTES / 16; i += 128) reinterpret_cast<uint4 *>(&b_tiles[0][0])[i] = make_uint4(0, 0, 0, 0);
    if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(TL_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tl_fence_before();
    __syncthreads();
    tl_fence_after();
    const uint32_t tmem_base = tmem_base_sh;

    // this thread's row: weights of (row, all four lanes) for a block pair are 32 contiguous bytes
    const int row_local = blockIdx.x * TL_ROWS + tid;
    const bool row_live = row_local < a.nrows;
    const int row = e * a.rows_per_expert + a.row0 + (row_live ? row_local : a.nrows - 1);   // out-of-range rows reread the last row, never stored
    const unsigned char *wrow = a.w.data + mx_unit_off(row >> 4, 0, np) + (row & 15) * 32;
    const unsigned char *erow = a.w.data + mx_unit_off(row >> 4, 0, np) + MX_UNIT_EXPS + (row & 15) * 2;
    // A element (row m, byte k) lives at (k / 16) * 2048 + (m / 8) * 128 + (m % 8) * 16 + k % 16
    const uint32_t a_off = (uint32_t)((tid >> 3) * 128 + (tid & 7) * 16);
    // B row n = token * 4 + lane holds the 8 activation bytes of `lane` at k = 8 * lane .. + 7
    const int bt = (tid & 63) >> 2, bl = tid & 3, bblk = tid >> 6;          // threads 0..63: first block of the pair, 64..127: second
    const uint32_t b_off = (uint32_t)((bl >> 1) * (TL_N * 16) + ((tid & 63) >> 3) * 128 + ((tid & 63) & 7) * 16 + (bl & 1) * 8);

    float acc[TL_N];
#pragma unroll
    for (int i = 0; i < TL_N; i++) acc[i] = 0.0f;

    // operands of a block pair are fetched one pair ahead, so their global-memory latency hides
    // behind the tensor-core work and the epilogue of the current pair
    const size_t srow = (size_t)(ent[bt] / a.src_div);
    const bool b_live = bt < n_ent;
    auto fetch_b = [&](int p, uint32_t &lo, uint32_t &hi, float &sc) {
        const int b = 2 * p + bblk;
        const uint32_t *xw = reinterpret_cast<const uint32_t *>(a.xq + (srow * nb + b) * 32);
        lo = b_live ? xw[bl] : 0u; hi = b_live ? xw[4 + bl] : 0u;
        sc = (b_live && bl == 0) ? a.xs[srow * nb + b] : 0.0f;
    };
    uint4 w0 = *reinterpret_cast<const uint4 *>(wrow), w1 = *reinterpret_cast<const uint4 *>(wrow + 16);
    uint32_t e2 = *reinterpret_cast<const unsigned short *>(erow);
    uint32_t xlo, xhi;
    float xsc;
    fetch_b(0, xlo, xhi, xsc);

    for (int p = 0; p < np; p++) {
        // ---- decode this row's two blocks into the four A tiles
        const uint32_t wl[4][2] = {{w0.x, w0.y}, {w0.z, w0.w}, {w1.x, w1.y}, {w1.z, w1.w}};
        const uint32_t e2c = e2;
#pragma unroll
        for (int j = 0; j < 4; j++) {
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const uint32_t w = wl[j][k], wx = w ^ 0x88888888u;
                const uint32_t off = (uint32_t)((j >> 1) * 2048) + a_off + (j & 1) * 8;
                *reinterpret_cast<uint2 *>(&a_tiles[2 * k][off]) = make_uint2(brrr_prmt(P_LO, P_HI, w), brrr_prmt(P_LO, P_HI, w >> 16));
                *reinterpret_cast<uint2 *>(&a_tiles[2 * k + 1][off]) = make_uint2(brrr_prmt(N_LO, N_HI, wx), brrr_prmt(N_LO, N_HI, wx >> 16));
            }
        }
        // ---- activations of the pair's two blocks into the B tiles (rows of absent tokens stay zero)
        {
            const int2 iv = mx_interleave(xlo, xhi);
            *reinterpret_cast<uint2 *>(&b_tiles[bblk][b_off]) = make_uint2((uint32_t)iv.x, (uint32_t)iv.y);
            if (bl == 0) xs_pair[bblk][bt] = xsc;
        }
        fence_proxy_async();               // generic-proxy writes above -> visible to the tensor core's reads
        __syncthreads();
        // ---- two blocks x two tables, one accumulator tile per block
        if (tid == 0) {
            tl_fence_after();
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const uint64_t db = tl_smem_desc(&b_tiles[k][0], TL_N * 16);
                tl_mma(tmem_base + k * TL_N, tl_smem_desc(&a_tiles[2 * k][0], 2048), db, 0u);
                tl_mma(tmem_base + k * TL_N, tl_smem_desc(&a_tiles[2 * k + 1][0], 2048), db, 1u);
            }
            tl_commit(&bar);
        }
        if (p + 1 < np) {                  // next pair's operands
            w0 = *reinterpret_cast<const uint4 *>(wrow + (size_t)(p + 1) * MX_UNIT);
            w1 = *reinterpret_cast<const uint4 *>(wrow + (size_t)(p + 1) * MX_UNIT + 16);
            e2 = *reinterpret_cast<const unsigned short *>(erow + (size_t)(p + 1) * MX_UNIT);
            fetch_b(p + 1, xlo, xhi, xsc);
        }
        waiter.wait(&bar, (uint32_t)p & 1u);
        tl_fence_after();
        // ---- float chains: thread = row (tensor-memory lane), 64 columns per block
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const float esc = tbl[k ? e2c >> 8 : e2c & 0xFFu];
            int d[4][16];
#pragma unroll
            for (int c = 0; c < 4; c++) tl_ld16(lane_addr + k * TL_N + 16 * c, d[c]);
            tl_wait_ld();
#pragma unroll
            for (int c = 0; c < 4; c++) {
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    const float s = __fmul_rn(esc, xs_pair[k][4 * c + t]);
#pragma unroll
                    for (int l = 0; l < 4; l++) acc[16 * c + 4 * t + l] = __fmaf_rn((float)d[c][4 * t + l], s, acc[16 * c + 4 * t + l]);
                }
            }
        }
        tl_fence_before();
        __syncthreads();                   // tiles and accumulators are free for the next pair
    }
    if (row_live) {
        const float bias = a.bias ? a.bias[(size_t)e * a.rows_per_expert + a.row0 + row_local] : 0.0f;
#pragma unroll
        for (int t = 0; t < TL_MAXTOK; t++)
            if (t < n_ent) {
                float v = __fadd_rn(__fadd_rn(acc[4 * t], acc[4 * t + 1]), __fadd_rn(acc[4 * t + 2], acc[4 * t + 3]));
                if (a.bias) v = __fadd_rn(v, bias);
                a.y[(size_t)ent[t] * a.ldy + a.col0 + row_local] = v;
            }
    }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TL_TMEM_COLS) : "memory");
}

// Per expert, the (token, slot) pairs routed to it, in ascending order: entry = token * topk + slot.
__global__ void tile_route_kernel(const int32_t *__restrict__ top, int ntok, int topk, int ne, int *__restrict__ cnt, int *__restrict__ list) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= ne) return;
    int c = 0;
    for (int t = 0; t < ntok; t++)
        for (int s = 0; s < topk; s++)
            if (top[t * 8 + s] == e && c < TL_MAXTOK) list[e * TL_MAXTOK + c++] = t * topk + s;
    cnt[e] = c;
}

// x[t] += w[t][k] * part[t * topk + k], k ascending (part already holds the bias): the fold of
// down_combine_kernel, one thread per (token, row).
__global__ void tile_combine_kernel(const float *__restrict__ part, const float *__restrict__ wts, int topk, int d, float *__restrict__ x) {
    const int t = blockIdx.y, r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= d) return;
    float s = x[(size_t)t * d + r];
    for (int k = 0; k < topk; k++) s = __fadd_rn(s, __fmul_rn(wts[t * 8 + k], part[((size_t)t * topk + k) * d + r]));
    x[(size_t)t * d + r] = s;
}

}  // namespace

cudaError_t launch_mx_tile(MxDev w, int row0, int nrows, const int8_t *xq, const float *xs, int ntok, float *y, int ldy, DevState *state,
                           cudaStream_t st) {
    TileArgs a{};
    a.w = w; a.row0 = row0; a.nrows = nrows; a.src_div = 1; a.xq = xq; a.xs = xs; a.ntok = ntok; a.y = y; a.ldy = ldy; a.state = state;
    mx_tile_kernel<<<dim3((nrows + TL_ROWS - 1) / TL_ROWS, 1), 128, 0, st>>>(a);
    return cudaGetLastError();
}

// All experts of one matrix kind against their routed entries (see TileArgs).
cudaError_t launch_mx_tile_experts(MxDev w, int ne, int rows_per_expert, const int *cnt, const int *list, int src_div, const int8_t *xq,
                                   const float *xs, const float *bias, float *y, int ldy, int col0, DevState *state, cudaStream_t st) {
    TileArgs a{};
    a.w = w; a.row0 = 0; a.nrows = rows_per_expert; a.rows_per_expert = rows_per_expert; a.cnt = cnt; a.list = list; a.src_div = src_div;
    a.xq = xq; a.xs = xs; a.bias = bias; a.y = y; a.ldy = ldy; a.col0 = col0; a.state = state;
    mx_tile_kernel<<<dim3((rows_per_expert + TL_ROWS - 1) / TL_ROWS, ne), 128, 0, st>>>(a);
    return cudaGetLastError();
}

void launch_tile_route(const int32_t *top, int ntok, int topk, int ne, int *cnt, int *list, cudaStream_t st) {
    tile_route_kernel<<<(ne + 63) / 64, 64, 0, st>>>(top, ntok, topk, ne, cnt, list);
}

void launch_tile_combine(const float *part, const float *wts, int topk, int d, int ntok, float *x, cudaStream_t st) {
    tile_combine_kernel<<<dim3((d + 255) / 256, ntok), 256, 0, st>>>(part, wts, topk, d, x);
}

}  // namespace brrr
