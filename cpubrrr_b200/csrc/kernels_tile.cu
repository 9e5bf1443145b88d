// Token-tile MXFP4 matmul on the 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators in
// tensor memory): the batched counterpart of the per-token expert matvec, for prefill tiles and
// batched decode.  One pass over the weights serves up to 512 tokens, as the reference's tile path
// does on the CPU for 16 (src/bin/engine_gpt2.rs:1005-1010, TILE = 16), and every output equals the
// per-token result bit for bit.
//
// Arithmetic.  A row's value is four lane chains, each fma(float(t_lane(b)), 2^(e_b-128) * xs[b], acc)
// over the 32-blocks b, with t_lane(b) the exact int32 sum of the lane's 8 products.  The integer
// sums of 128 rows x NT tokens x 4 lanes of one block are one 128 x 4 NT x 32 int8 matrix product:
//   A[row][k]           = the row's 32 codes decoded to signed bytes (k = 8*lane + i),
//   B[token*4+lane][k]  = the token's activation byte k if k belongs to `lane`, else 0,
// issued twice, once with the positive and once with the negative decode table (their sum is the
// signed value), accumulating in the same 128 x 4 NT int32 tile of tensor memory.  The four worker
// warps read their 32 lanes of tensor memory (tcgen05.ld) and run the float chains, one thread per
// row with 4 NT accumulators.  NT = 4 entries per CTA for tiles of up to 16 tokens, 8 up to 64, 16 beyond.
//
// Operands are written to shared memory by the threads themselves in the canonical K-major
// no-swizzle layout (8-row x 16-byte core matrices).
#include <cstdlib>
#include "brrr_kernels.h"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"
#include "brrr_mx.cuh"

namespace brrr {

namespace {

constexpr int TL_ROWS = 128;           // rows per CTA = MMA M

constexpr int TL_MAXTOK = BRRR_TILE_MAX; // entries per expert and launch (one per token of the tile at most)
constexpr int TL_A_BYTES = TL_ROWS * 32;       // one decoded A tile (128 rows x 32 k bytes)

constexpr int TL_THREADS = 224;        // four worker warps, the producer warp, two issuer warps (q8_tile_kernel)
// mx_tile_kernel: one or two issuing threads, ring depth and CTAs per SM.  Measured on the 2048-token prefill (tok/s): 2 issuers /
// depth 5 / 3 CTAs 3956; 1 issuer 3973; depth 3 3969; 1 issuer + depth 3 + 4 CTAs per SM (80 registers, spills) 3648.
constexpr int MT_ISSUERS = 2;
constexpr int MT_CTAS = 3;
constexpr int MT_NT16_FROM = 65;         // tile size from which a CTA takes 16 entries (128 registers, 2 CTAs per SM: one decode of the weights serves
                                         // twice the entries; 256-row prefill 5864 against 5469 tok/s); BRRR_TILE_NT16_FROM=n moves it
constexpr int MT_THREADS = 160 + 32 * MT_ISSUERS;   // four worker warps, the producer warp, the issuer warp(s)
constexpr int TL_DEPTH = 5;            // weight ring: block pairs in flight per CTA
constexpr int TL_SLOT = 9 * MX_UNIT;   // one pair of a 128-row tile: up to 9 units of 16 rows
constexpr int TL_CPL = (TL_SLOT / 16 + 31) / 32;   // 16-byte pieces per producer lane and pair

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

// kind::i8 product; instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, N / 8 at bit 17, M / 16 at bit 24
__device__ __forceinline__ void tl_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
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
// packed pairs of floats for fma.rn.f32x2
__device__ __forceinline__ unsigned long long tl_pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
    return r;
}
__device__ __forceinline__ void tl_unpack2(unsigned long long v, float &lo, float &hi) {
    uint32_t a, b;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a); hi = __uint_as_float(b);
}
__device__ __forceinline__ unsigned long long tl_fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ void tl_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One launch serves blockIdx.y = (expert or the single matrix, chunk of entries).  Each expert has a list of up to 512
// entries; entry i multiplies the activation row entry / src_div and writes output row entry.
struct TileArgs {
    MxDev w;
    int row0, nrows;         // rows [row0, row0 + nrows) of each expert's matrix
    int rows_per_expert;     // matrix row of (expert e, row r) = e * rows_per_expert + r
    const int *cnt;          // [experts] entries per expert; nullptr: one matrix, entries 0 .. ntok - 1
    const int *list;         // [experts][TL_MAXTOK]
    int src_div;
    const int8_t *xq;        // [activation rows][blocks * 32]
    const float *xs;         // [activation rows][blocks]
    int ntok;
    int chunks;              // CTAs per expert along blockIdx.y: ceil(most entries an expert can have / entries per CTA)
    const float *bias;       // nullable: [experts][rows_per_expert], added to every output
    float *y;                // element [entry][col0 + row - row0], rows ldy apart
    int ldy, col0;
    DevState *state;
};

// One CTA = 128 rows of one expert against one chunk of up to NT of its entries (NT = 4, 8 or 16, MMA N = 4 NT; an
// expert with more entries is served by several CTAs, which re-read its rows from L2).
//
// Roles.  A tcgen05.mma or a bulk copy costs its issuing thread on the order of a hundred cycles, so the
// asynchronous work is spread: warp 4 is the producer (every lane copies 16-byte pieces of the pairs' weight
// units into a ring TL_DEPTH pairs deep),
// one thread each of warps 5 and 6 issues the two products of one block of every pair as soon as the
// workers have staged the operands.  Warps 0-3 are the workers, one
// thread per row: stage(q) decodes the row's 64 codes of pair q from the ring into half (q & 1) of the
// operand tiles, chains(p) reads the pair's accumulators from tensor memory and runs the float chains.
// A worker runs stage(p + 1) before chains(p), so the tensor core works on pair p + 1 meanwhile.
//
// Barriers (all waits bounded).  full[slot], 32 arrivals: the producer lanes' copies of the pair have landed;
// empty[slot], 128 arrivals: the workers have read it.  staged[half], 128 arrivals: the
// half's operands are written and, because a worker stages pair p + 2 only after chains(p), the half's
// accumulators have been read.  done[half], 2 arrivals: the issuers' tcgen05.commit of the pair; workers wait for it before they read
// the accumulators and before they overwrite the half's operands two pairs later.
template <int NT>
__global__ void __launch_bounds__(MT_THREADS, NT == 16 ? 2 : MT_CTAS) mx_tile_kernel(TileArgs a) {
    constexpr int N = 4 * NT;                                    // columns per block: NT tokens x 4 chain lanes
    constexpr uint32_t TMEM_COLS = 4 * N;                        // two halves x two blocks x N columns (64 or 128)
    constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((TL_ROWS >> 4) << 24);
    extern __shared__ __align__(128) unsigned char tsm[];
    const int nb = a.w.blocks, np = nb / 2;
    unsigned char (*a_tiles)[TL_A_BYTES] = reinterpret_cast<unsigned char (*)[TL_A_BYTES]>(tsm);           // [half][block of the pair][P, N]
    unsigned char (*b_tiles)[N * 32] = reinterpret_cast<unsigned char (*)[N * 32]>(tsm + 8 * TL_A_BYTES);  // [half][block of the pair]
    unsigned char *ring = tsm + 8 * TL_A_BYTES + 4 * N * 32;                                               // [TL_DEPTH][8 units]
    float *xs_sm = reinterpret_cast<float *>(ring + TL_DEPTH * TL_SLOT);                                   // [NT][nb] activation block scales
    __shared__ float tbl[256];
    __shared__ __align__(8) uint64_t full[TL_DEPTH], empty[TL_DEPTH], staged[2], done[2];
    __shared__ uint32_t tmem_base_sh;
    __shared__ int ent[NT];
    const int tid = threadIdx.x, warp = tid >> 5;
    const int e = blockIdx.y / a.chunks, chunk = blockIdx.y % a.chunks;
    const int n_ent = min((a.cnt ? a.cnt[e] : a.ntok) - chunk * NT, NT);
    if (n_ent <= 0) return;                      // nothing routed here (before anything is allocated)
    if (tid < NT) ent[tid] = tid < n_ent ? (a.list ? a.list[e * TL_MAXTOK + chunk * NT + tid] : chunk * NT + tid) : 0;
    mx_fill_scale_table(tbl, tid, MT_THREADS);
    for (int i = tid; i < 4 * N * 32 / 16; i += MT_THREADS) reinterpret_cast<uint4 *>(&b_tiles[0][0])[i] = make_uint4(0, 0, 0, 0);   // rows of absent tokens stay zero
    if (tid == 0) {
        for (int i = 0; i < TL_DEPTH; i++) { mbar_init(&full[i], 32); mbar_init(&empty[i], 128); }
        mbar_init(&staged[0], 128); mbar_init(&staged[1], 128);
        mbar_init(&done[0], MT_ISSUERS); mbar_init(&done[1], MT_ISSUERS);
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tl_fence_before();
    __syncthreads();
    tl_fence_after();
    const uint32_t tmem_base = tmem_base_sh;
    uint32_t *err = a.state ? &a.state->err : nullptr;
    Waiter waiter(err);
    // the tile's live rows lie in up to nine units of 16 rows (a row window may start anywhere); only those are copied
    const int row_base = e * a.rows_per_expert + a.row0 + blockIdx.x * TL_ROWS;
    const int live_rows = min(TL_ROWS, a.nrows - (int)blockIdx.x * TL_ROWS);
    const int n_units = ((row_base & 15) + live_rows + 15) >> 4;

    if (warp == 4) {
        // ---------------- producer: 16-byte asynchronous copies, one arrival per lane on the slot's barrier
        const int lane = tid & 31;
        const int n_chunks = n_units * (MX_UNIT / 16);
        const unsigned char *wbase = a.w.data + mx_unit_off(row_base >> 4, 0, np);
        uint32_t src_off[TL_CPL], dst_off[TL_CPL];          // this lane's chunks of a pair: unit g, 16-byte piece o
#pragma unroll
        for (int i = 0; i < TL_CPL; i++) {
            const int c = lane + 32 * i, g = c / (MX_UNIT / 16), o = (c - g * (MX_UNIT / 16)) * 16;
            src_off[i] = (uint32_t)g * (uint32_t)np * MX_UNIT + o;
            dst_off[i] = (uint32_t)(g * MX_UNIT + o);
        }
        auto load = [&](int q, int slot) {
            const unsigned char *src = wbase + (size_t)q * MX_UNIT;
            unsigned char *dst = ring + slot * TL_SLOT;
#pragma unroll
            for (int i = 0; i < TL_CPL; i++)
                if (lane + 32 * i < n_chunks)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst + dst_off[i])), "l"(src + src_off[i]) : "memory");
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[slot])) : "memory");
        };
        const int pre = min(TL_DEPTH, np);
        for (int q = 0; q < pre; q++) load(q, q);
        int slot = 0;
        uint32_t par = 0;
        for (int p = 0; p + TL_DEPTH < np; p++) {
            waiter.wait_suspended(&empty[slot], par);                              // every worker has read pair p out of the slot
            load(p + TL_DEPTH, slot);
            if (++slot == TL_DEPTH) { slot = 0; par ^= 1u; }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (tid == 160 || (MT_ISSUERS == 2 && tid == 192)) {
        // ---------------- issuer(s): with two, block k of every pair each (two threads in two warps issue side by side); with one, both blocks
        const int k0 = tid == 160 ? 0 : 1, k1 = MT_ISSUERS == 2 ? k0 + 1 : 2;
        uint64_t da[2][4], db[2][2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
#pragma unroll
            for (int i = 0; i < 4; i++) da[h][i] = tl_smem_desc(&a_tiles[4 * h + i][0], 2048);
            db[h][0] = tl_smem_desc(&b_tiles[2 * h][0], N * 16);
            db[h][1] = tl_smem_desc(&b_tiles[2 * h + 1][0], N * 16);
        }
        for (int p = 0; p < np; p++) {
            const int h = p & 1;
            waiter.wait_suspended(&staged[h], (uint32_t)(p >> 1) & 1u);
            tl_fence_after();
#pragma unroll
            for (int k = 0; k < 2; k++)
                if (k >= k0 && k < k1) {
                    const uint32_t dcol = tmem_base + (uint32_t)((2 * h + k) * N);
                    if (h == 0) { tl_mma(dcol, da[0][2 * k], db[0][k], 0u, IDESC); tl_mma(dcol, da[0][2 * k + 1], db[0][k], 1u, IDESC); }
                    else        { tl_mma(dcol, da[1][2 * k], db[1][k], 0u, IDESC); tl_mma(dcol, da[1][2 * k + 1], db[1][k], 1u, IDESC); }
                }
            tl_commit(&done[h]);
        }
    } else if (tid < 128) {
        // ---------------- workers
        const uint32_t P_LO = 0x04030200u, P_HI = 0x0D090705u, N_LO = 0xFDFEFF00u, N_HI = 0xF4F8FAFCu;
        const int row_local = blockIdx.x * TL_ROWS + tid;
        const bool row_live = tid < live_rows;
        // this row in a ring slot: its unit, there its 32 code bytes of the pair and its two exponent bytes
        const int urow = (row_base & 15) + tid;
        const unsigned char *my_unit = ring + (urow >> 4) * MX_UNIT;
        const uint32_t w_off = (uint32_t)(urow & 15) * 32, e_off = MX_UNIT_EXPS + (uint32_t)(urow & 15) * 2;
        // A element (row m, byte k) lives at (k / 16) * 2048 + (m / 8) * 128 + (m % 8) * 16 + k % 16
        const uint32_t a_off = (uint32_t)((tid >> 3) * 128 + (tid & 7) * 16);
        // B row n = token * 4 + lane holds the 8 activation bytes of `lane` at k = 8 * lane .. + 7; threads 0 .. N - 1 serve
        // the first block of the pair, 64 .. 64 + N - 1 the second
        const int n_row = tid & 63, bt = n_row >> 2, bl = tid & 3, bblk = tid >> 6;
        const bool b_live = n_row < N && bt < n_ent;
        const uint32_t b_off = (uint32_t)((bl >> 1) * (N * 16) + (n_row >> 3) * 128 + (n_row & 7) * 16 + (bl & 1) * 8);
        // its activation words come straight from global memory (L2), one pair ahead
        const int8_t *my_x = a.xq + (size_t)(ent[b_live ? bt : 0] / a.src_div) * nb * 32 + bblk * 32 + 4 * bl;
        uint32_t xlo = 0, xhi = 0;
        if (b_live) { xlo = *reinterpret_cast<const uint32_t *>(my_x); xhi = *reinterpret_cast<const uint32_t *>(my_x + 16); }
        for (int i = tid; i < n_ent * nb; i += 128) xs_sm[i] = a.xs[(size_t)(ent[i / nb] / a.src_div) * nb + i % nb];
        asm volatile("bar.sync 1, 128;" ::: "memory");             // the workers' own barrier: xs_sm is complete

        int f_slot = 0;
        uint32_t f_par = 0;
        // operands of pair q -> half (q & 1) of the tiles; returns the row's two exponent bytes
        auto stage = [&](int q) -> uint32_t {
            const int h = q & 1;
            waiter.wait_suspended(&full[f_slot], f_par);
            const unsigned char *u = my_unit + f_slot * TL_SLOT;
            const int q_slot = f_slot;
            if (++f_slot == TL_DEPTH) { f_slot = 0; f_par ^= 1u; }
            const uint4 w0 = *reinterpret_cast<const uint4 *>(u + w_off), w1 = *reinterpret_cast<const uint4 *>(u + w_off + 16);
            const uint32_t e2 = *reinterpret_cast<const unsigned short *>(u + e_off);
            mbar_arrive(&empty[q_slot]);
            const uint32_t wl[4][2] = {{w0.x, w0.y}, {w0.z, w0.w}, {w1.x, w1.y}, {w1.z, w1.w}};
            // lanes (0, 1) and (2, 3) of a row are neighbours in the tile: one 16-byte store per (K half, block, table); a warp's
            // stores then cover 512 contiguous bytes (no bank conflict)
#pragma unroll
            for (int jh = 0; jh < 2; jh++) {
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const uint32_t wa = wl[2 * jh][k], wb = wl[2 * jh + 1][k], wax = wa ^ 0x88888888u, wbx = wb ^ 0x88888888u;
                    const uint32_t off = (uint32_t)(jh * 2048) + a_off;
                    *reinterpret_cast<uint4 *>(&a_tiles[4 * h + 2 * k][off]) =
                        make_uint4(brrr_prmt(P_LO, P_HI, wa), brrr_prmt(P_LO, P_HI, wa >> 16), brrr_prmt(P_LO, P_HI, wb), brrr_prmt(P_LO, P_HI, wb >> 16));
                    *reinterpret_cast<uint4 *>(&a_tiles[4 * h + 2 * k + 1][off]) =
                        make_uint4(brrr_prmt(N_LO, N_HI, wax), brrr_prmt(N_LO, N_HI, wax >> 16), brrr_prmt(N_LO, N_HI, wbx), brrr_prmt(N_LO, N_HI, wbx >> 16));
                }
            }
            if (b_live) {
                const int2 iv = mx_interleave(xlo, xhi);
                *reinterpret_cast<uint2 *>(&b_tiles[2 * h + bblk][b_off]) = make_uint2((uint32_t)iv.x, (uint32_t)iv.y);
                if (q + 1 < np) {
                    xlo = *reinterpret_cast<const uint32_t *>(my_x + (size_t)(q + 1) * 64);
                    xhi = *reinterpret_cast<const uint32_t *>(my_x + (size_t)(q + 1) * 64 + 16);
                }
            }
            fence_proxy_async();               // generic-proxy writes above -> visible to the tensor core's reads
            tl_fence_before();                 // and this thread's reads of the half's accumulators are done
            mbar_arrive(&staged[h]);
            return e2;
        };
        // the chains of lanes (0, 1) and (2, 3) of an entry share an instruction (fma.rn.f32x2: two independent
        // round-to-nearest fused multiply-adds)
        unsigned long long acc2[N / 2];
#pragma unroll
        for (int i = 0; i < N / 2; i++) acc2[i] = 0ull;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        // float chains of pair p: thread = row (tensor-memory lane), N columns per block
        auto chains = [&](int p, uint32_t e2c) {
            const int h = p & 1;
            waiter.wait_suspended(&done[h], (uint32_t)(p >> 1) & 1u);
            tl_fence_after();
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const float esc = tbl[k ? e2c >> 8 : e2c & 0xFFu];
                constexpr int G = N > 32 ? 32 : N;                // columns per tensor-memory read round (registers)
#pragma unroll
                for (int c0 = 0; c0 < N; c0 += G) {
                    int d[G / 16][16];
#pragma unroll
                    for (int c = 0; c < G / 16; c++) tl_ld16(lane_addr + (uint32_t)((2 * h + k) * N + c0 + 16 * c), d[c]);
                    tl_wait_ld();
#pragma unroll
                    for (int tt = 0; tt < G / 4; tt++) {
                        const int t = c0 / 4 + tt;
                        const float sxs = __fmul_rn(esc, xs_sm[t * nb + 2 * p + k]);
                        const unsigned long long s2 = tl_pack2(sxs, sxs);
#pragma unroll
                        for (int l = 0; l < 2; l++)
                            acc2[2 * t + l] = tl_fma2(tl_pack2((float)d[tt / 4][4 * (tt % 4) + 2 * l], (float)d[tt / 4][4 * (tt % 4) + 2 * l + 1]), s2, acc2[2 * t + l]);
                    }
                }
            }
        };
        uint32_t e2c = stage(0);
        for (int p = 0; p < np; p++) {
            uint32_t e2n = 0;
            if (p + 1 < np) e2n = stage(p + 1);      // the tensor core runs pair p + 1 ...
            chains(p, e2c);                          // ... beside the chains of pair p
            e2c = e2n;
        }
        if (row_live) {
            const float bias = a.bias ? a.bias[(size_t)e * a.rows_per_expert + a.row0 + row_local] : 0.0f;
#pragma unroll
            for (int t = 0; t < NT; t++)
                if (t < n_ent) {
                    float a0, a1, a2, a3;
                    tl_unpack2(acc2[2 * t], a0, a1);
                    tl_unpack2(acc2[2 * t + 1], a2, a3);
                    float v = __fadd_rn(__fadd_rn(a0, a1), __fadd_rn(a2, a3));
                    if (a.bias) v = __fadd_rn(v, bias);
                    a.y[(size_t)ent[t] * a.ldy + a.col0 + row_local] = v;
                }
        }
    }
    tl_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
}

// ---------------------------------------------------------------- Q8 matrix x token rows (dense projections of a tile)
// The Q8 row dot (dot_q8_i8, src/bin/engine_gpt2.rs:169-191) is 2 block parities x 4 lanes of chains,
// chain (p, j) accumulating fma(float(t_j(b)), w_scale[b] * xs[b], acc) over the blocks b of parity p, t_j(b) the
// exact integer dot of the lane's 8 weights with its 8 activation bytes; the row is (e0 + e1) + (e2 + e3) with
// e_j = acc[0][j] + acc[1][j].  The weights are int8 already, so the producer warp copies the 16-byte pieces of a
// unit straight to their place in the K-major operand tile and no thread decodes anything: one product per block
// (128 rows x 16 columns x 32), workers = entry staging + chains.  One CTA = 128 matrix rows x up to 4 token rows.
constexpr int QT_DEPTH = 4;
constexpr int QT_STAGE = 2 * TL_A_BYTES + TL_ROWS * 8;      // two operand tiles (the pair's blocks) + [128 rows][2] f32 block scales

struct Q8TileArgs {
    Q8Dev m;
    const int8_t *xq;       // [token rows][cols]
    const float *xs;        // [token rows][cols / 32]
    const float *bias;
    float *y;               // [token rows][ldy]
    int ntok, ldy;
    DevState *state;
};

template <int EPI, int NT>
__global__ void __maxnreg__(96) q8_tile_kernel(Q8TileArgs a) {      // 96 registers: three CTAs of 7 warps (TL_THREADS) per SM
    constexpr int N = 4 * NT;
    constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((TL_ROWS >> 4) << 24);
    constexpr uint32_t TMEM_COLS = 4 * N;
    extern __shared__ __align__(128) unsigned char tsm[];
    const int np = a.m.cols / 64, nb = np * 2;
    unsigned char *ring = tsm;                                                                                  // [QT_DEPTH][QT_STAGE]
    unsigned char (*b_tiles)[N * 32] = reinterpret_cast<unsigned char (*)[N * 32]>(tsm + QT_DEPTH * QT_STAGE);  // [half][block of the pair]
    float *xs_sm = reinterpret_cast<float *>(tsm + QT_DEPTH * QT_STAGE + 4 * N * 32);                           // [NT][nb]
    __shared__ __align__(8) uint64_t full[QT_DEPTH], empty[QT_DEPTH], staged[2], done[2];
    __shared__ uint32_t tmem_base_sh;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int t_first = blockIdx.y * NT, n_ent = min(a.ntok - t_first, NT);
    for (int i = tid; i < 4 * N * 32 / 16; i += TL_THREADS) reinterpret_cast<uint4 *>(&b_tiles[0][0])[i] = make_uint4(0, 0, 0, 0);   // rows of absent tokens stay zero
    if (tid == 0) {
        for (int i = 0; i < QT_DEPTH; i++) { mbar_init(&full[i], 32); mbar_init(&empty[i], 130); }
        mbar_init(&staged[0], 128); mbar_init(&staged[1], 128);
        mbar_init(&done[0], 2); mbar_init(&done[1], 2);
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tl_fence_before();
    __syncthreads();
    tl_fence_after();
    const uint32_t tmem_base = tmem_base_sh;
    uint32_t *err = a.state ? &a.state->err : nullptr;
    Waiter waiter(err);
    const int urow0 = blockIdx.x * (TL_ROWS / 16);
    const int n_units = min(TL_ROWS / 16, q8_urows(a.m.rows) - urow0);

    if (warp == 4) {
        // ---------------- producer: the weights are static, so the ring fills before the dependency wait
        const int lane = tid & 31;
        const unsigned char *wbase = a.m.data + q8_unit_off(urow0, 0, np);
        const uint32_t unit_stride = (uint32_t)np * Q8_UNIT;
        // this lane's pieces of a pair, offsets recomputed per copy (the producer has time; registers are the workers')
        auto load = [&](int q, int slot) {
            const unsigned char *src = wbase + (size_t)q * Q8_UNIT;
            unsigned char *dst = ring + slot * QT_STAGE;
#pragma unroll 4
            for (int i = 0; i < 16; i++) {                       // operand pieces: (unit g, row rl, block p, half kh) -> tile p, K half kh, row m
                const int idx = lane + 32 * i, kh = idx & 1, pp = (idx >> 1) & 1, rl = (idx >> 2) & 15, g = idx >> 6, m = g * 16 + rl;
                if (g < n_units)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst + pp * TL_A_BYTES + kh * 2048 + (m >> 3) * 128 + (m & 7) * 16)),
                                 "l"(src + g * unit_stride + rl * 64 + pp * 32 + kh * 16) : "memory");
            }
#pragma unroll
            for (int i = 0; i < 2; i++) {                        // block scales: 128 bytes per unit
                const int idx = lane + 32 * i, g = idx >> 3, part = idx & 7;
                if (g < n_units)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst + 2 * TL_A_BYTES + g * 128 + part * 16)),
                                 "l"(src + g * unit_stride + Q8_UNIT_SCALES + part * 16) : "memory");
            }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[slot])) : "memory");
        };
        const int pre = min(QT_DEPTH, np);
        for (int q = 0; q < pre; q++) load(q, q);
        pdl_wait();
        pdl_trigger();
        int slot = 0;
        uint32_t par = 0;
        for (int p = 0; p + QT_DEPTH < np; p++) {
            waiter.wait_suspended(&empty[slot], par);                    // the products of pair p are complete and its scales read
            load(p + QT_DEPTH, slot);
            if (++slot == QT_DEPTH) { slot = 0; par ^= 1u; }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (tid == 160 || tid == 192) {
        // ---------------- issuers: block k of every pair
        pdl_wait();
        pdl_trigger();
        const int k = tid == 160 ? 0 : 1;
        const uint64_t da0 = tl_smem_desc(ring + k * TL_A_BYTES, 2048);
        const uint64_t db[2] = {tl_smem_desc(&b_tiles[k][0], N * 16), tl_smem_desc(&b_tiles[2 + k][0], N * 16)};
        int slot = 0;
        for (int p = 0; p < np; p++) {
            const int h = p & 1;
            waiter.wait_suspended(&staged[h], (uint32_t)(p >> 1) & 1u);    // every worker has seen the pair's weights land and staged its entries
            tl_fence_after();
            tl_mma(tmem_base + (uint32_t)((2 * h + k) * N), da0 + (uint64_t)(slot * (QT_STAGE / 16)), h ? db[1] : db[0], 0u, IDESC);
            tl_commit(&done[h]);
            tl_commit(&empty[slot]);
            if (++slot == QT_DEPTH) slot = 0;
        }
    } else if (tid < 128) {
        // ---------------- workers: thread = matrix row of the tile
        pdl_wait();
        pdl_trigger();
        const int row = blockIdx.x * TL_ROWS + tid;
        const bool row_live = row < a.m.rows;
        const int n_row = tid & 63, bt = n_row >> 2, bl = tid & 3, bblk = tid >> 6;
        const bool b_live = n_row < N && bt < n_ent;
        // B row n = token * 4 + lane: the lane's 8 activation bytes (positions 4 lane .. + 3 and 16 + 4 lane .. + 3, the order of the unit) at k = 8 lane .. + 7
        const uint32_t b_off = (uint32_t)((bl >> 1) * (N * 16) + (n_row >> 3) * 128 + (n_row & 7) * 16 + (bl & 1) * 8);
        const int8_t *my_x = a.xq + (size_t)(t_first + (b_live ? bt : 0)) * a.m.cols + bblk * 32 + 4 * bl;
        uint32_t xlo = 0, xhi = 0;
        if (b_live) { xlo = *reinterpret_cast<const uint32_t *>(my_x); xhi = *reinterpret_cast<const uint32_t *>(my_x + 16); }
        for (int i = tid; i < n_ent * nb; i += 128) xs_sm[i] = a.xs[(size_t)t_first * nb + i];
        float bias_pre = 0.0f;
        if (row_live && (EPI == Q8_EPI_BIAS || EPI == Q8_EPI_RESID_BIAS)) bias_pre = a.bias[row];
        asm volatile("bar.sync 1, 128;" ::: "memory");             // the workers' own barrier: xs_sm is complete
        int f_slot = 0;
        uint32_t f_par = 0;
        auto stage = [&](int q) -> float2 {
            const int h = q & 1;
            waiter.wait_suspended(&full[f_slot], f_par);
            const float2 sc = *reinterpret_cast<const float2 *>(ring + f_slot * QT_STAGE + 2 * TL_A_BYTES + tid * 8);
            const int q_slot = f_slot;
            if (++f_slot == QT_DEPTH) { f_slot = 0; f_par ^= 1u; }
            if (b_live) {
                *reinterpret_cast<uint2 *>(&b_tiles[2 * h + bblk][b_off]) = make_uint2(xlo, xhi);
                if (q + 1 < np) {
                    xlo = *reinterpret_cast<const uint32_t *>(my_x + (size_t)(q + 1) * 64);
                    xhi = *reinterpret_cast<const uint32_t *>(my_x + (size_t)(q + 1) * 64 + 16);
                }
            }
            fence_proxy_async();               // generic-proxy writes (these, and the producer's copies seen through full[]) -> the tensor core's reads
            tl_fence_before();                 // this thread's reads of the half's accumulators are done
            mbar_arrive(&staged[h]);
            mbar_arrive(&empty[q_slot]);
            return sc;
        };
        float acc[2][N];
#pragma unroll
        for (int i = 0; i < N; i++) { acc[0][i] = 0.0f; acc[1][i] = 0.0f; }
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        auto chains = [&](int p, float2 sc) {
            const int h = p & 1;
            waiter.wait_suspended(&done[h], (uint32_t)(p >> 1) & 1u);
            tl_fence_after();
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const float ws = k ? sc.y : sc.x;
#pragma unroll
                for (int c = 0; c < N / 16; c++) {             // 16 columns = four token rows at a time (registers)
                    int d[16];
                    tl_ld16(lane_addr + (uint32_t)((2 * h + k) * N + 16 * c), d);
                    tl_wait_ld();
#pragma unroll
                    for (int t = 0; t < 4; t++) {
                        const float sxs = __fmul_rn(ws, xs_sm[(4 * c + t) * nb + 2 * p + k]);
#pragma unroll
                        for (int l = 0; l < 4; l++) acc[k][16 * c + 4 * t + l] = __fmaf_rn((float)d[4 * t + l], sxs, acc[k][16 * c + 4 * t + l]);
                    }
                }
            }
        };
        float2 scc = stage(0);
        for (int p = 0; p < np; p++) {
            float2 scn = make_float2(0.0f, 0.0f);
            if (p + 1 < np) scn = stage(p + 1);
            chains(p, scc);
            scc = scn;
        }
        if (row_live) {
#pragma unroll
            for (int t = 0; t < NT; t++)
                if (t < n_ent) {
                    const float e0 = __fadd_rn(acc[0][4 * t], acc[1][4 * t]), e1 = __fadd_rn(acc[0][4 * t + 1], acc[1][4 * t + 1]);
                    const float e2 = __fadd_rn(acc[0][4 * t + 2], acc[1][4 * t + 2]), e3 = __fadd_rn(acc[0][4 * t + 3], acc[1][4 * t + 3]);
                    const float r = __fadd_rn(__fadd_rn(e0, e1), __fadd_rn(e2, e3));
                    float *yp = a.y + (size_t)(t_first + t) * a.ldy + row;
                    if (EPI == Q8_EPI_PLAIN) *yp = r;
                    else if (EPI == Q8_EPI_BIAS) *yp = __fadd_rn(r, bias_pre);
                    else *yp = __fadd_rn(*yp, __fadd_rn(r, bias_pre));                // x += dot + bias
                }
        }
    } else {
        pdl_wait();
        pdl_trigger();
    }
    tl_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
}

// Per expert, the (token, slot) pairs routed to it, in ascending order: entry = token * topk + slot.  One CTA per
// expert, thread = token (a token routes to an expert at most once, so the order is the token order).
__global__ void __launch_bounds__(TL_MAXTOK) tile_route_kernel(const int32_t *__restrict__ top, int ntok, int topk, int *__restrict__ cnt, int *__restrict__ list) {
    __shared__ int warp_cnt[TL_MAXTOK / 32];
    const int e = blockIdx.x, t = threadIdx.x;
    int slot = -1;
    if (t < ntok)
        for (int s = 0; s < topk; s++)
            if (top[t * 8 + s] == e) { slot = s; break; }
    const unsigned m = __ballot_sync(0xffffffffu, slot >= 0);
    if ((t & 31) == 0) warp_cnt[t >> 5] = __popc(m);
    __syncthreads();
    int before = __popc(m & ((1u << (t & 31)) - 1u));
    for (int w = 0; w < (t >> 5); w++) before += warp_cnt[w];
    if (slot >= 0) list[e * TL_MAXTOK + before] = t * topk + slot;
    if (t == TL_MAXTOK - 1) cnt[e] = before + (slot >= 0 ? 1 : 0);
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

size_t tl_smem(int nt, int nb) { return 8 * TL_A_BYTES + 4 * (size_t)(4 * nt) * 32 + (size_t)TL_DEPTH * TL_SLOT + (size_t)nt * nb * 4; }

// Block pairs need an even block count.  Entries per CTA: 4 while no expert can have more than 16 entries, 8 up to 64, else 16.
cudaError_t tl_launch(TileArgs a, int tiles, int experts, int max_entries, cudaStream_t st) {
    if ((a.w.blocks & 1) || a.w.blocks < 2 || max_entries < 1 || max_entries > TL_MAXTOK) return cudaErrorInvalidValue;
    static const int wide_from = [] { const char *e = getenv("BRRR_TILE_NT16_FROM"); const int v = e ? atoi(e) : 0; return v >= 1 ? v : MT_NT16_FROM; }();
    const int nt = max_entries <= 16 ? 4 : max_entries < wide_from ? 8 : 16;
    const size_t smem = tl_smem(nt, a.w.blocks);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    static unsigned long long configured4 = 0, configured8 = 0, configured16 = 0;      // one bit per device
    cudaError_t ce = nt == 4 ? smem_optin(mx_tile_kernel<4>, 200 * 1024, configured4)
                   : nt == 8 ? smem_optin(mx_tile_kernel<8>, 200 * 1024, configured8) : smem_optin(mx_tile_kernel<16>, 200 * 1024, configured16);
    if (ce != cudaSuccess) return ce;
    a.chunks = (max_entries + nt - 1) / nt;
    const dim3 grid(tiles, experts * a.chunks);
    if (nt == 4) mx_tile_kernel<4><<<grid, MT_THREADS, smem, st>>>(a);
    else if (nt == 8) mx_tile_kernel<8><<<grid, MT_THREADS, smem, st>>>(a);
    else mx_tile_kernel<16><<<grid, MT_THREADS, smem, st>>>(a);
    return cudaGetLastError();
}

template <int EPI, int NT>
cudaError_t q8_tile_launch(const Q8TileArgs &a, bool pdl, cudaStream_t st) {
    static unsigned long long configured = 0;      // one bit per device
    cudaError_t e = smem_optin(q8_tile_kernel<EPI, NT>, 100 * 1024, configured);
    if (e != cudaSuccess) return e;
    const size_t smem = (size_t)QT_DEPTH * QT_STAGE + 4 * (4 * NT) * 32 + (size_t)NT * (a.m.cols / 32) * 4;
    if (smem > 100 * 1024) return cudaErrorInvalidValue;
    const dim3 grid((unsigned)((a.m.rows + TL_ROWS - 1) / TL_ROWS), (unsigned)((a.ntok + NT - 1) / NT));
    return launch_k(q8_tile_kernel<EPI, NT>, grid, dim3(TL_THREADS), smem, st, pdl, a);
}

}  // namespace

// y[t][r] (+)= row r of m . activation t (+ bias) on the tensor cores, t < ntok <= BRRR_TILE_MAX: bit-identical to the
// integer-unit kernels (kernels_q8.cu, kernels_rows.cu).  Four token rows per CTA up to 4 rows, eight beyond.
cudaError_t launch_q8_tile(Q8Dev m, const int8_t *xq, const float *xs, int ntok, const float *bias, float *y, int ldy, int epi, DevState *state,
                           bool pdl, cudaStream_t st) {
    if (ntok < 1 || ntok > BRRR_TILE_MAX || m.cols % 64 || m.cols < 64) return cudaErrorInvalidValue;
    Q8TileArgs a{m, xq, xs, bias, y, ntok, ldy, state};
    const bool wide = ntok > 4;
    switch (epi) {
    case Q8_EPI_PLAIN: return wide ? q8_tile_launch<Q8_EPI_PLAIN, 8>(a, pdl, st) : q8_tile_launch<Q8_EPI_PLAIN, 4>(a, pdl, st);
    case Q8_EPI_BIAS: return wide ? q8_tile_launch<Q8_EPI_BIAS, 8>(a, pdl, st) : q8_tile_launch<Q8_EPI_BIAS, 4>(a, pdl, st);
    case Q8_EPI_RESID_BIAS: return wide ? q8_tile_launch<Q8_EPI_RESID_BIAS, 8>(a, pdl, st) : q8_tile_launch<Q8_EPI_RESID_BIAS, 4>(a, pdl, st);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_mx_tile(MxDev w, int row0, int nrows, const int8_t *xq, const float *xs, int ntok, float *y, int ldy, DevState *state,
                           cudaStream_t st) {
    TileArgs a{};
    a.w = w; a.row0 = row0; a.nrows = nrows; a.src_div = 1; a.xq = xq; a.xs = xs; a.ntok = ntok; a.y = y; a.ldy = ldy; a.state = state;
    return tl_launch(a, (nrows + TL_ROWS - 1) / TL_ROWS, 1, ntok, st);
}

// All experts of one matrix kind against their routed entries (see TileArgs).
cudaError_t launch_mx_tile_experts(MxDev w, int ne, int rows_per_expert, const int *cnt, const int *list, int max_entries, int src_div, const int8_t *xq,
                                   const float *xs, const float *bias, float *y, int ldy, int col0, DevState *state, cudaStream_t st) {
    TileArgs a{};
    a.w = w; a.row0 = 0; a.nrows = rows_per_expert; a.rows_per_expert = rows_per_expert; a.cnt = cnt; a.list = list; a.src_div = src_div;
    a.xq = xq; a.xs = xs; a.bias = bias; a.y = y; a.ldy = ldy; a.col0 = col0; a.state = state;
    return tl_launch(a, (rows_per_expert + TL_ROWS - 1) / TL_ROWS, ne, max_entries, st);
}

void launch_tile_route(const int32_t *top, int ntok, int topk, int ne, int *cnt, int *list, cudaStream_t st) {
    tile_route_kernel<<<ne, TL_MAXTOK, 0, st>>>(top, ntok, topk, cnt, list);
}

void launch_tile_combine(const float *part, const float *wts, int topk, int d, int ntok, float *x, cudaStream_t st) {
    tile_combine_kernel<<<dim3((d + 255) / 256, ntok), 256, 0, st>>>(part, wts, topk, d, x);
}

}  // namespace brrr
