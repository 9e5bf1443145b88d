// Single-token MXFP4 expert matvecs on the 5th-generation tensor cores in their native 4-bit format
// (tcgen05.mma kind::mxf4.block_scale): the e2m1 codes of the GGUF blocks are the tensor-core operand
// as they are, so the weight bytes go from HBM to shared memory by bulk copy and from there straight
// into the MMA, with no decode instructions at all.
//
// Arithmetic (bit-identical to the integer-unit kernels of kernels_mx.cu).  A row's value is four
// lane chains, chain j accumulating fma(float(t_j(b)), 2^(e_b-128) * xs[b], acc) over the 32-blocks
// b, where t_j(b) is the exact integer dot of the lane's 8 doubled e2m1 values with the lane's 8
// activation bytes.  The tensor core supplies t_j(b):
//   * an activation byte x in [-127, 127] is written as 49 a + 7 b + c with digits in [-3, 3];
//     twice a digit (0, +-2, +-4, +-6) is an e2m1 value, and (true e2m1 value) x (twice the digit)
//     = (doubled e2m1 value) x digit, so the three digit planes give three exact partial sums;
//   * one MMA covers a block pair (K = 64): operand A = 128 weight rows x 64 codes, operand B = 24
//     columns (digit plane t, block of the pair q, lane j), each holding the plane's codes of the 8
//     positions of lane j in block q and zero elsewhere; all block scales are 1 (ue8m0 0x7F);
//   * every product and partial sum is a small dyadic number (|sum| <= 8 * 12 * 3), exact in the
//     f32 accumulator, and t_j(b) = fma(D_a, 49, fma(D_b, 7, D_c)) is exact as well.
// The four epilogue warps read the 24 accumulator columns of their rows from tensor memory
// (tcgen05.ld) and run the float chains, one thread per row.
//
// Layout ("tile units").  A tile is 128 matrix rows; its unit for block pair p is the 4096-byte
// shared-memory image of operand A in the canonical K-major no-swizzle layout (16-byte chunk of
// (row m, block q) at q * 2048 + (m / 8) * 128 + (m % 8) * 16, the chunk being the 16 nibble bytes
// of the GGUF block) followed by 128 x 2 e8m0 bytes.  The units of a tile are contiguous, so any run
// of them is one bulk copy.  Gate and up share tiles (rows 0-63 gate, 64-127 up, same 64 outputs),
// so the SwiGLU and the Q8 quantiser of h run in the same CTA.
//
// Operand B (brrr_mxt.cuh) is written once per activation by the kernel that quantises it (the
// routing-estimate kernel for the token, the gate/up epilogue for h) and bulk-copied by every CTA.
//
// Pipeline per CTA: warp 4 issues the bulk copies into a ring of stages, one thread of warp 5 issues
// the MMAs into a ring of 8 accumulator regions of tensor memory, warps 0-3 drain them two pairs at
// a time with the next loads in flight.  Every wait is bounded.
#include "brrr_kernels.h"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"
#include "brrr_mx.cuh"
#include "brrr_mxt.cuh"

namespace brrr {

namespace {

constexpr int XT_CH = 4;                 // block pairs per ring stage = per round of the pipeline
constexpr int XT_REGION_COLS = XT_CH * XT_N;   // accumulator region = one round = 96 tensor-memory columns
constexpr int XT_REGIONS = 2;
constexpr uint32_t XT_TMEM_COLS = 256;   // 2 regions + 64 columns of unit scale factors
constexpr int XT_SF_COL = XT_REGIONS * XT_REGION_COLS;
constexpr int XT_THREADS = 192;
#ifdef BRRR_TEST_HOOKS
#define XT_T0() long long xt_t0_ = clock64()
#define XT_ACC(v) do { long long xt_t1_ = clock64(); (v) += xt_t1_ - xt_t0_; xt_t0_ = xt_t1_; } while (0)
#define XT_STAMP(state, i) do { if ((state) && blockIdx.x == BRRR_STAMP_BX && blockIdx.y == 0) (state)->stamps[i] = clock64(); } while (0)
#else
#define XT_T0() do { } while (0)
#define XT_ACC(v) do { } while (0)
#define XT_STAMP(state, i) do { } while (0)
#endif

// ---------------------------------------------------------------- pack: 16-row units -> tile units
struct PackArgs {
    MxDev a, b;              // b.data == nullptr: one matrix, 128 rows per tile; else rows 0-63 from a, 64-127 from b
    int rows_per_expert;     // logical rows of one expert in a (and b)
    int tiles_per_expert;
    MxtDev out;
};

__global__ void mxt_pack_kernel(PackArgs p, size_t total_words) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total_words) return;
    // word index within the destination: [tile][pair][1024 words of operand A | 64 words of exponents]
    const int np = p.out.np;
    const size_t unit = idx / (MXT_UNIT / 4);
    const int w = (int)(idx % (MXT_UNIT / 4));
    const int pair = (int)(unit % np);
    const size_t tile = unit / np;
    const int e = (int)(tile / p.tiles_per_expert), t = (int)(tile % p.tiles_per_expert);
    // source unit and row within it of tile row m; nullptr for rows past the end of the matrix
    auto locate = [&](int m, int &rl) -> const uint8_t * {
        const MxDev &mat = (p.b.data && m >= 64) ? p.b : p.a;
        const int r = p.b.data ? t * 64 + (m & 63) : t * 128 + m;
        if (r >= p.rows_per_expert) return nullptr;
        const int row = e * p.rows_per_expert + r;
        rl = row & 15;
        return mat.data + mx_unit_off(row >> 4, pair, np);
    };
    uint32_t v = 0;
    if (w < 1024) {
        const int q = w >> 9, rem = w & 511, m = (rem >> 5) * 8 + ((rem >> 2) & 7), j = rem & 3;
        int rl = 0;
        const uint8_t *u = locate(m, rl);
        if (u) v = *reinterpret_cast<const uint32_t *>(u + rl * 32 + j * 8 + q * 4);
    } else {
        for (int k = 0; k < 2; k++) {                 // rows m0, m0 + 1: two exponent bytes each
            int rl = 0;
            const uint8_t *u = locate((w - 1024) * 2 + k, rl);
            if (u) v |= (uint32_t)*reinterpret_cast<const unsigned short *>(u + MX_UNIT_EXPS + rl * 2) << (16 * k);
        }
    }
    reinterpret_cast<uint32_t *>(p.out.data + unit * MXT_UNIT)[w] = v;
}

// ---------------------------------------------------------------- tensor-core plumbing
// shared-memory matrix descriptor: K-major, no swizzle; core matrix = 8 rows x 16 bytes, 128 bytes
// apart along M/N, `lbo` bytes apart along K
// block-scaled instruction descriptor: A = B = e2m1 (format 1), both K-major, N / 8 at bit 17,
// ue8m0 scales (bit 23), M / 16 at bit 24, scale-factor ids 0, K = 64
constexpr uint32_t XT_IDESC = (1u << 7) | (1u << 10) | ((uint32_t)(XT_N >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);

__device__ __forceinline__ void xt_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(XT_IDESC), "r"(0u), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}
__device__ __forceinline__ void xt_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void xt_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void xt_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// The 96 accumulator columns of a region (four block pairs) of this thread's row, asynchronously:
// the registers are valid only after xt_wait_ld96 on the same array
__device__ __forceinline__ void xt_ld96(uint32_t taddr, uint32_t *v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]), "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(v[64]), "=r"(v[65]), "=r"(v[66]), "=r"(v[67]), "=r"(v[68]), "=r"(v[69]), "=r"(v[70]), "=r"(v[71]), "=r"(v[72]), "=r"(v[73]), "=r"(v[74]), "=r"(v[75]), "=r"(v[76]), "=r"(v[77]), "=r"(v[78]), "=r"(v[79]), "=r"(v[80]), "=r"(v[81]), "=r"(v[82]), "=r"(v[83]), "=r"(v[84]), "=r"(v[85]), "=r"(v[86]), "=r"(v[87]), "=r"(v[88]), "=r"(v[89]), "=r"(v[90]), "=r"(v[91]), "=r"(v[92]), "=r"(v[93]), "=r"(v[94]), "=r"(v[95])
                 : "r"(taddr + 64) : "memory");
}
// Wait for the loads in flight; the registers pass through the statement so that no use of them can
// be scheduled before it.
__device__ __forceinline__ void xt_wait_ld96(uint32_t *v) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31]), "+r"(v[32]), "+r"(v[33]), "+r"(v[34]), "+r"(v[35]), "+r"(v[36]), "+r"(v[37]), "+r"(v[38]), "+r"(v[39]), "+r"(v[40]), "+r"(v[41]), "+r"(v[42]), "+r"(v[43]), "+r"(v[44]), "+r"(v[45]), "+r"(v[46]), "+r"(v[47]), "+r"(v[48]), "+r"(v[49]), "+r"(v[50]), "+r"(v[51]), "+r"(v[52]), "+r"(v[53]), "+r"(v[54]), "+r"(v[55]), "+r"(v[56]), "+r"(v[57]), "+r"(v[58]), "+r"(v[59]), "+r"(v[60]), "+r"(v[61]), "+r"(v[62]), "+r"(v[63]), "+r"(v[64]), "+r"(v[65]), "+r"(v[66]), "+r"(v[67]), "+r"(v[68]), "+r"(v[69]), "+r"(v[70]), "+r"(v[71]), "+r"(v[72]), "+r"(v[73]), "+r"(v[74]), "+r"(v[75]), "+r"(v[76]), "+r"(v[77]), "+r"(v[78]), "+r"(v[79]), "+r"(v[80]), "+r"(v[81]), "+r"(v[82]), "+r"(v[83]), "+r"(v[84]), "+r"(v[85]), "+r"(v[86]), "+r"(v[87]), "+r"(v[88]), "+r"(v[89]), "+r"(v[90]), "+r"(v[91]), "+r"(v[92]), "+r"(v[93]), "+r"(v[94]), "+r"(v[95])
                 :: "memory");
}
__device__ __forceinline__ void xt_bar_epi() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Waits of the pipeline loops.  The loops are executed by one warp per scheduler, so their code
// has to stay small enough for the instruction cache next to the scheduler: the common case (phase
// already complete) is one probe inline, everything else is out of line.  Bounded like Waiter::wait;
// returns false (after recording the error) when the wait ran out.
__device__ __noinline__ bool xt_wait_slow(uint64_t *bar, uint32_t parity, uint32_t *err, bool sleep) {
    if (err && *reinterpret_cast<volatile uint32_t *>(err) != 0u) return false;      // a wait has already failed: do not wait again
    const long long t0 = clock64();
    do {
        for (int i = 0; i < 64; i++) {
            if (sleep) __nanosleep(32);
            if (sleep ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
        }
    } while (clock64() - t0 < WAIT_CYCLES);
    if (err) atomicCAS(err, (uint32_t)DEV_ERR_NONE, (uint32_t)DEV_ERR_COPY_TIMEOUT);
    return false;
}
__device__ __forceinline__ void xt_wait(uint64_t *bar, uint32_t parity, uint32_t *err, bool sleep = false) {
    if (!mbar_test_wait(bar, parity)) xt_wait_slow(bar, parity, err, sleep);
}

// Operand image of an activation that some other kernel quantised (stage-level entry points).
__global__ void xt_bimg_kernel(const int8_t *__restrict__ xq, int nb, uint8_t *bimg) {
    const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (b >= nb) return;
    xt_emit_block((int)xq[b * 32 + lane], lane, b, bimg);
}

// ---------------------------------------------------------------- the two expert kernels
struct XtArgs {
    MxtDev w;                   // gate|up tiles, or down tiles
    const float *bias_a;        // gate bias, or down bias       [expert][d]
    const float *bias_b;        // up bias
    const int32_t *top;         // exact routing (used when est == nullptr)
    const float *wts;           // down: nullable, see launch_down_t
    const float *est;           // nullable: router estimate; slot s belongs to its s-th largest entry
    int ne, topk, d;
    const uint8_t *bimg;        // operand image of the activation: gate/up [np][768]; down [slot][np][768]
    const float *xs;            // its block scales:                gate/up [blocks];   down [slot][blocks]
    int8_t *hq;                 // gate/up outputs: Q8 of h per slot, its scales, its operand image
    float *hs;
    uint8_t *himg;
    float *x;                   // down: residual stream, updated in place
    float *part;                // down: [topk][tiles * 128] row sums before bias
    uint32_t *counter;          // down: [tiles] arrival counters, zero between launches
    DevState *state;
    int stages;
    // expert parallelism (ep_on): w holds the experts [ep.e_lo, ep.e_lo + ep.e_cnt) only; CTAs of a slot
    // whose expert lives on another rank do nothing; down stores its row sums, each tagged with the step
    // number in one 64-bit word, into every rank's buffer ep.pairs ([layer][slot][d])
    int ep_on, layer;
    EpCtx ep;
};

struct XtShared {
    unsigned char *ring, *bimg;
    float *xsc, *tbl;
    uint64_t *full, *empty, *dfull, *dempty, *bfull;
};

// One block pair of one row: the 8 exact lane dots from the three digit planes, then the two
// blocks' fused multiply-adds of the four chains, in block order.  Two chains share an instruction
// (fma.rn.f32x2: two independent round-to-nearest fused multiply-adds).
struct XtAcc { unsigned long long a01, a23; };       // chains (0, 1) and (2, 3), packed f32x2
__device__ __forceinline__ unsigned long long xt_pack(uint32_t lo, uint32_t hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ unsigned long long xt_fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ void xt_pair(const uint32_t *v, float s0, float s1, XtAcc &acc) {
    const unsigned long long k49 = xt_pack(0x42440000u, 0x42440000u), k7 = xt_pack(0x40E00000u, 0x40E00000u);
    unsigned long long tq[4];
#pragma unroll
    for (int i = 0; i < 4; i++)
        tq[i] = xt_fma2(xt_pack(v[2 * i], v[2 * i + 1]), k49, xt_fma2(xt_pack(v[8 + 2 * i], v[9 + 2 * i]), k7, xt_pack(v[16 + 2 * i], v[17 + 2 * i])));
    const unsigned long long p0 = xt_pack(__float_as_uint(s0), __float_as_uint(s0)), p1 = xt_pack(__float_as_uint(s1), __float_as_uint(s1));
    acc.a01 = xt_fma2(tq[0], p0, acc.a01); acc.a23 = xt_fma2(tq[1], p0, acc.a23);
    acc.a01 = xt_fma2(tq[2], p1, acc.a01); acc.a23 = xt_fma2(tq[3], p1, acc.a23);
}
__device__ __forceinline__ float xt_row_sum(const XtAcc &acc) {       // (a0 + a1) + (a2 + a3)
    uint32_t a0, a1, a2, a3;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a0), "=r"(a1) : "l"(acc.a01));
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a2), "=r"(a3) : "l"(acc.a23));
    return __fadd_rn(__fadd_rn(__uint_as_float(a0), __uint_as_float(a1)), __fadd_rn(__uint_as_float(a2), __uint_as_float(a3)));
}

template <bool DOWN, bool EP>
__global__ void __launch_bounds__(XT_THREADS) xt_expert_kernel(XtArgs a) {
    extern __shared__ __align__(128) unsigned char smraw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int np = a.w.np, nb = np * 2;
    const int t = blockIdx.x, ei = blockIdx.y;
    const int nchunks = (np + XT_CH - 1) / XT_CH;
    const size_t stage_bytes = (size_t)XT_CH * MXT_UNIT;
    XtShared sh;
    sh.ring = smraw;
    sh.bimg = smraw + stage_bytes * a.stages;
    sh.xsc = reinterpret_cast<float *>(sh.bimg + (size_t)np * XT_B_PAIR);
    sh.tbl = sh.xsc + nb;
    sh.full = reinterpret_cast<uint64_t *>(sh.tbl + 256);
    sh.empty = sh.full + a.stages;
    sh.dfull = sh.empty + a.stages;
    sh.dempty = sh.dfull + XT_REGIONS;
    sh.bfull = sh.dempty + XT_REGIONS;
    __shared__ uint32_t tmem_base_sh;
    __shared__ int sel[8];
    __shared__ float lg[256];
    __shared__ float gu_s[2][64];
    __shared__ int last_sh;
    uint32_t *err = a.state ? &a.state->err : nullptr;
    constexpr int SB = DOWN ? 128 : 96;          // clock stamps of timeline builds
    (void)SB;
    BRRR_STAMP(a.state, SB);
    BRRR_GT_START(a.state, DOWN ? 237 : 236);

    // ---- set-up that needs nothing from the kernels before
    mx_fill_scale_table(sh.tbl, tid, XT_THREADS);
    if (tid == 0) {
        for (int s = 0; s < a.stages; s++) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 4); }
        for (int r = 0; r < XT_REGIONS; r++) { mbar_init(&sh.dfull[r], 1); mbar_init(&sh.dempty[r], 4); }
        mbar_init(sh.bfull, 1);
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(XT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    xt_fence_before();
    __syncthreads();
    xt_fence_after();
    const uint32_t tmem_base = tmem_base_sh;
    if (warp < 4) {
        // unit scale factors (ue8m0 0x7F) in the 64 columns behind the accumulator regions, every lane
        const uint32_t one = 0x7F7F7F7Fu, addr = tmem_base + ((uint32_t)(warp * 32) << 16) + XT_SF_COL;
        for (int c = 0; c < 64; c += 8)
            asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(addr + c), "r"(one) : "memory");
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    xt_fence_before();
    __syncthreads();                 // scale factors in place before the issuing thread can reach its first MMA
    xt_fence_after();
    // ---- routing of this slot (the ei-th largest entry of the estimate, or the exact routing), the
    // weight stream, the activation image (one bulk copy) and its block scales
    int e = 0;
    bool local = true;
    const unsigned char *src = nullptr;
    const uint32_t ep_epoch = EP ? *a.ep.epoch : 0u;          // the step in flight (written by the step's first kernel)
    auto route_and_start = [&]() {
        if (a.est) {
            block_spec_select(a.est, a.ne, a.topk, a.state, lg, sel, tid, XT_THREADS);
            __syncthreads();
            e = sel[ei];
        } else e = a.top[ei];
        local = !EP || (e >= a.ep.e_lo && e < a.ep.e_lo + a.ep.e_cnt);
        src = a.w.data + ((size_t)(EP ? e - a.ep.e_lo : e) * a.w.tiles_per_expert + t) * np * MXT_UNIT;
        if (local && warp == 4 && lane < min(a.stages, nchunks)) {          // one lane per copy: the first stages of the weight stream
            const int cnt = min(XT_CH, np - lane * XT_CH);
            mbar_expect_tx(&sh.full[lane], (uint32_t)cnt * MXT_UNIT);
            bulk_g2s(sh.ring + stage_bytes * lane, src + (size_t)lane * stage_bytes, (uint32_t)cnt * MXT_UNIT, &sh.full[lane]);
        }
    };
    // The down projection knows its expert before gate/up has finished (the routing is two kernels
    // old), and its CTAs have the footprint of a gate/up CTA: they become resident beside running
    // gate/up CTAs and start their weight stream there, before they wait for h.
    constexpr bool early = DOWN;
    if (early) route_and_start();
    BRRR_STAMP(a.state, SB + 1);
    pdl_wait();
    BRRR_STAMP(a.state, SB + 2);
    BRRR_GT_GO(a.state, SB + 30);
    pdl_trigger();
    // (gate/up learns whether its slot is local only below: it copies the image in any case)
    const bool img_copy = early ? local : true;
    if (img_copy && warp == 4 && lane == 31) {
        const uint8_t *img = a.bimg + (DOWN ? (size_t)ei * np * XT_B_PAIR : 0);
        mbar_expect_tx(sh.bfull, (uint32_t)np * XT_B_PAIR);
        bulk_g2s(sh.bimg, img, (uint32_t)np * XT_B_PAIR, sh.bfull);
    }
    float xs_mine = 0.0f;
    if (tid < nb) xs_mine = (DOWN ? a.xs + (size_t)ei * nb : a.xs)[tid];      // nb <= 128: the epilogue warps hold all of it
    if (!early) route_and_start();
    if (tid < nb) sh.xsc[tid] = xs_mine;
    if (warp < 4) xt_bar_epi();                                  // block scales visible to the epilogue warps
    BRRR_STAMP(a.state, SB + 3);

    // Loop structure shared by the three roles: round r = ring stage r % stages = 4 block pairs =
    // accumulator region r % 2.  All indices advance incrementally.
    if (EP && !local) {
        // the slot's expert lives on another rank: nothing to compute here (a copy in flight must land first)
        if (img_copy && warp == 4 && lane == 31) xt_wait(sh.bfull, 0u, err, true);
    } else if (warp == 4) {
        // ---- producer: refill a stage once the four epilogue warps have left it
        if (lane == 0) {
            int s = 0;
            uint32_t par = 0;                        // parity of the release being waited for
            for (int c = a.stages; c < nchunks; c++) {
                const int cnt = min(XT_CH, np - c * XT_CH);
                xt_wait(&sh.empty[s], par, err, true);
                mbar_expect_tx(&sh.full[s], (uint32_t)cnt * MXT_UNIT);
                bulk_g2s(sh.ring + stage_bytes * s, src + (size_t)c * stage_bytes, (uint32_t)cnt * MXT_UNIT, &sh.full[s]);
                if (++s == a.stages) { s = 0; par ^= 1u; }
            }
        }
    } else if (warp == 5) {
        // ---- MMA issue: one instruction per block pair, four per round into one accumulator region
        if (lane == 0) {
            const uint32_t sfa = tmem_base + XT_SF_COL, sfb = tmem_base + XT_SF_COL + 32;
            const uint64_t dhi = ((uint64_t)((128u >> 4) & 0x3FFF) << 32) | ((uint64_t)1 << 46);     // descriptor bits common to A and B
            const uint64_t alo = dhi | ((uint64_t)((2048u >> 4) & 0x3FFF) << 16), blo = dhi | ((uint64_t)(((uint32_t)XT_B_PAIR / 2 >> 4) & 0x3FFF) << 16);
            uint32_t baddr = smem_u32(sh.bimg) >> 4;              // descriptor start-address fields (16-byte units)
            const uint32_t r0 = smem_u32(sh.ring) >> 4, stage16 = (uint32_t)(stage_bytes >> 4);
            xt_wait(sh.bfull, 0u, err, true);
            int s = 0, reg = 0, left = np;
            uint32_t fpar = 0, epar = 1;             // full-stage parity; region-free parity (first pass: free)
#pragma unroll 1
            for (int r = 0; r < nchunks; r++) {
                xt_wait(&sh.full[s], fpar, err, true);
                xt_wait(&sh.dempty[reg], epar, err, true);
                xt_fence_after();
                const uint32_t aaddr = r0 + s * stage16, d0 = tmem_base + reg * XT_REGION_COLS;
                const int cnt = left < XT_CH ? left : XT_CH;
#pragma unroll
                for (int k = 0; k < XT_CH; k++)
                    if (k < cnt) xt_mma(d0 + k * XT_N, alo | (aaddr + k * (MXT_UNIT / 16)), blo | (baddr + k * (XT_B_PAIR / 16)), sfa, sfb);
                xt_commit(&sh.dfull[reg]);
                baddr += XT_CH * XT_B_PAIR / 16;
                left -= XT_CH;
                if (++s == a.stages) { s = 0; fpar ^= 1u; }
                if (++reg == XT_REGIONS) { reg = 0; epar ^= 1u; }
            }
        }
    } else {
        // ---- epilogue: thread m owns tile row m
        const int m = tid;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        XtAcc acc{0ull, 0ull};
        const float bias_pre = DOWN ? 0.0f : ((m >> 6) ? a.bias_b : a.bias_a)[(size_t)e * a.d + t * 64 + (m & 63)];   // in flight during the stream
        uint32_t dv[XT_REGION_COLS] = {};
        int s = 0, reg = 0, left = np;
        uint32_t spar = 0, dpar = 0;
        const float *xsp = sh.xsc;
        long long tw_full = 0, tw_sc = 0, tw_d = 0, tw_ld = 0, tw_math = 0;
        (void)tw_full; (void)tw_sc; (void)tw_d; (void)tw_ld; (void)tw_math;
#pragma unroll 1
        for (int r = 0; r < nchunks; r++) {
            const int cnt = left < XT_CH ? left : XT_CH;
            XT_T0();
            xt_wait(&sh.full[s], spar, err);                    // the stage's exponent bytes are visible
            XT_ACC(tw_full);
            const unsigned char *ex = sh.ring + stage_bytes * s + MXT_UNIT_EXPS + m * 2;
            uint32_t e2[XT_CH];
#pragma unroll
            for (int k = 0; k < XT_CH; k++) e2[k] = k < cnt ? *reinterpret_cast<const unsigned short *>(ex + k * MXT_UNIT) : 0u;
            const float4 xa = *reinterpret_cast<const float4 *>(xsp), xb = *reinterpret_cast<const float4 *>(xsp + 4);
            float sc[2 * XT_CH];                                // block scales: 2^(e-128) * xs
            sc[0] = __fmul_rn(sh.tbl[e2[0] & 0xFFu], xa.x); sc[1] = __fmul_rn(sh.tbl[e2[0] >> 8], xa.y);
            sc[2] = __fmul_rn(sh.tbl[e2[1] & 0xFFu], xa.z); sc[3] = __fmul_rn(sh.tbl[e2[1] >> 8], xa.w);
            sc[4] = __fmul_rn(sh.tbl[e2[2] & 0xFFu], xb.x); sc[5] = __fmul_rn(sh.tbl[e2[2] >> 8], xb.y);
            sc[6] = __fmul_rn(sh.tbl[e2[3] & 0xFFu], xb.z); sc[7] = __fmul_rn(sh.tbl[e2[3] >> 8], xb.w);
            XT_ACC(tw_sc);
            xt_wait(&sh.dfull[reg], dpar, err);
            XT_ACC(tw_d);
            xt_fence_after();
            xt_ld96(lane_addr + reg * XT_REGION_COLS, dv);
            xt_wait_ld96(dv);
            XT_ACC(tw_ld);
            xt_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&sh.dempty[reg]);
                mbar_arrive(&sh.empty[s]);                      // the stage's MMAs are complete and its exponents read
            }
#pragma unroll
            for (int k = 0; k < XT_CH; k++)
                if (k < cnt) xt_pair(dv + XT_N * k, sc[2 * k], sc[2 * k + 1], acc);
            xsp += 2 * XT_CH;
            left -= XT_CH;
            if (++s == a.stages) { s = 0; spar ^= 1u; }
            if (++reg == XT_REGIONS) { reg = 0; dpar ^= 1u; }
            XT_ACC(tw_math);
            if (r < 12) BRRR_STAMP(a.state, SB + 4 + r);
        }
        BRRR_STAMP(a.state, SB + 16);
#ifdef BRRR_TEST_HOOKS
        if (a.state && tid == 0 && blockIdx.x == BRRR_STAMP_BX && blockIdx.y == 0) {
            long long *o = a.state->stamps + (DOWN ? 205 : 200);
            o[0] = tw_full; o[1] = tw_sc; o[2] = tw_d; o[3] = tw_ld; o[4] = tw_math;
        }
#endif
        const float v = xt_row_sum(acc);
        if (!DOWN) {
            gu_s[m >> 6][m & 63] = __fadd_rn(v, bias_pre);
            xt_bar_epi();
            if (warp < 2) {
                // SwiGLU, Q8 of this 32-block of h, and its share of the operand image down reads
                const float h = swiglu_oai(gu_s[0][warp * 32 + lane], gu_s[1][warp * 32 + lane]);
                const float amax = fmaxf(warp_max(fabsf(h)), 1e-12f);
                const float sc = __fdiv_rn(amax, 127.0f);
                const int qv = brrr_q8_round(h, sc), b = t * 2 + warp;
                if (lane == 0) a.hs[ei * nb + b] = sc;
                a.hq[(size_t)ei * a.d + b * 32 + lane] = (int8_t)qv;
                xt_emit_block(qv, lane, b, a.himg + (size_t)ei * np * XT_B_PAIR);
            }
        } else {
            const int r = t * 128 + m, dpad = a.w.tiles_per_expert * 128;
            if (EP) {
                // the row sum, tagged with the step number, to every rank: one plain 64-bit store over
                // NVLink peer memory per rank; the consumer polls the word itself
                const size_t off = ((size_t)a.layer * a.topk + ei) * a.d + r;
                const unsigned long long word = ((unsigned long long)ep_epoch << 32) | __float_as_uint(v);
                if (r < a.d)
                    for (int p = 0; p < a.ep.world; p++) if (p != a.ep.rank) a.ep.pairs[p][off] = word;
                a.part[(size_t)ei * dpad + r] = v;          // this rank's own fold reads it after the kernel boundary
            } else a.part[(size_t)ei * dpad + r] = v;
            if (a.wts) {                     // exact routing known: fold here; else a fold kernel follows
                __threadfence();
                xt_bar_epi();
                if (m == 0) last_sh = atomicAdd(&a.counter[t], 1u) == (uint32_t)(a.topk - 1);
                xt_bar_epi();
            } else if (m == 0) last_sh = 0;
            if (a.wts && last_sh) {
                // the last of the top-k CTAs of these 128 rows folds them in slot order
                __threadfence();
                if (r < a.d) {
                    float s = a.x[r];
                    for (int k = 0; k < a.topk; k++)
                        s = __fadd_rn(s, __fmul_rn(a.wts[k], __fadd_rn(__ldcg(&a.part[(size_t)k * dpad + r]), a.bias_a[(size_t)a.top[k] * a.d + r])));
                    a.x[r] = s;
                }
                if (m == 0) a.counter[t] = 0;
            }
        }
    }
    BRRR_STAMP(a.state, SB + 17);
    BRRR_GT_END(a.state, SB + 31);
    xt_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(XT_TMEM_COLS) : "memory");
}

// Fold of the down-projection partial sums once the exact routing is known:
//   x[r] += sum over k ascending of wts[k] * (part[slot of top[k]][r] + bias[top[k]][r])
// (multiply, then add, as the reference's combine).  With est != nullptr the partial sums were
// computed for the top-k of the estimate: exact experts missing from it flag the step.
struct FoldArgs {
    const int32_t *top;
    const float *wts, *est;
    int ne, topk, d, dpad;
    const float *part, *down_b;
    float *x;
    DevState *state;
};

__global__ void __launch_bounds__(128) xt_fold_kernel(FoldArgs a) {
    __shared__ int sel[8];
    __shared__ float lg[256];
    __shared__ int slot_of[8];
    const int tid = threadIdx.x;
    BRRR_GT_START(a.state, 238);
    pdl_wait();
    BRRR_GT_GO(a.state, 239);
    pdl_trigger();
    if (a.est) {
        block_spec_select(a.est, a.ne, a.topk, a.state, lg, sel, tid, 128);
        __syncthreads();
    }
    if (tid < a.topk) {
        int slot = tid;
        if (a.est) {
            slot = -1;
            const int want = a.top[tid];
            for (int s = 0; s < a.topk; s++) if (sel[s] == want) slot = s;
            if (slot < 0) {                  // the estimate missed this expert: flag the step, keep going
                slot = 0;
                if (blockIdx.x == 0 && a.state) atomicMin(&a.state->spec_fail_step, a.state->n_out);
            }
        }
        slot_of[tid] = slot;
    }
    __syncthreads();
    const int r = blockIdx.x * 128 + tid;
    if (r < a.d) {
        float s = a.x[r];
        for (int k = 0; k < a.topk; k++)
            s = __fadd_rn(s, __fmul_rn(a.wts[k], __fadd_rn(a.part[(size_t)slot_of[k] * a.dpad + r], a.down_b[(size_t)a.top[k] * a.d + r])));
        a.x[r] = s;
    }
    BRRR_GT_END(a.state, 240);
}

// The same fold as one CTA that also prepares the next projection's activation.  Used by the
// speculative decode step, where the exact router runs on another stream beside gate/up and down:
// instead of a graph edge from the router (which would cost this kernel its programmatic launch),
// one lane per word polls, bounded, the routing words the router publishes, each tagged with the
// router's sequence number (this launch expects fold_seq + 1; the router does not depend on this
// kernel, so the wait cannot deadlock).  The partial sums, the
// residual and the routing estimate are fetched before that wait.  After the fold the whole
// residual is in shared memory, so the RMS norm (fixed 16-chain order) and the Q8 image that the
// next q/k/v projection (or the vocabulary head) needs are computed here once, rather than by every
// CTA of that projection.
struct FoldNormArgs {
    FoldArgs f;
    const float *norm_w;     // nullable: fold only
    float eps;
    int8_t *nq;              // Q8 of the normalised residual, element order
    float *ns;               // its block scales
    uint32_t *router_seq, *fold_seq;
    // expert parallelism: the row sums come from the ranks that own the estimate's experts, as 64-bit
    // words (step number << 32 | float bits) in this rank's buffer of the layer ([slot][d]); a word is
    // valid once it carries the step number *ep_epoch
    const unsigned long long *ep_pairs;
    const uint32_t *ep_epoch;
    int ep_lo, ep_cnt;       // this rank's experts: their slots' row sums are in f.part, as on a single GPU
};

constexpr int FN_THREADS = 1024;

template <int MAXS, bool EP>       // slots held in registers: top-k <= MAXS; EP: expert-parallel exchange
__global__ void __launch_bounds__(FN_THREADS) xt_fold_norm_kernel(FoldNormArgs a) {
    extern __shared__ __align__(16) float fsm[];          // d floats of the residual
    __shared__ int sel[8];
    __shared__ float lg[256];
    __shared__ int slot_of[8];
    __shared__ float wts_sh[8];
    __shared__ float inv_sh;
    const int tid = threadIdx.x, d = a.f.d, dpad = a.f.dpad, topk = a.f.topk;
    float *xf = fsm;
    // ---- everything that kernels before down produced, before the dependency wait: norm weights,
    // the residual, the speculative expert set and those experts' biases
    float4 wreg[1];
    norm_prefetch<1>(a.norm_w, d, wreg, tid, FN_THREADS);
    BRRR_GT_START(a.f.state, 238);
    // thread g owns rows 4g .. 4g+3 (one 16-byte access per operand)
    const bool live = tid < (d >> 2);
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 xr = live ? reinterpret_cast<const float4 *>(a.f.x)[tid] : zero4, pb[MAXS], ps[MAXS];
    if (a.f.est) {
        block_spec_select(a.f.est, a.f.ne, topk, a.f.state, lg, sel, tid, FN_THREADS);
        __syncthreads();
#pragma unroll
        for (int s = 0; s < MAXS; s++) pb[s] = (live && s < topk) ? reinterpret_cast<const float4 *>(a.f.down_b + (size_t)sel[s] * d)[tid] : zero4;
    }
    const uint32_t want_seq = a.fold_seq ? __ldcg(a.fold_seq) + 1u : 0u;      // written by the previous launch of this kernel
    const uint32_t ep_epoch = EP ? *a.ep_epoch : 0u;                  // the step in flight (written by the step's first kernel)
#ifdef BRRR_FOLD_EARLY_TRIGGER
    pdl_trigger();       // the next projection may become resident and stream its weights while down still runs
#endif
    pdl_wait();          // down's partial sums are complete
    BRRR_GT_GO(a.f.state, 239);
    BRRR_STAMP(a.f.state, 241);
#ifndef BRRR_FOLD_EARLY_TRIGGER
    pdl_trigger();
#endif
    // ---- slot s: partial sum of the s-th expert of the estimate
#pragma unroll
    for (int s = 0; s < MAXS; s++) {
        const bool mine = !EP || (sel[s < topk ? s : 0] >= a.ep_lo && sel[s < topk ? s : 0] < a.ep_lo + a.ep_cnt);
        ps[s] = (live && s < topk && mine) ? reinterpret_cast<const float4 *>(a.f.part + (size_t)s * dpad)[tid] : zero4;
    }
    if (EP && live) {
        // slots whose expert lives on another rank: every thread polls (bounded) the four tagged words
        // of its rows until all of them carry this step's number
        uint32_t *errp = a.f.state ? &a.f.state->err : nullptr;
        const long long t0 = clock64();
        bool ok = false;
        while (!ok) {
            ok = true;
#pragma unroll
            for (int s = 0; s < MAXS; s++) {
                if (s < topk && !(sel[s] >= a.ep_lo && sel[s] < a.ep_lo + a.ep_cnt)) {
                    // read at the L2, where the peers' stores to this GPU's memory land
                    const ulonglong2 *w = reinterpret_cast<const ulonglong2 *>(a.ep_pairs + (size_t)s * d) + 2 * tid;
                    const ulonglong2 lo = __ldcg(w), hi = __ldcg(w + 1);
                    ok = ok && (uint32_t)(lo.x >> 32) == ep_epoch && (uint32_t)(lo.y >> 32) == ep_epoch && (uint32_t)(hi.x >> 32) == ep_epoch &&
                         (uint32_t)(hi.y >> 32) == ep_epoch;
                    ps[s] = make_float4(__uint_as_float((uint32_t)lo.x), __uint_as_float((uint32_t)lo.y), __uint_as_float((uint32_t)hi.x),
                                        __uint_as_float((uint32_t)hi.y));
                }
            }
            if (!ok && (clock64() - t0 > EP_WAIT_CYCLES || (errp && *reinterpret_cast<volatile uint32_t *>(errp) != 0u))) {
                if (errp) atomicCAS(errp, (uint32_t)DEV_ERR_NONE, (uint32_t)DEV_ERR_PEER_TIMEOUT);
                break;
            }
        }
    }
    BRRR_STAMP(a.f.state, 242);
    // ---- the exact routing: the router publishes sequence-tagged words; one lane per word polls
    // (bounded) until its word carries this launch's sequence number
    if (tid < 32) {
        uint32_t payload = 0u;
        if (a.router_seq) {
            if (tid < 16 && (tid & 7) < topk) {
                const volatile unsigned long long *w = a.f.state->route_pub + tid;
                bool ok = false;
                const long long t0 = clock64();
                do {
                    for (int i = 0; i < 64 && !ok; i++) {
                        const unsigned long long v = *w;
                        ok = (uint32_t)(v >> 32) == want_seq;
                        payload = (uint32_t)v;
                    }
                    // give up at once when the error word is already set (an earlier wait of this step ran out)
                } while (!ok && clock64() - t0 < WAIT_CYCLES && *reinterpret_cast<volatile uint32_t *>(&a.f.state->err) == 0u);
                if (!ok) {
                    // the step is void from here: record where, so that the host can run it again without speculation
                    atomicCAS(&a.f.state->err, (uint32_t)DEV_ERR_NONE, (uint32_t)DEV_ERR_PEER_TIMEOUT);
                    atomicMin(&a.f.state->spec_fail_step, a.f.state->n_out);
                }
            }
        } else if (tid < 16 && (tid & 7) < topk) {
            payload = tid < 8 ? (uint32_t)__ldcg(a.f.top + tid) : __float_as_uint(__ldcg(a.f.wts + (tid - 8)));
        }
        __syncwarp();
        if (tid >= 8 && tid < 8 + topk) wts_sh[tid - 8] = __uint_as_float(payload);
        if (tid < topk) {
            const int want = (int)payload;
            int slot = tid;
            if (a.f.est) {
                slot = -1;
                for (int s = 0; s < topk; s++) if (sel[s] == want) slot = s;
                if (slot < 0) {                  // the estimate missed this expert: flag the step, keep going
                    slot = 0;
                    if (a.f.state) atomicMin(&a.f.state->spec_fail_step, a.f.state->n_out);
                }
            }
            slot_of[tid] = slot;
            if (!a.f.est) sel[tid] = want;
        }
    }
    BRRR_STAMP(a.f.state, 243);
    __syncthreads();
    BRRR_STAMP(a.f.state, 244);
    if (!a.f.est) {      // exact routing only: the biases could not be fetched ahead
#pragma unroll
        for (int s = 0; s < MAXS; s++) pb[s] = (live && s < topk) ? reinterpret_cast<const float4 *>(a.f.down_b + (size_t)sel[s] * d)[tid] : zero4;
    }
    if (live) {
        float4 acc = xr;
        for (int kk = 0; kk < topk; kk++) {
            const int sl = slot_of[kk];
            const float w = wts_sh[kk];
            float4 p = ps[0], bb = pb[0];
            switch (sl) {                    // uniform over the block: a branch, not a chain of selects
            case 1: p = ps[1]; bb = pb[1]; break;
            case 2: p = ps[2]; bb = pb[2]; break;
            case 3: p = ps[3]; bb = pb[3]; break;
            default:
                if (MAXS > 4) {
#pragma unroll
                    for (int q = 4; q < MAXS; q++) if (q == sl) { p = ps[q]; bb = pb[q]; }
                }
            }
            acc.x = __fadd_rn(acc.x, __fmul_rn(w, __fadd_rn(p.x, bb.x)));
            acc.y = __fadd_rn(acc.y, __fmul_rn(w, __fadd_rn(p.y, bb.y)));
            acc.z = __fadd_rn(acc.z, __fmul_rn(w, __fadd_rn(p.z, bb.z)));
            acc.w = __fadd_rn(acc.w, __fmul_rn(w, __fadd_rn(p.w, bb.w)));
        }
        reinterpret_cast<float4 *>(a.f.x)[tid] = acc;
        reinterpret_cast<float4 *>(xf)[tid] = acc;
    }
    BRRR_STAMP(a.f.state, 245);
    if (a.norm_w) {
        __syncthreads();
        BRRR_STAMP(a.f.state, 246);
        block_norm_quant_staged<NQ_NATURAL, 1>(a.norm_w, wreg, a.eps, d, xf, reinterpret_cast<int2 *>(a.nq), a.ns, &inv_sh, tid, FN_THREADS);
    }
    BRRR_STAMP(a.f.state, 247);
    if (tid == 0 && a.fold_seq) *a.fold_seq = want_seq;
    BRRR_GT_END(a.f.state, 240);
}

size_t xt_smem_bytes(int np, int stages) {
    return (size_t)stages * XT_CH * MXT_UNIT + (size_t)np * XT_B_PAIR + (size_t)np * 2 * 4 + 256 * 4 + (size_t)(2 * stages + 2 * XT_REGIONS + 1) * 8;
}

}  // namespace

// ---------------------------------------------------------------- launchers
size_t mxt_bytes(int experts, int tiles_per_expert, int np) { return (size_t)experts * tiles_per_expert * np * MXT_UNIT; }

void launch_mxt_pack(MxDev a, MxDev b, int experts, int rows_per_expert, MxtDev out, cudaStream_t st) {
    PackArgs p{};
    p.a = a; p.b = b; p.rows_per_expert = rows_per_expert; p.tiles_per_expert = out.tiles_per_expert; p.out = out;
    const size_t words = mxt_bytes(experts, out.tiles_per_expert, out.np) / 4;
    if (!words) return;
    mxt_pack_kernel<<<(unsigned)((words + 255) / 256), 256, 0, st>>>(p, words);
}

void launch_xt_bimg(const int8_t *xq, int nb, uint8_t *bimg, cudaStream_t st) {
    if (nb > 0) xt_bimg_kernel<<<(nb + 3) / 4, 128, 0, st>>>(xq, nb, bimg);
}

cudaError_t launch_gate_up_t(MxtDev gu, const float *gate_b, const float *up_b, const int32_t *top, const float *est, int ne, int topk,
                             int d, const uint8_t *ximg, const float *xs, int8_t *hq, float *hs, uint8_t *himg, DevState *state,
                             bool pdl, cudaStream_t st, const EpCtx *ep, int layer) {
    XtArgs a{};
    if (ep) { a.ep_on = 1; a.ep = *ep; a.layer = layer; }
    a.w = gu; a.bias_a = gate_b; a.bias_b = up_b; a.top = top; a.est = est; a.ne = ne; a.topk = topk; a.d = d;
    a.bimg = ximg; a.xs = xs; a.hq = hq; a.hs = hs; a.himg = himg; a.state = state;
    const int nchunks = (gu.np + XT_CH - 1) / XT_CH;
#ifndef XT_GU_STAGES
#define XT_GU_STAGES 4
#endif
    a.stages = nchunks < XT_GU_STAGES ? nchunks : XT_GU_STAGES;            // two CTAs per SM at the 20b shape
    static unsigned long long configured = 0, configured_ep = 0;      // one bit per device
    {
        cudaError_t e = smem_optin(xt_expert_kernel<false, false>, 200 * 1024, configured);
        if (e == cudaSuccess) e = smem_optin(xt_expert_kernel<false, true>, 200 * 1024, configured_ep);
        if (e != cudaSuccess) return e;
    }
    if (ep) return launch_k(xt_expert_kernel<false, true>, dim3(gu.tiles_per_expert, topk), dim3(XT_THREADS), xt_smem_bytes(gu.np, a.stages), st, pdl, a);
    return launch_k(xt_expert_kernel<false, false>, dim3(gu.tiles_per_expert, topk), dim3(XT_THREADS), xt_smem_bytes(gu.np, a.stages), st, pdl, a);
}

cudaError_t launch_down_t(MxtDev down, const float *down_b, const int32_t *top, const float *wts, const float *est, int ne, int topk,
                          int d, const uint8_t *himg, const float *hs, float *x, float *part, uint32_t *counter, DevState *state,
                          bool pdl, cudaStream_t st, const EpCtx *ep, int layer) {
    XtArgs a{};
    if (ep) { a.ep_on = 1; a.ep = *ep; a.layer = layer; }
    a.w = down; a.bias_a = down_b; a.top = top; a.wts = wts; a.est = est; a.ne = ne; a.topk = topk; a.d = d;
    a.bimg = himg; a.xs = hs; a.x = x; a.part = part; a.counter = counter; a.state = state;
    const int nchunks = (down.np + XT_CH - 1) / XT_CH;
    // the same footprint as a gate/up CTA: a down CTA fits beside a running gate/up CTA, sets up and
    // starts its weight stream there, before gate/up has finished (measured: 745 tok/s against 728
    // with a 9-stage ring that needs an SM of its own)
#ifndef XT_DOWN_STAGES
#define XT_DOWN_STAGES 4
#endif
    a.stages = nchunks < XT_DOWN_STAGES ? nchunks : XT_DOWN_STAGES;
    static unsigned long long configured = 0, configured_ep = 0;      // one bit per device
    {
        cudaError_t e = smem_optin(xt_expert_kernel<true, false>, 210 * 1024, configured);
        if (e == cudaSuccess) e = smem_optin(xt_expert_kernel<true, true>, 210 * 1024, configured_ep);
        if (e != cudaSuccess) return e;
    }
    if (ep) return launch_k(xt_expert_kernel<true, true>, dim3(down.tiles_per_expert, topk), dim3(XT_THREADS), xt_smem_bytes(down.np, a.stages), st, pdl, a);
    return launch_k(xt_expert_kernel<true, false>, dim3(down.tiles_per_expert, topk), dim3(XT_THREADS), xt_smem_bytes(down.np, a.stages), st, pdl, a);
}

cudaError_t launch_down_fold(const int32_t *top, const float *wts, const float *est, int ne, int topk, int d, const float *part,
                             const float *down_b, float *x, DevState *state, bool pdl, cudaStream_t st) {
    FoldArgs a{};
    a.top = top; a.wts = wts; a.est = est; a.ne = ne; a.topk = topk; a.d = d; a.dpad = (d + 127) / 128 * 128;
    a.part = part; a.down_b = down_b; a.x = x; a.state = state;
    return launch_k(xt_fold_kernel, dim3((d + 127) / 128), dim3(128), 0, st, pdl, a);
}

cudaError_t launch_fold_norm(const int32_t *top, const float *wts, const float *est, int ne, int topk, int d, const float *part,
                             const float *down_b, float *x, const float *next_norm_w, float eps, int8_t *nq, float *ns,
                             uint32_t *router_seq, uint32_t *fold_seq, DevState *state, bool pdl, cudaStream_t st, const EpCtx *ep, int layer) {
    if (d > 4 * FN_THREADS || d % 32 || topk > 8 || (router_seq && !state)) return cudaErrorInvalidValue;
    FoldNormArgs a{};

    a.f.top = top; a.f.wts = wts; a.f.est = est; a.f.ne = ne; a.f.topk = topk; a.f.d = d; a.f.dpad = (d + 127) / 128 * 128;
    a.f.part = part; a.f.down_b = down_b; a.f.x = x; a.f.state = state;
    a.norm_w = next_norm_w; a.eps = eps; a.nq = nq; a.ns = ns; a.router_seq = router_seq; a.fold_seq = fold_seq;
    if (ep) { a.ep_pairs = ep->pairs[ep->rank] + (size_t)layer * topk * d; a.ep_epoch = ep->epoch; a.ep_lo = ep->e_lo; a.ep_cnt = ep->e_cnt; }
    const size_t smem = (size_t)d * sizeof(float);
    if (ep) return topk <= 4 ? launch_k(xt_fold_norm_kernel<4, true>, dim3(1), dim3(FN_THREADS), smem, st, pdl, a)
                             : launch_k(xt_fold_norm_kernel<8, true>, dim3(1), dim3(FN_THREADS), smem, st, pdl, a);
    if (topk <= 4) return launch_k(xt_fold_norm_kernel<4, false>, dim3(1), dim3(FN_THREADS), smem, st, pdl, a);
    return launch_k(xt_fold_norm_kernel<8, false>, dim3(1), dim3(FN_THREADS), smem, st, pdl, a);
}

}  // namespace brrr
