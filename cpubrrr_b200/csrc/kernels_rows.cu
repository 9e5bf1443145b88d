// Token rows: the dense half of a layer for up to 512 tokens at once (prompt tiles and batched decode
// over independent sequences; forward_tile_worker, src/bin/engine_gpt2.rs:1011-1250, keeps the
// per-token arithmetic and shares each weight pass among the tokens of a tile).  Every value is
// computed by the same operation sequence as in the one-token kernels, so results are bit-identical
// to the token-serial schedule.
//
//   rmsnorm_quant (grid = rows)      one CTA per row, the one-token kernel with row offsets (kernels_small.cu)
//   q8_rows_kernel                   Q8 matrix x the Q8 activations of the rows: a CTA = 16 matrix rows x 8 token rows;
//                                    its weights go into registers once (before the dependency wait), the rows'
//                                    activations into shared memory, then one chain walk per four token rows
//   kv_append_rows_kernel            RoPE of every row's k and the cache append of k and v, before any row attends
//   attn_decode_kernel (grid.y = rows, kernels_attn.cu)
#include <cstdlib>
#include "brrr_kernels.h"
#include "brrr_block.cuh"
#include "brrr_tma.cuh"

namespace brrr {

namespace {

constexpr int QR_THREADS = 128;
constexpr int QR_TPC = 8;               // token rows per CTA (blockIdx.y walks the groups)

// packed pairs of floats (mul / fma .rn.f32x2)
__device__ __forceinline__ unsigned long long qr_pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
    return r;
}
__device__ __forceinline__ void qr_unpack2(unsigned long long v, float &lo, float &hi) {
    uint32_t a, b;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a); hi = __uint_as_float(b);
}
__device__ __forceinline__ unsigned long long qr_mul2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long qr_fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

struct Q8RowsArgs {
    Q8Dev m;
    const int8_t *xq;       // [rows][cols]
    const float *xs;        // [rows][cols / 32]
    const float *bias;
    float *y;               // [rows][ldy]
    int ntok, ldy;
};

// NP > 0: block pairs per matrix row, weights resident in registers.  NP == 0: any shape, weights read
// from global memory for every token row (small test shapes).
template <int EPI, int NP>
__global__ void __launch_bounds__(QR_THREADS) q8_rows_kernel(Q8RowsArgs a) {
    extern __shared__ __align__(16) unsigned char rsm[];
    const int np = NP > 0 ? NP : a.m.cols / 64, nb = np * 2;
    const int tid = threadIdx.x, rl = tid >> 3, c8 = tid & 7, p = c8 >> 2;
    const int u = blockIdx.x, row = u * 16 + rl;
    const uint8_t *unit0 = a.m.data + q8_unit_off(u, 0, np);
    const int2 *wp = reinterpret_cast<const int2 *>(unit0 + rl * 64 + c8 * 8);
    const float *sp = reinterpret_cast<const float *>(unit0 + Q8_UNIT_SCALES + rl * 8 + p * 4);
    int2 w[NP > 0 ? NP : 1];
    float s[NP > 0 ? NP : 1];
    if (NP > 0) {
#pragma unroll
        for (int i = 0; i < (NP > 0 ? NP : 1); i++) {
            w[i] = __ldg(wp + (size_t)i * (Q8_UNIT / 8));
            s[i] = __ldg(sp + (size_t)i * (Q8_UNIT / 4));
        }
    }
    const bool out = c8 == 0 && row < a.m.rows;
    float bias_pre = 0.0f;
    if (out && (EPI == Q8_EPI_BIAS || EPI == Q8_EPI_RESID_BIAS)) bias_pre = a.bias[row];
    pdl_wait();
    pdl_trigger();
    // the activation images of this CTA's token rows: [row][np * 8] int2 then [row][nb] floats
    const int t_first = blockIdx.y * QR_TPC, ntok = min(QR_TPC, a.ntok - t_first);
    int2 *xp = reinterpret_cast<int2 *>(rsm);
    float *xsc = reinterpret_cast<float *>(xp + (size_t)QR_TPC * np * 8);
    const int nidx = np * 8;
    for (int i = tid; i < ntok * nidx; i += QR_THREADS) {
        const int t = i / nidx, idx = i % nidx;
        const int *xw = reinterpret_cast<const int *>(a.xq + (size_t)(t_first + t) * a.m.cols + (idx >> 2) * 32);
        xp[i] = make_int2(xw[idx & 3], xw[4 + (idx & 3)]);
    }
    // block scales transposed to [block][token row]: two neighbouring rows' scales are one 8-byte read
    for (int i = tid; i < ntok * nb; i += QR_THREADS) xsc[(i % nb) * QR_TPC + i / nb] = a.xs[(size_t)t_first * nb + i];
    __syncthreads();
    // four token rows per walk over the weights: their chains are independent, so their instructions interleave, and
    // rows (0, 1) and (2, 3) share the float instructions (mul / fma .f32x2: two independent round-to-nearest operations)
    for (int t0 = 0; t0 < ntok; t0 += 4) {
        const int2 *xpt[4];
        unsigned long long acc2[2] = {0ull, 0ull};
#pragma unroll
        for (int g = 0; g < 4; g++) xpt[g] = xp + (size_t)min(t0 + g, ntok - 1) * nidx + c8;      // rows past the end repeat the last one (never stored)
        const float *xst = xsc + (size_t)p * QR_TPC + t0;          // scales of rows t0 .. t0 + 3 for block 2 i + p at + 2 i * QR_TPC (rows past the end: stale, never stored)
        auto step = [&](int2 wv, float sv, int i) {
            const unsigned long long s2 = qr_pack2(sv, sv);
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int2 xa = xpt[2 * h][i * 8], xb = xpt[2 * h + 1][i * 8];
                const int da = __dp4a(wv.y, xa.y, __dp4a(wv.x, xa.x, 0)), db = __dp4a(wv.y, xb.y, __dp4a(wv.x, xb.x, 0));
                const unsigned long long sx2 = qr_mul2(s2, *reinterpret_cast<const unsigned long long *>(xst + (size_t)2 * i * QR_TPC + 2 * h));
                acc2[h] = qr_fma2(qr_pack2((float)da, (float)db), sx2, acc2[h]);
            }
        };
        if (NP > 0) {
#pragma unroll
            for (int i = 0; i < (NP > 0 ? NP : 1); i++) step(w[i], s[i], i);
        } else {
            for (int i = 0; i < np; i++) step(__ldg(wp + (size_t)i * (Q8_UNIT / 8)), __ldg(sp + (size_t)i * (Q8_UNIT / 4)), i);
        }
        float acc[4];
        qr_unpack2(acc2[0], acc[0], acc[1]);
        qr_unpack2(acc2[1], acc[2], acc[3]);
#pragma unroll
        for (int g = 0; g < 4; g++) {
            float r = __fadd_rn(acc[g], __shfl_xor_sync(0xffffffffu, acc[g], 4));      // acc_even + acc_odd per lane, then (l0+l1)+(l2+l3)
            r = brrr_hsum4(r);
            if (out && t0 + g < ntok) {
                float *yp = a.y + (size_t)(t_first + t0 + g) * a.ldy + row;
                if (EPI == Q8_EPI_PLAIN) *yp = r;
                else if (EPI == Q8_EPI_BIAS) *yp = __fadd_rn(r, bias_pre);
                else *yp = __fadd_rn(*yp, __fadd_rn(r, bias_pre));                // x += dot + bias
            }
        }
    }
}

template <int NP>
cudaError_t q8_rows_launch(const Q8RowsArgs &a, int epi, dim3 grid, size_t smem, bool pdl, cudaStream_t st) {
    static unsigned long long configured[3] = {0, 0, 0};
    cudaError_t e;
    switch (epi) {
    case Q8_EPI_PLAIN:
        if ((e = smem_optin(q8_rows_kernel<Q8_EPI_PLAIN, NP>, 160 * 1024, configured[0])) != cudaSuccess) return e;
        return launch_k(q8_rows_kernel<Q8_EPI_PLAIN, NP>, grid, dim3(QR_THREADS), smem, st, pdl, a);
    case Q8_EPI_BIAS:
        if ((e = smem_optin(q8_rows_kernel<Q8_EPI_BIAS, NP>, 160 * 1024, configured[1])) != cudaSuccess) return e;
        return launch_k(q8_rows_kernel<Q8_EPI_BIAS, NP>, grid, dim3(QR_THREADS), smem, st, pdl, a);
    case Q8_EPI_RESID_BIAS:
        if ((e = smem_optin(q8_rows_kernel<Q8_EPI_RESID_BIAS, NP>, 160 * 1024, configured[2])) != cudaSuccess) return e;
        return launch_k(q8_rows_kernel<Q8_EPI_RESID_BIAS, NP>, grid, dim3(QR_THREADS), smem, st, pdl, a);
    }
    return cudaErrorInvalidValue;
}

// RoPE of k (NeoX halves, the same operations as attn_decode_kernel) and the cache append of k and v for every row.
struct KvRowsArgs {
    const float *qkv;        // [rows][ldq]: q | k | v of every row, bias added, not rotated
    int ldq, nh, nkv;
    float *kc, *vc;          // [sequence][nkv][MAXSEQ][64]
    size_t seq_stride;       // floats between two sequences' caches
    const float *rope;
    const int *row_pos, *row_seq;
};

__global__ void __launch_bounds__(64) kv_append_rows_kernel(KvRowsArgs a) {
    const int kvh = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, i = tid & 31;
    const int pos = a.row_pos[t];
    const float c = a.rope[((size_t)pos * 32 + i) * 2], s = a.rope[((size_t)pos * 32 + i) * 2 + 1];
    pdl_wait();
    pdl_trigger();
    const float *k = a.qkv + (size_t)t * a.ldq + (size_t)(a.nh + kvh) * 64, *v = k + (size_t)a.nkv * 64;
    const size_t o = (size_t)a.row_seq[t] * a.seq_stride + ((size_t)kvh * BRRR_MAXSEQ + pos) * 64;
    const float x0 = k[i], x1 = k[32 + i];
    if (tid < 32) a.kc[o + i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    else a.kc[o + 32 + i] = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
    a.vc[o + tid] = v[tid];
}

// Index of the largest logit of every row, the lowest index among equals: the same 64-bit key (ordered float bits,
// inverted index) the one-token head folds with atomicMax.  One CTA per row.
__global__ void __launch_bounds__(1024) rows_argmax_kernel(const float *__restrict__ logits, int n_vocab, uint32_t *__restrict__ out) {
    __shared__ unsigned long long wbest[32];
    const float *row = logits + (size_t)blockIdx.x * n_vocab;
    unsigned long long best = 0ull;
    for (int i = threadIdx.x; i < n_vocab; i += 1024) {
        const unsigned long long key = ((unsigned long long)float_orderable(row[i]) << 32) | (0xFFFFFFFFu - (uint32_t)i);
        best = key > best ? key : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) wbest[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 32; w++) best = wbest[w] > best ? wbest[w] : best;
        out[blockIdx.x] = 0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull);
    }
}

}  // namespace

void launch_rows_argmax(const float *logits, int n_vocab, int rows, uint32_t *out, cudaStream_t st) {
    rows_argmax_kernel<<<rows, 1024, 0, st>>>(logits, n_vocab, out);
}

// y[t][r] (+)= row r of m . activation t (+ bias) for t < ntok <= BRRR_TILE_MAX.  epi: Q8_EPI_PLAIN / BIAS / RESID_BIAS.
// engine: 0 = integer units (the default: measured faster at every tile size so far), 1 = tensor cores (launch_q8_tile,
// kernels_tile.cu), -1 = the environment variable BRRR_Q8_TILE=1 selects the tensor cores for tiles of at least 32 rows of
// the layer projections.  Same bits either way.
cudaError_t launch_q8_rows(Q8Dev m, const int8_t *xq, const float *xs, int ntok, const float *bias, float *y, int ldy, int epi, bool pdl,
                           cudaStream_t st, DevState *state, int engine) {
    if (ntok < 1 || ntok > BRRR_TILE_MAX || m.cols % 64) return cudaErrorInvalidValue;
    static const bool env_tile = [] { const char *e = getenv("BRRR_Q8_TILE"); return e && e[0] && e[0] != '0'; }();
    const bool tile = engine == 1 || (engine < 0 && env_tile && ntok >= 32 && m.rows <= 16384);
    if (tile) return launch_q8_tile(m, xq, xs, ntok, bias, y, ldy, epi, state, pdl, st);
    Q8RowsArgs a{m, xq, xs, bias, y, ntok, ldy};
    const int np = m.cols / 64, urows = q8_urows(m.rows);
    const size_t smem = (size_t)QR_TPC * np * 72;
    const dim3 grid((unsigned)urows, (unsigned)((ntok + QR_TPC - 1) / QR_TPC));
    if (np == 45) return q8_rows_launch<45>(a, epi, grid, smem, pdl, st);
    if (np == 64) return q8_rows_launch<64>(a, epi, grid, smem, pdl, st);
    return q8_rows_launch<0>(a, epi, grid, smem, pdl, st);
}

cudaError_t launch_kv_append_rows(const float *qkv, int ldq, int nh, int nkv, float *kc, float *vc, size_t seq_stride, const float *rope,
                                  const int *row_pos, const int *row_seq, int rows, bool pdl, cudaStream_t st) {
    KvRowsArgs a{qkv, ldq, nh, nkv, kc, vc, seq_stride, rope, row_pos, row_seq};
    return launch_k(kv_append_rows_kernel, dim3(nkv, rows), dim3(64), 0, st, pdl, a);
}

}  // namespace brrr
