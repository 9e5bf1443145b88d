// Host-callable launchers of the decode kernels.  Every launcher only enqueues work on the given
// stream (capturable into a CUDA graph) and reports launch-configuration errors through
// cudaGetLastError at the call site.
#pragma once
#include "brrr_dev.cuh"

namespace brrr {

// ---- elementwise / small stages (kernels_small.cu)
void launch_quant_q8(const float *x, int n, int8_t *q, float *s, cudaStream_t st);
// rows > 1: one CTA per row; rows are n apart in x / xn / q and n / 32 apart in s
cudaError_t launch_rmsnorm_quant(const float *x, const float *w, float eps, int n, float *xn, int8_t *q, float *s, bool pdl, cudaStream_t st,
                                 int rows = 1);
// ---- token rows (kernels_rows.cu): y[t][r] (+)= row r of m . activation t (+ bias), t < ntok <= 16
cudaError_t launch_q8_rows(Q8Dev m, const int8_t *xq, const float *xs, int ntok, const float *bias, float *y, int ldy, int epi, bool pdl,
                           cudaStream_t st, DevState *state = nullptr, int engine = -1);
// RoPE of every row's k and the cache append of k and v (row t: position row_pos[t] of sequence row_seq[t])
cudaError_t launch_kv_append_rows(const float *qkv, int ldq, int nh, int nkv, float *kc, float *vc, size_t seq_stride, const float *rope,
                                  const int *row_pos, const int *row_seq, int rows, bool pdl, cudaStream_t st);
void launch_embed(const uint16_t *embd, int d, const DevState *state, float *x, cudaStream_t st);
void launch_embed_tok(const uint16_t *embd, int d, uint32_t tok, float *x, cudaStream_t st);
// ntok rows from token ids in device memory: x[t] = embedding of toks[t]
void launch_rows_argmax(const float *logits, int n_vocab, int rows, uint32_t *out, cudaStream_t st);   // out[t] = first index of the largest logit of row t
void launch_embed_tile(const uint16_t *embd, int d, const uint32_t *toks_dev, int ntok, float *x, cudaStream_t st);
void launch_swiglu_quant(const float *gu, int topk, int d, int8_t *hq, float *hs, cudaStream_t st);
void launch_finish_token(DevState *state, cudaStream_t st);
void launch_expf(const float *x, int n, float *y, cudaStream_t st);
// first_elem: index of the first generated element within the whole tensor (MXFP4 only; a multiple of 32)
void launch_synth(uint64_t seed, uint32_t layer, uint32_t kind, uint32_t type, uint64_t nelems, void *out, cudaStream_t st, uint64_t first_elem = 0);

// ---- K-quants of the qwen3moe path (kernels_kq.cu): weights stay in the GGUF byte layout
void launch_quant_q8k(const float *x, int n, int8_t *q, float *s, int32_t *bsum, cudaStream_t st);
void launch_q4k_matvec(const uint8_t *w, int rows, int cols, const int8_t *xq, const float *ys, const int32_t *bsum, float *y,
                       int32_t *dbg, cudaStream_t st);
void launch_q6k_matvec(const uint8_t *w, int rows, int cols, const int8_t *xq, const float *ys, float *y, int32_t *dbg, cudaStream_t st);

// ---- qwen3moe decode kernels (kernels_qwen.cu); KMatDev is declared in brrr_kq.cuh
struct KMatDev;
cudaError_t launch_qw_embed(const uint8_t *embd_q4k, int d, const DevState *state, float *x, bool pdl, cudaStream_t st);
cudaError_t launch_qw_norm_quant(const float *x, const float *w, float eps, int d, float *xn, int8_t *q, float *s, int32_t *bsum,
                                 bool pdl, cudaStream_t st);
// mats: up to three matrices of equal width stacked row-wise (q | k | v); weights are fetched into registers before the
// dependency wait.  pf_k / pf_v (nullable): K/V cache of the attention that follows, requested into L2 up to state->pos.
cudaError_t launch_qw_matvec(const KMatDev *mats, float *const *ys_out, int n, bool resid, const int8_t *xq, const float *ys,
                             const int32_t *bsum, bool pdl, cudaStream_t st, const float *pf_k = nullptr, const float *pf_v = nullptr,
                             int pf_nkv = 0, const DevState *state = nullptr);
cudaError_t launch_qw_qknorm_rope(float *q, const float *k, const float *v, const float *q_norm, const float *k_norm, const float *rope,
                                  float eps, int nh, int nkv, const DevState *state, int pos_val, float *kc, float *vc, bool pdl,
                                  cudaStream_t st);
// attention of all heads (two per CTA) and the Q8_K image of its output (aq, as per 256, asum per 32)
cudaError_t launch_qw_attn(const float *q, const float *kc, const float *vc, int nh, int nkv, const DevState *state, int pos_val, int8_t *aq,
                           float *as, int32_t *asum, bool pdl, cudaStream_t st);
cudaError_t launch_qw_gate_up(const KMatDev &gate, const KMatDev &up, const int32_t *top, int topk, int ff, const int8_t *xq, const float *ys,
                              const int32_t *bsum, float *hbuf, bool pdl, cudaStream_t st);
// hbuf: [topk][ff] floats of h (quantised in the kernel's prologue); counter: one zeroed word; next_norm_w (nullable): the last CTA
// to finish writes the Q8_K image (nq, ns, nsum) of RMSNorm(x, next_norm_w)
cudaError_t launch_qw_down(const KMatDev &down, const int32_t *top, const float *wts, int topk, int d, int ff, const float *hbuf, float *x,
                           unsigned int *counter, const float *next_norm_w, float eps, int8_t *nq, float *ns, int32_t *nsum, bool pdl,
                           cudaStream_t st);
cudaError_t launch_qw_head(const KMatDev &head, const int8_t *xq, const float *ys, const int32_t *bsum, float *logits, DevState *state,
                           bool pdl, cudaStream_t st);
// Q6_K rows from the GGUF layout (210-byte superblocks) into the aligned planes of KMatDev (planes = 1)
void launch_q6k_planes(const uint8_t *src, size_t rows, int cols, uint8_t *dst, cudaStream_t st);
char *host_err_buf();   // thread-local text behind brrr_last_cuda_error (512 bytes)

// ---- Q8 matrices (kernels_q8.cu)
void launch_q8_pack(const uint16_t *w_bf16, int rows_src, int row0_dst, Q8Dev m, cudaStream_t st);
void launch_q8_export(Q8Dev m, int8_t *q, float *s, cudaStream_t st);
enum { Q8_EPI_PLAIN = 0, Q8_EPI_BIAS = 1, Q8_EPI_RESID_BIAS = 2, Q8_EPI_HEAD = 3 };
// Streaming GEMV.  x_f32 != nullptr: RMSNorm(x_f32, norm_w, eps) + Q8 quantisation in the prologue;
// otherwise the Q8 activation (xq, xs) is used.  pdl: launch with programmatic stream serialization.
cudaError_t launch_q8_stream(Q8Dev m, const float *x_f32, const float *norm_w, float eps, const int8_t *xq, const float *xs,
                             const float *bias, float *y, int epi, DevState *state, bool pdl, cudaStream_t st,
                             const float *pf_k = nullptr, const float *pf_v = nullptr, int pf_nkv = 0, int pf_window = 0);

// Direct-from-global GEMV for very large matrices (the vocabulary head); activation pre-quantised.
cudaError_t launch_q8_direct(Q8Dev m, const int8_t *xq, const float *xs, const float *bias, float *y, int epi, DevState *state, bool pdl, cudaStream_t st);
cudaError_t launch_q8_head(Q8Dev m, const int8_t *xq, const float *xs, float *y, DevState *state, bool pdl, cudaStream_t st);

// ---- MXFP4 matrices (kernels_mx.cu)
void launch_mx_pack(const uint8_t *raw, MxDev m, cudaStream_t st);
void launch_mx_gemv(MxDev m, int row0, int nrows, const int8_t *xq, const float *xs, float *y, int32_t *blockdots, cudaStream_t st);
// gate/up of the selected experts + clamped SwiGLU + Q8 of h.  Activation: x_f32 with norm_w
// (RMSNorm + quantise), x_f32 without norm_w (quantise only), or (xq, xs).  gu nullable.
cudaError_t launch_gate_up(MxDev gate, MxDev up, const float *gate_b, const float *up_b, const int32_t *top, int topk, int d,
                           const float *x_f32, const float *norm_w, float eps, const int8_t *xq, const float *xs,
                           int8_t *hq, float *hs, float *gu, DevState *state, bool pdl, cudaStream_t st,
                           const float *est = nullptr, int ne = 0, int e_lo = 0, int e_cnt = 1 << 30);
// e_lo, e_cnt: the matrices hold experts [e_lo, e_lo + e_cnt) only (biases stay indexed by the
// global expert id); CTAs of slots whose expert lives elsewhere return at once.
// est (nullable): slot s of hq/hs belongs to the s-th largest of the router estimate est[0..ne)
// rather than to top[s]; a step whose
// exact experts are not all among them is flagged in state->spec_fail_step.
cudaError_t launch_down_combine(MxDev down, const float *down_b, const int32_t *top, const float *wts, const float *est, int ne,
                                int topk, int d, const int8_t *hq, const float *hs, float *x, DevState *state, bool pdl, cudaStream_t st);

// ---- expert parallelism over NVLink peer memory (kernels_ep.cu)
constexpr int EP_MAX_WORLD = 8;
struct EpCtx {
    int rank, world, e_lo, e_cnt;          // experts [e_lo, e_lo + e_cnt) live on this rank
    uint32_t *epoch;                       // local: number of the step in flight
    float *xchg[EP_MAX_WORLD];             // every rank's exchange buffer [layer][slot][d]
    uint32_t *flags[EP_MAX_WORLD];         // every rank's slice flags [layer][slot][d / 16]
    uint32_t *done[EP_MAX_WORLD];          // every rank's completed-step counters [world]
    // speculative step: every rank's buffer of self-validating row sums [layer][slot][d], one 64-bit
    // word each = (step number << 32) | float bits, written with one store: no flag, no fence
    unsigned long long *pairs[EP_MAX_WORLD];
};
// ---- single-token expert matvecs on the tensor cores in native fp4 (kernels_mxt.cu)
// Tile units: [expert][tile of 128 rows][block pair][4096 B operand image | 128 x 2 e8m0 bytes].
constexpr int MXT_UNIT = 4352;
constexpr int MXT_UNIT_EXPS = 4096;
struct MxtDev {
    uint8_t *data;
    int tiles_per_expert, np;
};
size_t mxt_bytes(int experts, int tiles_per_expert, int np);
// b.data == nullptr: tiles of 128 rows of a (rows past the end are zero); else rows 0-63 of a tile
// come from a and rows 64-127 from b (same 64 row indices)
void launch_mxt_pack(MxDev a, MxDev b, int experts, int rows_per_expert, MxtDev out, cudaStream_t st);
// The activation enters as its digit-plane operand image (brrr_mxt.cuh; [blocks / 2][768] bytes, zero
// except for the words its producer writes) and its block scales.
void launch_xt_bimg(const int8_t *xq, int nb, uint8_t *bimg, cudaStream_t st);
// same results, bit for bit, as launch_gate_up / launch_down_combine on the same Q8 activation;
// himg: [topk][blocks / 2][768] operand images of h for launch_down_t
cudaError_t launch_gate_up_t(MxtDev gu, const float *gate_b, const float *up_b, const int32_t *top, const float *est, int ne, int topk,
                             int d, const uint8_t *ximg, const float *xs, int8_t *hq, float *hs, uint8_t *himg, DevState *state,
                             bool pdl, cudaStream_t st, const EpCtx *ep = nullptr, int layer = 0);
// part: [topk][tiles_per_expert * 128] floats of scratch; counter: [tiles_per_expert] words, zero before the first launch.
// wts != nullptr (exact routing in top/wts, est == nullptr): the last CTA of a row tile folds it onto x.
// wts == nullptr: slot s is the s-th largest entry of est (or top[s]); only part[] is written and
// launch_down_fold finishes the step once the exact routing is there.
cudaError_t launch_down_fold(const int32_t *top, const float *wts, const float *est, int ne, int topk, int d, const float *part,
                             const float *down_b, float *x, DevState *state, bool pdl, cudaStream_t st);
// The fold for a step whose exact router runs on another stream: one CTA waits (bounded) until
// *router_seq == *fold_seq + 1, folds as launch_down_fold, then RMS-normalises the new residual with
// next_norm_w and writes its Q8 image (nq natural int8 order, ns block scales) for the projection
// that follows, and increments *fold_seq.  next_norm_w == nullptr: fold only.
cudaError_t launch_fold_norm(const int32_t *top, const float *wts, const float *est, int ne, int topk, int d, const float *part,
                             const float *down_b, float *x, const float *next_norm_w, float eps, int8_t *nq, float *ns,
                             uint32_t *router_seq, uint32_t *fold_seq, DevState *state, bool pdl, cudaStream_t st,
                             const EpCtx *ep = nullptr, int layer = 0);
cudaError_t launch_down_t(MxtDev down, const float *down_b, const int32_t *top, const float *wts, const float *est, int ne, int topk,
                          int d, const uint8_t *himg, const float *hs, float *x, float *part, uint32_t *counter, DevState *state,
                          bool pdl, cudaStream_t st, const EpCtx *ep = nullptr, int layer = 0);

// ---- token-tile matmul on tcgen05 tensor cores (kernels_tile.cu): y[t][r] = row (row0 + r) . activation t,
// t < ntok <= BRRR_TILE_MAX, every value bit-identical to launch_mx_gemv on token t alone
cudaError_t launch_mx_tile(MxDev w, int row0, int nrows, const int8_t *xq, const float *xs, int ntok, float *y, int ldy, DevState *state,
                           cudaStream_t st);

// every expert of one matrix kind against the (token, slot) entries routed to it (cnt[e], list[e][BRRR_TILE_MAX], at most max_entries per expert);
// entry i reads activation row entry / src_div and writes y[entry * ldy + col0 + row] (+ bias[e][row])
cudaError_t launch_mx_tile_experts(MxDev w, int ne, int rows_per_expert, const int *cnt, const int *list, int max_entries, int src_div, const int8_t *xq,
                                   const float *xs, const float *bias, float *y, int ldy, int col0, DevState *state, cudaStream_t st);
cudaError_t launch_q8_tile(Q8Dev m, const int8_t *xq, const float *xs, int ntok, const float *bias, float *y, int ldy, int epi, DevState *state,
                           bool pdl, cudaStream_t st);          // Q8 matrix x token rows on kind::i8 (kernels_tile.cu)
void launch_tile_route(const int32_t *top, int ntok, int topk, int ne, int *cnt, int *list, cudaStream_t st);
void launch_tile_combine(const float *part, const float *wts, int topk, int d, int ntok, float *x, cudaStream_t st);

void launch_ep_begin(const EpCtx &c, DevState *state, cudaStream_t st);
// down-projection of the local experts, exchange of the 16-row slices, fold in slot order
cudaError_t launch_down_ep(MxDev down, const float *down_b, const int32_t *top, const float *wts, int topk, int d, int layer, const int8_t *hq,
                           const float *hs, float *x, DevState *state, const EpCtx &ep, bool pdl, cudaStream_t st);

// ---- router (kernels_router.cu)
// The router matrix is used in a tiled layout: [32-expert group][tile][32][RT_STRIDE] floats.
constexpr int RT_TJ = 256;                       // tile width (elements of d)
constexpr int RT_STRIDE = RT_TJ + 4;             // padded row stride in floats
constexpr int RT_TILE_FLOATS = 32 * RT_STRIDE;
size_t router_packed_floats(int ne, int d);
void launch_router_pack(const float *W, int ne, int d, float *out, cudaStream_t st);
// x_in is the residual stream when norm_w != nullptr (RMSNorm applied first) or an already
// normalised vector otherwise.
cudaError_t launch_ffn_in(const float *x_in, const float *norm_w, float eps, int d, const float *Wt, const float *b, int ne, int topk,
                          float *logits, int32_t *top, float *wts, unsigned int *counter, DevState *state, bool pdl, cudaStream_t st,
                          int ntok = 1, uint32_t *signal = nullptr, int qwen_norm = 0, int8_t *q8k_q = nullptr, float *q8k_s = nullptr,
                          int32_t *q8k_bsum = nullptr);
// ntok > 1: a tile of tokens in one launch (token t reads x_in + t * d, writes logits + t * ne, top + 8 t, wts + 8 t, uses counter + t)
// signal (nullable, ntok == 1): a device word the kernel increments after its routing is written, for a
// consumer that runs beside it instead of after it (launch_fold_norm)

// Order-free estimate of the router used only to start the gate/up weight stream early
// (speculative routing): est[ne] receives the estimated logits, xq_out/xs_out the Q8 image of the
// normalised vector (each CTA writes a share).
cudaError_t launch_router_hint(const float *x_in, const float *norm_w, float eps, int d, const float *Wt, const float *b, int ne, int topk,
                               float *est, int8_t *xq_out, float *xs_out, DevState *state, bool pdl, cudaStream_t st,
                               uint8_t *bimg_out = nullptr);
// bimg_out (nullable): also the operand image of the quantised vector for the tensor-core expert kernels

// ---- attention (kernels_attn.cu)
// KV cache layout [n_head_kv][BRRR_MAXSEQ][64].  pos is read from state when state != nullptr,
// else pos_val.  window = 0 means full attention.
cudaError_t launch_attn_rows(const float *qkv, int ldq, const float *kc, const float *vc, size_t seq_stride, const float *rope, const float *sinks,
                             int nh, int nkv, int window, const int *row_pos, const int *row_seq, int rows, float *ao, int8_t *aq, float *as,
                             DevState *err_state, bool pdl, cudaStream_t st);       // rows of one sequence share their K / V tiles (prompt tiles)
cudaError_t launch_attn_decode(const float *qkv, float *kc, float *vc, const float *rope, const float *sinks, int nh, int nkv,
                               const DevState *state, int pos_val, int window, float *ao, int8_t *aq, float *as,
                               DevState *err_state, bool pdl, cudaStream_t st, int pos_off = 0, const int *row_pos = nullptr,
                               const int *row_seq = nullptr, size_t seq_stride = 0, int ldq = 0, int rows = 1);
// row_pos != nullptr: `rows` tokens in one launch (grid.y), see AttnArgs in kernels_attn.cu; the rows' k / v must be in the cache already
// pos_off is added to the position read from state (ignored with pos_val)

}  // namespace brrr
