// Stage-level C ABI (include/brrr.h): device pointers in, device pointers out.  Each function
// launches the same kernel the forward pass uses for that stage.
#include "../../include/brrr.h"
#include "brrr_kernels.h"

#include <cstdio>

using namespace brrr;

namespace {
int check_launch() { return cudaGetLastError() == cudaSuccess ? BRRR_OK : BRRR_ERR_CUDA; }
}  // namespace

struct brrr_q8mat { Q8Dev m; };
struct brrr_mxmat { MxDev m; };

extern "C" int brrr_quant_q8(const float *d_x, int n, int8_t *d_q, float *d_s, void *stream) {
    if (!d_x || !d_q || !d_s || n <= 0 || n % 32) return BRRR_ERR_ARG;
    launch_quant_q8(d_x, n, d_q, d_s, (cudaStream_t)stream);
    return check_launch();
}

extern "C" int brrr_quant_q8k(const float *d_x, int n, int8_t *d_q, float *d_s, int32_t *d_bsum, void *stream) {
    if (!d_x || !d_q || !d_s || !d_bsum || n <= 0 || n % 256) return BRRR_ERR_ARG;
    if (((uintptr_t)d_x & 15) || ((uintptr_t)d_q & 7)) return BRRR_ERR_ARG;
    launch_quant_q8k(d_x, n, d_q, d_s, d_bsum, (cudaStream_t)stream);
    return check_launch();
}

extern "C" int brrr_q4k_matvec(const uint8_t *d_w, int rows, int cols, const int8_t *d_xq, const float *d_ys, const int32_t *d_bsum,
                               float *d_y, int32_t *d_sbdots, void *stream) {
    if (!d_w || !d_xq || !d_ys || !d_bsum || !d_y || rows <= 0 || cols <= 0 || cols % 256) return BRRR_ERR_ARG;
    if (((uintptr_t)d_w & 3) || ((uintptr_t)d_xq & 3)) return BRRR_ERR_ARG;
    launch_q4k_matvec(d_w, rows, cols, d_xq, d_ys, d_bsum, d_y, d_sbdots, (cudaStream_t)stream);
    return check_launch();
}

extern "C" int brrr_q6k_matvec(const uint8_t *d_w, int rows, int cols, const int8_t *d_xq, const float *d_ys, float *d_y,
                               int32_t *d_sbdots, void *stream) {
    if (!d_w || !d_xq || !d_ys || !d_y || rows <= 0 || cols <= 0 || cols % 256) return BRRR_ERR_ARG;
    if (((uintptr_t)d_w & 1) || ((uintptr_t)d_xq & 1)) return BRRR_ERR_ARG;
    launch_q6k_matvec(d_w, rows, cols, d_xq, d_ys, d_y, d_sbdots, (cudaStream_t)stream);
    return check_launch();
}

extern "C" int brrr_rmsnorm_quant(const float *d_x, const float *d_w, float eps, int n, float *d_xn, int8_t *d_q, float *d_s, void *stream) {
    if (!d_x || !d_w || !d_q || !d_s || n <= 0 || n % 32 || n > 8192) return BRRR_ERR_ARG;
    if (launch_rmsnorm_quant(d_x, d_w, eps, n, d_xn, d_q, d_s, false, (cudaStream_t)stream) != cudaSuccess) return BRRR_ERR_CUDA;
    return check_launch();
}

extern "C" int brrr_q8mat_from_bf16(const uint16_t *d_w, int rows, int cols, brrr_q8mat **out, void *stream) {
    if (!d_w || !out || rows <= 0 || cols <= 0 || cols % 64 || cols > 4096) return BRRR_ERR_ARG;
    brrr_q8mat *q = new brrr_q8mat();
    q->m.rows = rows; q->m.cols = cols;
    if (cudaMalloc(&q->m.data, q8_bytes(rows, cols)) != cudaSuccess) { delete q; return BRRR_ERR_NOMEM; }
    if (cudaMemsetAsync(q->m.data, 0, q8_bytes(rows, cols), (cudaStream_t)stream) != cudaSuccess) { cudaFree(q->m.data); delete q; return BRRR_ERR_CUDA; }
    launch_q8_pack(d_w, rows, 0, q->m, (cudaStream_t)stream);
    *out = q;
    return check_launch();
}

extern "C" int brrr_q8mat_export(const brrr_q8mat *m, int8_t *d_q, float *d_s, void *stream) {
    if (!m || !d_q || !d_s) return BRRR_ERR_ARG;
    launch_q8_export(m->m, d_q, d_s, (cudaStream_t)stream);
    return check_launch();
}

extern "C" void brrr_q8mat_free(brrr_q8mat *m) {
    if (!m) return;
    cudaFree(m->m.data);
    delete m;
}

extern "C" int brrr_q8_matvec(const brrr_q8mat *w, const int8_t *d_xq, const float *d_xs, float *d_y, void *stream) {
    if (!w || !d_xq || !d_xs || !d_y) return BRRR_ERR_ARG;
    if (launch_q8_stream(w->m, nullptr, nullptr, 0.0f, d_xq, d_xs, nullptr, d_y, Q8_EPI_PLAIN, nullptr, false, (cudaStream_t)stream) != cudaSuccess) return BRRR_ERR_CUDA;
    return check_launch();
}

extern "C" int brrr_q8_matmul_rows(const brrr_q8mat *w, const int8_t *d_xq, const float *d_xs, int ntok, float *d_y, int ldy, int tensor_cores,
                                   void *stream) {
    if (!w || !d_xq || !d_xs || !d_y || ntok < 1 || ntok > BRRR_TILE_MAX || ldy < w->m.rows) return BRRR_ERR_ARG;
    if (launch_q8_rows(w->m, d_xq, d_xs, ntok, nullptr, d_y, ldy, Q8_EPI_PLAIN, false, (cudaStream_t)stream, nullptr, tensor_cores ? 1 : 0) != cudaSuccess)
        return BRRR_ERR_CUDA;
    return check_launch();
}

extern "C" int brrr_mxmat_from_gguf(const uint8_t *d_raw, int rows, int blocks, brrr_mxmat **out, void *stream) {
    if (!d_raw || !out || rows <= 0 || rows % 16 || blocks <= 0 || blocks % 2) return BRRR_ERR_ARG;
    brrr_mxmat *x = new brrr_mxmat();
    x->m.rows = rows; x->m.blocks = blocks;
    if (cudaMalloc(&x->m.data, mx_bytes(rows, blocks)) != cudaSuccess) { delete x; return BRRR_ERR_NOMEM; }
    launch_mx_pack(d_raw, x->m, (cudaStream_t)stream);
    *out = x;
    return check_launch();
}

extern "C" void brrr_mxmat_free(brrr_mxmat *m) {
    if (!m) return;
    cudaFree(m->m.data);
    delete m;
}

extern "C" int brrr_mx_matvec(const brrr_mxmat *w, int row0, int nrows, const int8_t *d_xq, const float *d_xs, float *d_y, int32_t *d_blockdots, void *stream) {
    if (!w || !d_xq || !d_xs || !d_y || row0 < 0 || nrows <= 0 || row0 + nrows > w->m.rows) return BRRR_ERR_ARG;
    launch_mx_gemv(w->m, row0, nrows, d_xq, d_xs, d_y, d_blockdots, (cudaStream_t)stream);
    return check_launch();
}

extern "C" int brrr_mx_matmul_tile(const brrr_mxmat *w, int row0, int nrows, const int8_t *d_xq, const float *d_xs, int ntok, float *d_y, int ldy,
                                   void *stream) {
    if (!w || !d_xq || !d_xs || !d_y || row0 < 0 || nrows <= 0 || row0 + nrows > w->m.rows || ntok < 1 || ntok > BRRR_TILE_MAX || ldy < nrows) return BRRR_ERR_ARG;
    if (((uintptr_t)d_xq & 3)) return BRRR_ERR_ARG;
    if (launch_mx_tile(w->m, row0, nrows, d_xq, d_xs, ntok, d_y, ldy, nullptr, (cudaStream_t)stream) != cudaSuccess) return BRRR_ERR_CUDA;
    return check_launch();
}

extern "C" int brrr_router_topk(const float *d_w, const float *d_b, const float *d_xn, int ne, int d, int topk,
                                float *d_logits, int32_t *d_top, float *d_wts, void *stream) {
    if (!d_w || !d_xn || !d_logits || !d_top || !d_wts || ne <= 0 || d <= 0 || topk <= 0 || topk > 8 || topk > ne) return BRRR_ERR_ARG;
    if (ne > 256 || d > 4096) return BRRR_ERR_RANGE;      // the top-k keeps 8 experts per lane; d floats of x and of norm weights share the CTA's shared memory with the tile ring
    if (d % 64) return BRRR_ERR_ARG;
    // arrival counter of the router CTAs (self-resetting), one per device
    static unsigned int *counters[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BRRR_ERR_CUDA;
    if (!counters[dev]) {
        if (cudaMalloc(&counters[dev], sizeof(unsigned int)) != cudaSuccess) return BRRR_ERR_NOMEM;
        if (cudaMemset(counters[dev], 0, sizeof(unsigned int)) != cudaSuccess) return BRRR_ERR_CUDA;
    }
    unsigned int *counter = counters[dev];
    // stage-level call: re-lay the natural [ne][d] matrix into the tiled form first
    float *wt = nullptr;
    if (cudaMalloc(&wt, router_packed_floats(ne, d) * sizeof(float)) != cudaSuccess) return BRRR_ERR_NOMEM;
    launch_router_pack(d_w, ne, d, wt, (cudaStream_t)stream);
    cudaError_t e = launch_ffn_in(d_xn, nullptr, 0.0f, d, wt, d_b, ne, topk, d_logits, d_top, d_wts, counter, nullptr, false, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    cudaFree(wt);
    return e == cudaSuccess ? check_launch() : BRRR_ERR_CUDA;
}

extern "C" int brrr_swiglu_quant(const float *d_gu, int topk, int d, int8_t *d_hq, float *d_hs, void *stream) {
    if (!d_gu || !d_hq || !d_hs || topk <= 0 || d <= 0 || d % 32) return BRRR_ERR_ARG;
    launch_swiglu_quant(d_gu, topk, d, d_hq, d_hs, (cudaStream_t)stream);
    return check_launch();
}

extern "C" int brrr_attn_decode(const float *d_qkv, float *d_kc, float *d_vc, const float *d_rope, const float *d_sinks,
                                int n_head, int n_head_kv, int pos, int start, float *d_ao, int8_t *d_aq, float *d_as, void *stream) {
    if (!d_qkv || !d_kc || !d_vc || !d_rope || !d_sinks || !d_ao || !d_aq || !d_as) return BRRR_ERR_ARG;
    if (n_head <= 0 || n_head_kv <= 0 || n_head % n_head_kv || pos < 0 || pos >= BRRR_MAXSEQ || start < 0 || start > pos) return BRRR_ERR_ARG;
    int window = start > 0 ? pos - start + 1 : 0;
    if (launch_attn_decode(d_qkv, d_kc, d_vc, d_rope, d_sinks, n_head, n_head_kv, nullptr, pos, window, d_ao, d_aq, d_as, nullptr, false, (cudaStream_t)stream) != cudaSuccess) return BRRR_ERR_CUDA;
    return check_launch();
}

extern "C" int brrr_synth_tensor(uint64_t seed, uint32_t layer, uint32_t kind, uint32_t type, uint64_t nelems, void *d_out, void *stream) {
    if (!d_out || (type != 0 && type != 30 && type != 39) || (type == 39 && nelems % 32)) return BRRR_ERR_ARG;
    launch_synth(seed, layer, kind, type, nelems, d_out, (cudaStream_t)stream);
    return check_launch();
}

extern "C" int brrr_expf(const float *d_x, int n, float *d_y, void *stream) {
    if (!d_x || !d_y || n <= 0) return BRRR_ERR_ARG;
    launch_expf(d_x, n, d_y, (cudaStream_t)stream);
    return check_launch();
}

// The last kernel of a layer in the default decode step, as a stage: fold of the down-projection
// partial sums with the exact routing, then RMS norm + Q8 of the new residual.
extern "C" int brrr_fold_norm(const int32_t *d_top, const float *d_wts, int topk, int d, const float *d_part, const float *d_down_b, float *d_x,
                              const float *d_norm_w, float eps, int8_t *d_q, float *d_s, int wait_for_router, void *stream) {
    if (!d_top || !d_wts || !d_part || !d_down_b || !d_x || topk <= 0 || topk > 8 || d <= 0 || d % 32 || d > 4096) return BRRR_ERR_ARG;
    if (d_norm_w && (!d_q || !d_s)) return BRRR_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    // a private device state: the kernel reports a wait that ran out through its error word
    DevState *state = nullptr;
    if (cudaMalloc(&state, sizeof(DevState)) != cudaSuccess) return BRRR_ERR_NOMEM;
    int rc = BRRR_OK;
    if (cudaMemsetAsync(state, 0, sizeof(DevState), st) != cudaSuccess) rc = BRRR_ERR_CUDA;
    // wait_for_router: the kernel polls for routing words tagged 1; nobody publishes them here
    if (rc == BRRR_OK &&
        launch_fold_norm(d_top, d_wts, nullptr, 0, topk, d, d_part, d_down_b, d_x, d_norm_w, eps, d_q, d_s, wait_for_router ? &state->router_seq : nullptr,
                         wait_for_router ? &state->fold_seq : nullptr, state, false, st) != cudaSuccess)
        rc = BRRR_ERR_CUDA;
    uint32_t err = 0;
    if (rc == BRRR_OK && cudaMemcpyAsync(&err, &state->err, sizeof err, cudaMemcpyDeviceToHost, st) != cudaSuccess) rc = BRRR_ERR_CUDA;
    if (rc == BRRR_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = BRRR_ERR_CUDA;
    cudaFree(state);
    if (rc == BRRR_OK && err != 0) rc = BRRR_ERR_STATE;
    return rc == BRRR_OK ? check_launch() : rc;
}
