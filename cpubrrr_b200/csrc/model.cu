// Host side of the engine: data-directory loader, synthetic-model builder, the decode step as a
// CUDA graph, and the model-level C ABI (include/brrr.h).
//
// It mirrors the reference's host program for this path (src/bin/engine_gpt2.rs): load_cfg
// (64-80), the manifest/mmap loader (1276-1285), the per-layer weight preparation (1290-1315),
// the activation buffers (1340-1347) and run() (1379-1385) — with the 12-worker barrier
// scheduler (619-687, 1354-1378) replaced by one CUDA graph launch per token.
#include "../../include/brrr.h"
#include "brrr_kernels.h"
#include "brrr_synth.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <fcntl.h>
#include <map>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

using namespace brrr;

static thread_local char g_cuda_err[512] = "";

#define CU(call)                                                                                         \
    do {                                                                                                 \
        cudaError_t _e = (call);                                                                         \
        if (_e != cudaSuccess) {                                                                         \
            snprintf(g_cuda_err, sizeof g_cuda_err, "%s:%d %s: %s", __FILE__, __LINE__, #call, cudaGetErrorString(_e)); \
            return BRRR_ERR_CUDA;                                                                        \
        }                                                                                                \
    } while (0)

extern "C" const char *brrr_last_cuda_error(void) { return g_cuda_err; }
namespace brrr { char *host_err_buf() { return g_cuda_err; } }   // shared with the other model files (512 bytes)
extern "C" const char *brrr_strerror(int s) {
    switch (s) {
    case BRRR_OK: return "ok";
    case BRRR_ERR_ARG: return "bad argument or unsupported shape";
    case BRRR_ERR_IO: return "data directory or blob unreadable or malformed";
    case BRRR_ERR_CUDA: return "CUDA call failed";
    case BRRR_ERR_NOMEM: return "out of memory";
    case BRRR_ERR_RANGE: return "position, token or count out of range";
    case BRRR_ERR_STATE: return "call not valid in the current state";
    }
    return "unknown status";
}

namespace {

struct Layer {
    float *attn_norm = nullptr, *ffn_norm = nullptr;
    Q8Dev wqkv{}, wo{};
    float *bqkv = nullptr, *bo = nullptr, *sinks = nullptr, *ginp = nullptr, *ginp_b = nullptr;
    MxDev gate{}, up{}, down{};
    float *gate_b = nullptr, *up_b = nullptr, *down_b = nullptr;
    MxtDev gu_t{}, down_t{};     // tensor-core tile units of gate|up and down (use_mxt)
    float *kc = nullptr, *vc = nullptr;
};

// Where raw GGUF-format tensor bytes come from: a mapped blob or the synthetic generator.
struct Source {
    bool synth = false;
    uint64_t seed = 0;
    const uint8_t *blob = nullptr;
    size_t blob_len = 0;
    struct Ent { uint32_t type; size_t off, nel; };
    std::map<std::string, Ent> idx;
};

const char *kind_name(int kind) {
    switch (kind) {
    case BRRR_T_ATTN_NORM: return "attn_norm.weight"; case BRRR_T_FFN_NORM: return "ffn_norm.weight";
    case BRRR_T_WQ: return "attn_q.weight"; case BRRR_T_WK: return "attn_k.weight";
    case BRRR_T_WV: return "attn_v.weight"; case BRRR_T_WO: return "attn_out.weight";
    case BRRR_T_BQ: return "attn_q.bias"; case BRRR_T_BK: return "attn_k.bias";
    case BRRR_T_BV: return "attn_v.bias"; case BRRR_T_BO: return "attn_out.bias";
    case BRRR_T_SINKS: return "attn_sinks"; case BRRR_T_ROUTER_W: return "ffn_gate_inp.weight";
    case BRRR_T_ROUTER_B: return "ffn_gate_inp.bias"; case BRRR_T_GATE: return "ffn_gate_exps.weight";
    case BRRR_T_UP: return "ffn_up_exps.weight"; case BRRR_T_DOWN: return "ffn_down_exps.weight";
    case BRRR_T_GATE_B: return "ffn_gate_exps.bias"; case BRRR_T_UP_B: return "ffn_up_exps.bias";
    case BRRR_T_DOWN_B: return "ffn_down_exps.bias";
    case BRRR_T_TOK_EMBD: return "token_embd.weight"; case BRRR_T_OUT_NORM: return "output_norm.weight";
    case BRRR_T_OUTPUT: return "output.weight";
    }
    return "?";
}

size_t type_bytes(uint32_t type, size_t nel) {
    switch (type) {
    case 0: return nel * 4;
    case 30: return nel * 2;
    case 39: return nel / 32 * 17;
    }
    return 0;
}

}  // namespace

struct brrr_model {
    brrr_cfg cfg{};
    int device = 0;
    cudaStream_t stream = nullptr;
    std::vector<Layer> L;
    float *out_norm = nullptr;
    Q8Dev head{};
    uint16_t *tok_embd = nullptr;
    float *rope = nullptr;
    // activations
    float *x = nullptr, *qkv = nullptr, *ao = nullptr, *gu = nullptr, *rlogits = nullptr, *logits = nullptr;
    float *xs = nullptr, *as = nullptr, *hs = nullptr, *wts = nullptr;
    int8_t *xq = nullptr, *aq = nullptr, *hq = nullptr;
    int32_t *top = nullptr;
    DevState *st = nullptr;
    // host staging (pinned)
    uint32_t *h_in = nullptr, *h_out = nullptr;
    cudaGraphExec_t g_head = nullptr, g_nohead = nullptr;            // speculative-routing step (or plain when disabled)
    cudaGraphExec_t g_head_safe = nullptr, g_nohead_safe = nullptr;  // plain step, used to redo a missed speculation
    cudaStream_t side = nullptr;                                     // the exact router runs here, beside gate/up
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    bool use_spec = true;        // start gate/up from a fast router estimate, verify with the exact router
    uint32_t test_hooks = 0;     // BRRR_TEST_HOOKS builds: copied into DevState.test_hooks (see there)
    bool spec_off = false;       // a bounded device wait of the speculative step ran out once: plain graphs from then on
    uint64_t wait_fallbacks = 0; // how often that happened
    float *est = nullptr;        // estimated router logits
    uint32_t run_tok = 0, run_pos = 0;   // arguments of the decode run in flight (for a redo)
    uint64_t spec_redos = 0;
    int launches_head = 0, launches_nohead = 0;
    bool use_pdl = true;         // chain the step's kernels with programmatic dependent launch
    // expert matvecs of the speculative step on the tensor cores in native fp4 (kernels_mxt.cu);
    // needs a second copy of the expert matrices in tile units
    bool use_mxt = false;
    float *dpart = nullptr;      // down: [topk][tiles * 128] row sums
    uint32_t *dcount = nullptr;  // down: arrival counters per row tile
    uint8_t *ximg = nullptr, *himg = nullptr;   // operand images of the token's and of h's Q8 activation
    int8_t *nq = nullptr;        // Q8 of the normalised residual that the fold leaves for the next q/k/v projection
    float *ns = nullptr;
    bool fused_fold = true;      // speculative tensor-core step: fold + next norm/quant in one kernel that waits for the router by flag
    // expert parallelism: this rank holds experts [epc.e_lo, epc.e_lo + epc.e_cnt); the exchange
    // region (slices, flags, step counters) is one allocation shared with the peers through IPC
    bool ep = false, ep_attached = false;
    EpCtx epc{};
    void *ep_buf = nullptr;
    std::vector<void *> ep_peers;
    // scratch of the token-tile MoE step (allocated at first use): BRRR_TILE_MAX tokens x top-k entries
    int8_t *tl_xq = nullptr, *tl_hq = nullptr;
    float *tl_xs = nullptr, *tl_hs = nullptr, *tl_logits = nullptr, *tl_wts = nullptr, *tl_gu = nullptr, *tl_part = nullptr;
    int32_t *tl_top = nullptr;
    int *tl_cnt = nullptr, *tl_list = nullptr;
    // token rows (prompt tiles, batched decode): up to BRRR_TILE_MAX rows walk the layers together
    float *tl_x = nullptr, *tl_xn = nullptr;     // residual and normalised residual of the rows
    float *tl_qkv = nullptr, *tl_ao = nullptr, *tl_ns = nullptr, *tl_as = nullptr;
    int8_t *tl_nq = nullptr, *tl_aq = nullptr;
    uint32_t *tl_toks = nullptr;                 // per row: token id, position, sequence (device; filled from a pinned slot)
    int *tl_pos = nullptr, *tl_seq = nullptr;
    uint32_t *h_tile = nullptr;                  // pinned: one 64-word slot per tile in flight
    uint32_t h_tile_next = 0;
    cudaGraphExec_t g_rows[3][BRRR_TILE_MAX + 1] = {};          // [ROWS_PROMPT | ROWS_BATCH | ROWS_BATCH_PROMPT][rows]: layers without the head
    bool rows_graph_failed = false;
    // batched decode over independent sequences: one KV cache per sequence and layer
    int nseq = 0;
    std::vector<float *> kcb, vcb;               // per layer: [nseq][nkv][MAXSEQ][64]
    float *bt_logits = nullptr;                  // [BRRR_TILE_MAX][n_vocab]
    uint32_t *bt_tok = nullptr;                  // [BRRR_TILE_MAX] argmax per row
    bool no_attn_rows = false;                   // BRRR_NO_ATTN_ROWS=1: prompt tiles use the per-(head, row) attention kernel (same bits)
    int tile_rows = BRRR_TILE_MAX;               // tokens per prompt tile (BRRR_TILE_ROWS=n, 2..BRRR_TILE_MAX): any size gives the same bits
    bool tile_prefill = true;                    // run_tile on token tiles (brrr_model_set_tile_prefill / BRRR_TILE_PREFILL=0 switch to token-serial; same bits)
    unsigned int *tl_counter = nullptr;
    std::vector<void *> allocs;

    template <typename T> int alloc(T **p, size_t n) {
        void *v = nullptr;
        if (cudaMalloc(&v, n ? n * sizeof(T) : 16) != cudaSuccess) {
            snprintf(g_cuda_err, sizeof g_cuda_err, "cudaMalloc of %zu bytes failed", n * sizeof(T));
            return BRRR_ERR_NOMEM;
        }
        allocs.push_back(v);
        *p = (T *)v;
        return BRRR_OK;
    }
};

namespace {

#define TRY(expr) do { int _s = (expr); if (_s != BRRR_OK) return _s; } while (0)

// Fetch one tensor's raw bytes into device scratch: nel elements starting at element `first` of a
// tensor of `total` elements (total = 0: the whole tensor, first = 0).
int fetch(brrr_model *m, const Source &s, uint32_t layer, int kind, uint32_t type, size_t nel, void *scratch, size_t first = 0, size_t total = 0) {
    if (total == 0) total = nel;
    if (s.synth) {
        launch_synth(s.seed, layer, kind, type, nel, scratch, m->stream, first);
        CU(cudaGetLastError());
        return BRRR_OK;
    }
    char name[160];
    if (layer == BRRR_L_GLOBAL) snprintf(name, sizeof name, "%s", kind_name(kind));
    else snprintf(name, sizeof name, "blk.%u.%s", layer, kind_name(kind));
    auto it = s.idx.find(name);
    if (it == s.idx.end()) { snprintf(g_cuda_err, sizeof g_cuda_err, "missing tensor %s", name); return BRRR_ERR_IO; }
    if (it->second.type != type || it->second.nel != total) { snprintf(g_cuda_err, sizeof g_cuda_err, "tensor %s: type/size mismatch", name); return BRRR_ERR_IO; }
    size_t bytes = type_bytes(type, nel), skip = type_bytes(type, first);
    if (it->second.off + skip + bytes > s.blob_len) { snprintf(g_cuda_err, sizeof g_cuda_err, "tensor %s exceeds blob", name); return BRRR_ERR_IO; }
    CU(cudaMemcpyAsync(scratch, s.blob + it->second.off + skip, bytes, cudaMemcpyHostToDevice, m->stream));
    CU(cudaStreamSynchronize(m->stream));
    return BRRR_OK;
}

int load_f32(brrr_model *m, const Source &s, uint32_t layer, int kind, size_t n, float **out) {
    TRY(m->alloc(out, n));
    return fetch(m, s, layer, kind, 0, n, *out);
}

int alloc_q8(brrr_model *m, int rows, int cols, Q8Dev *q) {
    q->rows = rows; q->cols = cols;
    TRY(m->alloc(&q->data, q8_bytes(rows, cols)));
    CU(cudaMemsetAsync(q->data, 0, q8_bytes(rows, cols), m->stream));   // padding rows quantise to zero
    return BRRR_OK;
}

int load_q8_part(brrr_model *m, const Source &s, uint32_t layer, int kind, int rows, int row0, Q8Dev q, void *scratch) {
    TRY(fetch(m, s, layer, kind, 30, (size_t)rows * q.cols, scratch));
    launch_q8_pack((const uint16_t *)scratch, rows, row0, q, m->stream);
    CU(cudaGetLastError());
    return BRRR_OK;
}

// rows [row0, row0 + rows) of an MXFP4 tensor of rows_total rows (an expert-parallel rank loads its experts only)
int load_mx(brrr_model *m, const Source &s, uint32_t layer, int kind, int rows, int blocks, MxDev *x, void *scratch, int row0 = 0, int rows_total = 0) {
    x->rows = rows; x->blocks = blocks;
    TRY(m->alloc(&x->data, mx_bytes(rows, blocks)));
    TRY(fetch(m, s, layer, kind, 39, (size_t)rows * blocks * 32, scratch, (size_t)row0 * blocks * 32, (size_t)(rows_total ? rows_total : rows) * blocks * 32));
    launch_mx_pack((const uint8_t *)scratch, *x, m->stream);
    CU(cudaGetLastError());
    return BRRR_OK;
}

void rope_table_host(const brrr_cfg &c, float *tab) {
    // YaRN table (src/bin/engine_gpt2.rs:536-572): factor 32, original context 4096, beta 32 / 1,
    // mscale 1 + 0.1 ln 32; entries are the rotation of (1, 0), i.e. (cos*mscale, sin*mscale).
    int hd = c.head_dim, half = hd / 2;
    float base = c.rope_freq_base;
    const float PI = 3.14159265358979323846f;
    float lb = logf(base);
    float fd32 = (float)hd * logf(4096.0f / (32.0f * 2.0f * PI)) / (2.0f * lb);
    float fd1 = (float)hd * logf(4096.0f / (1.0f * 2.0f * PI)) / (2.0f * lb);
    float low = floorf(fd32); if (low < 0.0f) low = 0.0f;
    float high = ceilf(fd1); if (high > (float)hd - 1.0f) high = (float)hd - 1.0f;
    float mscale = 1.0f + 0.1f * logf(32.0f);
    float den = high - low; if (den < 0.001f) den = 0.001f;
    for (int pos = 0; pos < BRRR_MAXSEQ; pos++)
        for (int i = 0; i < half; i++) {
            float theta_ex = (float)pos * powf(base, -(2.0f * (float)i) / (float)hd);
            float theta_in = theta_ex / 32.0f;
            float y = ((float)i - low) / den;
            if (y < 0.0f) y = 0.0f;
            if (y > 1.0f) y = 1.0f;
            float mix = 1.0f - y;
            float theta = theta_in * (1.0f - mix) + theta_ex * mix;
            tab[((size_t)pos * half + i) * 2] = cosf(theta) * mscale;
            tab[((size_t)pos * half + i) * 2 + 1] = sinf(theta) * mscale;
        }
}

int check_cfg(const brrr_cfg &c) {
    if (c.n_embd <= 0 || c.n_embd % 64 || c.n_embd > 4096) return BRRR_ERR_ARG;
    if (c.n_ff_exp != c.n_embd) return BRRR_ERR_ARG;                     // engine_gpt2.rs:73
    if (c.head_dim != 64) return BRRR_ERR_ARG;                           // engine_gpt2.rs:74
    if (c.n_head <= 0 || c.n_head_kv <= 0 || c.n_head % c.n_head_kv) return BRRR_ERR_ARG;
    if (c.n_expert <= 0 || c.n_expert > 256 || c.n_expert_used <= 0 || c.n_expert_used > 8 || c.n_expert_used > c.n_expert) return BRRR_ERR_ARG;
    if (c.n_vocab <= 0 || c.n_vocab % 4 || c.n_layer <= 0) return BRRR_ERR_ARG;
    if (c.sliding_window <= 0) return BRRR_ERR_ARG;
    return BRRR_OK;
}

// The decode step, enqueued kernel by kernel (captured into a graph, or run directly by the
// trace path).  Stage order and data flow follow forward_worker (engine_gpt2.rs:751-934).
enum { ST_EMBED = 0, ST_QKV, ST_ATTN, ST_OPROJ, ST_ROUTER, ST_GATE_UP, ST_DOWN, ST_FOLD, ST_HEAD_NORM, ST_HEAD, ST_FINISH, ST_COUNT };
const char *const kStageNames[ST_COUNT] = {"embed", "norm_qkv_gemv", "attention", "oproj_gemv", "norm_router_topk",
                                           "norm_gate_up_swiglu_mxfp4", "down_combine_mxfp4", "fold_norm_quant", "head_norm_quant", "head_gemv_argmax",
                                           "finish_token"};

#define CUL(call)                                                                                        \
    do {                                                                                                 \
        cudaError_t _e = (call);                                                                         \
        if (_e != cudaSuccess) {                                                                         \
            snprintf(g_cuda_err, sizeof g_cuda_err, "%s:%d %s: %s", __FILE__, __LINE__, #call, cudaGetErrorString(_e)); \
            return BRRR_ERR_CUDA;                                                                        \
        }                                                                                                \
    } while (0)

// The decode step, enqueued kernel by kernel (captured into a graph, or run directly by the
// trace path).  Stage order and data flow follow forward_worker (engine_gpt2.rs:751-934); the
// reference's nine barrier-separated stages per layer are six kernels here, chained with
// programmatic dependent launch.
int enqueue_step(brrr_model *m, bool want, float *trace_dev, int *nlaunch, unsigned mask = ~0u, bool spec = false) {
    const brrr_cfg &c = m->cfg;
    const int d = c.n_embd, nh = c.n_head, nkv = c.n_head_kv, topk = c.n_expert_used;
    cudaStream_t s = m->stream;
    const bool pdl = m->use_pdl && !trace_dev && mask == ~0u;
    int n = 0;
    auto on = [&](int st) { if (mask & (1u << st)) { n++; return true; } return false; };
    if (m->ep) { launch_ep_begin(m->epc, m->st, s); n++; }
    if (on(ST_EMBED)) launch_embed(m->tok_embd, d, m->st, m->x, s);
    if (trace_dev) CU(cudaMemcpyAsync(trace_dev, m->x, d * sizeof(float), cudaMemcpyDeviceToDevice, s));
    for (int il = 0; il < c.n_layer; il++) {
        Layer &ly = m->L[il];
        // fused: the previous layer's fold has left the normalised, quantised residual in nq / ns
        const bool fused = spec && m->use_mxt && m->fused_fold;
        const int kv_window = (((il + 1) % 2 != 0) && c.sliding_window < BRRR_MAXSEQ) ? c.sliding_window : 0;
        if (fused && il > 0) { n++; CUL(launch_q8_stream(ly.wqkv, nullptr, nullptr, 0.0f, m->nq, m->ns, ly.bqkv, m->qkv, Q8_EPI_BIAS, m->st, pdl, s,
                                                         ly.kc, ly.vc, nkv, kv_window)); }
        else if (mask != ~0u && m->use_mxt && m->use_spec && m->fused_fold && il > 0) {      // stage replay of the fused step's q/k/v (image left by the last step)
            if (on(ST_QKV)) CUL(launch_q8_stream(ly.wqkv, nullptr, nullptr, 0.0f, m->nq, m->ns, ly.bqkv, m->qkv, Q8_EPI_BIAS, m->st, pdl, s));
        } else if (on(ST_QKV)) CUL(launch_q8_stream(ly.wqkv, m->x, ly.attn_norm, c.rms_eps, nullptr, nullptr, ly.bqkv, m->qkv, Q8_EPI_BIAS, m->st, pdl && n > 1, s));
        int window = ((il + 1) % 2 != 0) ? c.sliding_window : 0;         // even layer index: sliding window
        if (window >= BRRR_MAXSEQ) window = 0;
        if (on(ST_ATTN)) CUL(launch_attn_decode(m->qkv, ly.kc, ly.vc, m->rope, ly.sinks, nh, nkv, m->st, 0, window, m->ao, m->aq, m->as, m->st, pdl, s));
        if (on(ST_OPROJ)) CUL(launch_q8_stream(ly.wo, nullptr, nullptr, 0.0f, m->aq, m->as, ly.bo, m->x, Q8_EPI_RESID_BIAS, m->st, pdl, s));
        if (spec) {
            // Speculative routing: the exact serial-chain router runs on the side stream while the
            // main stream estimates the expert set and streams gate/up for it; down joins both,
            // uses the exact routing and flags the step if the estimate missed an expert.
            CU(cudaEventRecord(m->ev_fork, s));
            CU(cudaStreamWaitEvent(m->side, m->ev_fork, 0));
            n++;
            CUL(launch_ffn_in(m->x, ly.ffn_norm, c.rms_eps, d, ly.ginp, ly.ginp_b, c.n_expert, topk, m->rlogits, m->top, m->wts,
                              &m->st->router_done, m->st, false, m->side, 1, fused ? &m->st->router_seq : nullptr));
            CU(cudaEventRecord(m->ev_join, m->side));
            n++;
            CUL(launch_router_hint(m->x, ly.ffn_norm, c.rms_eps, d, ly.ginp, ly.ginp_b, c.n_expert, topk, m->est, m->xq, m->xs, m->st, pdl, s,
                                   m->use_mxt ? m->ximg : nullptr));
            n++;
            const EpCtx *epc = m->ep ? &m->epc : nullptr;      // expert parallelism: local slots only, row sums exchanged by down, awaited by the fold
            if (m->use_mxt) CUL(launch_gate_up_t(ly.gu_t, ly.gate_b, ly.up_b, nullptr, m->est, c.n_expert, topk, d, m->ximg, m->xs,
                                                 m->hq, m->hs, m->himg, m->st, pdl, s, epc, il));
            else CUL(launch_gate_up(ly.gate, ly.up, ly.gate_b, ly.up_b, nullptr, topk, d, nullptr, nullptr, c.rms_eps, m->xq, m->xs,
                                    m->hq, m->hs, nullptr, m->st, pdl, s, m->est, c.n_expert));
            if (m->use_mxt) {
                // down for the estimated experts as well; only the fold waits for the exact routing
                n++;
                CUL(launch_down_t(ly.down_t, ly.down_b, nullptr, nullptr, m->est, c.n_expert, topk, d, m->himg, m->hs, m->x,
                                  m->dpart, m->dcount, m->st, pdl, s, epc, il));
            }
            if (fused) {
                // The fold is launched programmatically behind down and waits for the router's
                // publication counter itself; it also normalises and quantises the new residual for
                // the next q/k/v projection (the last layer: for the vocabulary head).  The side
                // stream joins once, after the last layer.
                const bool last = il == c.n_layer - 1;
                const float *nw = last ? (want ? m->out_norm : nullptr) : m->L[il + 1].attn_norm;
                n++;
                CUL(launch_fold_norm(m->top, m->wts, m->est, c.n_expert, topk, d, m->dpart, ly.down_b, m->x, nw, c.rms_eps,
                                     last ? m->xq : m->nq, last ? m->xs : m->ns, &m->st->router_seq, &m->st->fold_seq, m->st, pdl, s, epc, il));
                if (last) CU(cudaStreamWaitEvent(s, m->ev_join, 0));
                continue;
            }
            CU(cudaStreamWaitEvent(s, m->ev_join, 0));
            n++;
            // full dependency on both predecessors: a programmatic launch here was observed to start
            // before the side-stream router had finished
            if (m->use_mxt) CUL(launch_down_fold(m->top, m->wts, m->est, c.n_expert, topk, d, m->dpart, ly.down_b, m->x, m->st, false, s));
            else CUL(launch_down_combine(ly.down, ly.down_b, m->top, m->wts, m->est, c.n_expert, topk, d, m->hq, m->hs, m->x, m->st, false, s));
        } else if (m->use_mxt && mask != ~0u) {
            // single-stage replays (stage timing) of the kernels the speculative step runs, on the
            // activation and routing the last step left behind
            if (on(ST_ROUTER)) CUL(launch_ffn_in(m->x, ly.ffn_norm, c.rms_eps, d, ly.ginp, ly.ginp_b, c.n_expert, topk, m->rlogits, m->top, m->wts,
                                                 &m->st->router_done, m->st, pdl, s));
            if (on(ST_GATE_UP)) CUL(launch_gate_up_t(ly.gu_t, ly.gate_b, ly.up_b, m->top, nullptr, 0, topk, d, m->ximg, m->xs, m->hq, m->hs, m->himg,
                                                     m->st, pdl, s));
            const bool ff = m->use_spec && m->fused_fold;     // the fused step: down leaves partial sums, a fold kernel finishes
            if (on(ST_DOWN)) CUL(launch_down_t(ly.down_t, ly.down_b, m->top, ff ? nullptr : m->wts, nullptr, 0, topk, d, m->himg, m->hs, m->x, m->dpart,
                                               m->dcount, m->st, pdl, s));
            if (ff && on(ST_FOLD))
                CUL(launch_fold_norm(m->top, m->wts, nullptr, 0, topk, d, m->dpart, ly.down_b, m->x,
                                     il + 1 < c.n_layer ? m->L[il + 1].attn_norm : m->out_norm, c.rms_eps, m->nq, m->ns, nullptr, nullptr, m->st, pdl, s));
        } else {
        if (on(ST_ROUTER)) CUL(launch_ffn_in(m->x, ly.ffn_norm, c.rms_eps, d, ly.ginp, ly.ginp_b, c.n_expert, topk, m->rlogits, m->top, m->wts,
                                             &m->st->router_done, m->st, pdl, s));
        if (on(ST_GATE_UP)) CUL(launch_gate_up(ly.gate, ly.up, ly.gate_b, ly.up_b, m->top, topk, d, m->x, ly.ffn_norm, c.rms_eps, nullptr, nullptr,
                                               m->hq, m->hs, nullptr, m->st, pdl, s, nullptr, 0, m->ep ? m->epc.e_lo : 0,
                                               m->ep ? m->epc.e_cnt : (1 << 30)));
        if (m->ep) { if (on(ST_DOWN)) CUL(launch_down_ep(ly.down, ly.down_b, m->top, m->wts, topk, d, il, m->hq, m->hs, m->x, m->st, m->epc, pdl, s)); }
        else if (on(ST_DOWN)) CUL(launch_down_combine(ly.down, ly.down_b, m->top, m->wts, nullptr, 0, topk, d, m->hq, m->hs, m->x, m->st, pdl, s));
        }
        if (trace_dev) CU(cudaMemcpyAsync(trace_dev + (size_t)(il + 1) * d, m->x, d * sizeof(float), cudaMemcpyDeviceToDevice, s));
    }
    if (want) {
        const bool fused = spec && m->use_mxt && m->fused_fold;      // the last fold has written the head's activation; the side stream has just joined
        const bool replay_fused = mask != ~0u && m->use_mxt && m->use_spec && m->fused_fold;      // stage replays mirror the fused step
        if (!fused && !replay_fused && on(ST_HEAD_NORM)) CUL(launch_rmsnorm_quant(m->x, m->out_norm, c.rms_eps, d, nullptr, m->xq, m->xs, pdl, s));
        if (on(ST_HEAD)) CUL(launch_q8_head(m->head, m->xq, m->xs, m->logits, m->st, pdl && !fused, s));
        if (on(ST_FINISH)) launch_finish_token(m->st, s);
    }
    CU(cudaGetLastError());
    if (nlaunch) *nlaunch = n;
    return BRRR_OK;
}

int capture(brrr_model *m, bool want, cudaGraphExec_t *out, int *nlaunch, unsigned mask = ~0u, bool spec = false) {
    cudaGraph_t g = nullptr;
    CU(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
    int s = enqueue_step(m, want, nullptr, nlaunch, mask, spec);
    cudaError_t e = cudaStreamEndCapture(m->stream, &g);
    if (s != BRRR_OK) { if (g) cudaGraphDestroy(g); return s; }
    CU(e);
    CU(cudaGraphInstantiate(out, g, 0));
    CU(cudaGraphDestroy(g));
    return BRRR_OK;
}

// Device state as a fresh model has it.
int reset_state(brrr_model *m) {
    CU(cudaMemsetAsync(m->st, 0, sizeof(DevState), m->stream));
    CU(cudaMemsetAsync(&m->st->spec_fail_step, 0xFF, 4, m->stream));
    if (m->test_hooks) CU(cudaMemcpyAsync(&m->st->test_hooks, &m->test_hooks, 4, cudaMemcpyHostToDevice, m->stream));
    return BRRR_OK;
}

// First step and graph capture (needs every buffer the step touches, peers included).
int finish_build(brrr_model *m) {
    // expert-parallel ranks speculate only on the tensor-core path with the fused fold (its partial
    // sums are what the ranks exchange); otherwise they run the plain step
    if (m->ep && !(m->use_mxt && m->fused_fold)) m->use_spec = false;
    // one direct (un-captured) step configures every kernel's attributes and validates the launches
    TRY(reset_state(m));
    TRY(enqueue_step(m, true, nullptr, nullptr));
    CU(cudaStreamSynchronize(m->stream));
    TRY(reset_state(m));
    TRY(capture(m, true, &m->g_head_safe, &m->launches_head));
    TRY(capture(m, false, &m->g_nohead_safe, &m->launches_nohead));
    if (m->use_spec) {
        // direct speculative step once (kernel attributes), then capture
        TRY(enqueue_step(m, true, nullptr, nullptr, ~0u, true));
        CU(cudaStreamSynchronize(m->stream));
        TRY(reset_state(m));
        TRY(capture(m, true, &m->g_head, &m->launches_head, ~0u, true));
        TRY(capture(m, false, &m->g_nohead, &m->launches_nohead, ~0u, true));
    } else {
        TRY(capture(m, true, &m->g_head, &m->launches_head));
        TRY(capture(m, false, &m->g_nohead, &m->launches_nohead));
    }
    CU(cudaStreamSynchronize(m->stream));
    return BRRR_OK;
}

int build_model(brrr_model *m, const Source &src) {
    const brrr_cfg &c = m->cfg;
    const int d = c.n_embd, nh = c.n_head, nkv = c.n_head_kv, hd = c.head_dim, nb = d / 32, ne = c.n_expert, topk = c.n_expert_used;
    CU(cudaSetDevice(m->device));
    CU(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
    if (const char *e = getenv("BRRR_NOPDL")) m->use_pdl = !(e[0] && e[0] != '0');
    if (const char *e = getenv("BRRR_NOSPEC")) m->use_spec = !(e[0] && e[0] != '0');
#ifdef BRRR_TEST_HOOKS
    if (const char *e = getenv("BRRR_SPEC_SABOTAGE")) if (e[0] && e[0] != '0') m->test_hooks |= 1u;
    if (const char *e = getenv("BRRR_ROUTER_MUTE")) if (e[0] && e[0] != '0') m->test_hooks |= 2u;
#endif
    CU(cudaStreamCreateWithFlags(&m->side, cudaStreamNonBlocking));
    CU(cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming));
    CU(cudaEventCreateWithFlags(&m->ev_join, cudaEventDisableTiming));

    // scratch for one raw tensor: the largest of the bf16 matrices and one MXFP4 expert tensor
    size_t scratch_bytes = std::max({(size_t)c.n_vocab * d * 2, (size_t)ne * d * nb * 17, (size_t)nh * hd * d * 2});
    void *scratch = nullptr;
    if (cudaMalloc(&scratch, scratch_bytes) != cudaSuccess) return BRRR_ERR_NOMEM;
    struct Guard { void *p; ~Guard() { cudaFree(p); } } guard{scratch};

    m->L.resize(c.n_layer);
    const int qkv_rows = (nh + 2 * nkv) * hd;
    {
        // tensor-core expert path: single GPU, speculative step, shapes the tiles cover, and room
        // for the second copy of the expert matrices (about 1.08 x their size)
        size_t free_b = 0, total_b = 0;
        CU(cudaMemGetInfo(&free_b, &total_b));
        const size_t experts = (size_t)c.n_layer * (m->ep ? m->epc.e_cnt : ne) * 3 * d * nb * 17;      // this rank's share
        const size_t rest = (size_t)c.n_vocab * d * 4 + (size_t)c.n_layer * ((size_t)(qkv_rows + d) * d * 2 + (size_t)BRRR_MAXSEQ * nkv * hd * 8) + (2ull << 30);
        m->use_mxt = d % 64 == 0 && nb % 2 == 0 && topk <= 8 && free_b > experts * 2.2 + rest;
        if (const char *e = getenv("BRRR_NOMXT")) if (e[0] && e[0] != '0') m->use_mxt = false;
        if (const char *e = getenv("BRRR_NOFUSEDFOLD")) if (e[0] && e[0] != '0') m->fused_fold = false;
        if (const char *e = getenv("BRRR_TILE_PREFILL")) m->tile_prefill = e[0] && e[0] != '0';
        if (const char *e = getenv("BRRR_NO_ATTN_ROWS")) m->no_attn_rows = e[0] && e[0] != '0';
        if (const char *e = getenv("BRRR_TILE_ROWS")) { const int v = atoi(e); if (v >= 2 && v <= BRRR_TILE_MAX) m->tile_rows = v; }
    }
    for (int il = 0; il < c.n_layer; il++) {
        Layer &ly = m->L[il];
        TRY(load_f32(m, src, il, BRRR_T_ATTN_NORM, d, &ly.attn_norm));
        TRY(load_f32(m, src, il, BRRR_T_FFN_NORM, d, &ly.ffn_norm));
        TRY(alloc_q8(m, qkv_rows, d, &ly.wqkv));
        TRY(load_q8_part(m, src, il, BRRR_T_WQ, nh * hd, 0, ly.wqkv, scratch));
        TRY(load_q8_part(m, src, il, BRRR_T_WK, nkv * hd, nh * hd, ly.wqkv, scratch));
        TRY(load_q8_part(m, src, il, BRRR_T_WV, nkv * hd, (nh + nkv) * hd, ly.wqkv, scratch));
        TRY(alloc_q8(m, d, nh * hd, &ly.wo));
        TRY(load_q8_part(m, src, il, BRRR_T_WO, d, 0, ly.wo, scratch));
        TRY(m->alloc(&ly.bqkv, (size_t)qkv_rows));
        TRY(fetch(m, src, il, BRRR_T_BQ, 0, nh * hd, ly.bqkv));
        TRY(fetch(m, src, il, BRRR_T_BK, 0, nkv * hd, ly.bqkv + nh * hd));
        TRY(fetch(m, src, il, BRRR_T_BV, 0, nkv * hd, ly.bqkv + (nh + nkv) * hd));
        TRY(load_f32(m, src, il, BRRR_T_BO, d, &ly.bo));
        TRY(load_f32(m, src, il, BRRR_T_SINKS, nh, &ly.sinks));
        TRY(m->alloc(&ly.ginp, router_packed_floats(ne, d)));
        TRY(fetch(m, src, il, BRRR_T_ROUTER_W, 0, (size_t)ne * d, scratch));
        launch_router_pack((const float *)scratch, ne, d, ly.ginp, m->stream);
        CU(cudaGetLastError());
        TRY(load_f32(m, src, il, BRRR_T_ROUTER_B, ne, &ly.ginp_b));
        const int e_lo = m->ep ? m->epc.e_lo : 0, e_cnt = m->ep ? m->epc.e_cnt : ne;
        TRY(load_mx(m, src, il, BRRR_T_GATE, e_cnt * d, nb, &ly.gate, scratch, e_lo * d, ne * d));
        TRY(load_mx(m, src, il, BRRR_T_UP, e_cnt * d, nb, &ly.up, scratch, e_lo * d, ne * d));
        TRY(load_mx(m, src, il, BRRR_T_DOWN, e_cnt * d, nb, &ly.down, scratch, e_lo * d, ne * d));
        if (m->use_mxt) {
            ly.gu_t.tiles_per_expert = d / 64; ly.gu_t.np = nb / 2;
            ly.down_t.tiles_per_expert = (d + 127) / 128; ly.down_t.np = nb / 2;
            TRY(m->alloc(&ly.gu_t.data, mxt_bytes(e_cnt, ly.gu_t.tiles_per_expert, nb / 2)));       // this rank's experts
            TRY(m->alloc(&ly.down_t.data, mxt_bytes(e_cnt, ly.down_t.tiles_per_expert, nb / 2)));
            launch_mxt_pack(ly.gate, ly.up, e_cnt, d, ly.gu_t, m->stream);
            launch_mxt_pack(ly.down, MxDev{nullptr, 0, 0}, e_cnt, d, ly.down_t, m->stream);
            CU(cudaGetLastError());
        }
        TRY(load_f32(m, src, il, BRRR_T_GATE_B, (size_t)ne * d, &ly.gate_b));
        TRY(load_f32(m, src, il, BRRR_T_UP_B, (size_t)ne * d, &ly.up_b));
        TRY(load_f32(m, src, il, BRRR_T_DOWN_B, (size_t)ne * d, &ly.down_b));
        TRY(m->alloc(&ly.kc, (size_t)BRRR_MAXSEQ * nkv * hd));
        TRY(m->alloc(&ly.vc, (size_t)BRRR_MAXSEQ * nkv * hd));
        CU(cudaMemsetAsync(ly.kc, 0, (size_t)BRRR_MAXSEQ * nkv * hd * 4, m->stream));   // layout [kv head][position][64]
        CU(cudaMemsetAsync(ly.vc, 0, (size_t)BRRR_MAXSEQ * nkv * hd * 4, m->stream));
    }
    TRY(m->alloc(&m->tok_embd, (size_t)c.n_vocab * d));
    TRY(fetch(m, src, BRRR_L_GLOBAL, BRRR_T_TOK_EMBD, 30, (size_t)c.n_vocab * d, m->tok_embd));
    TRY(load_f32(m, src, BRRR_L_GLOBAL, BRRR_T_OUT_NORM, d, &m->out_norm));
    TRY(alloc_q8(m, c.n_vocab, d, &m->head));
    TRY(load_q8_part(m, src, BRRR_L_GLOBAL, BRRR_T_OUTPUT, c.n_vocab, 0, m->head, scratch));

    std::vector<float> tab((size_t)BRRR_MAXSEQ * hd);
    rope_table_host(c, tab.data());
    TRY(m->alloc(&m->rope, tab.size()));
    CU(cudaMemcpyAsync(m->rope, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, m->stream));

    TRY(m->alloc(&m->x, d)); TRY(m->alloc(&m->qkv, qkv_rows)); TRY(m->alloc(&m->ao, nh * hd));
    TRY(m->alloc(&m->gu, (size_t)topk * 2 * d)); TRY(m->alloc(&m->rlogits, ne)); TRY(m->alloc(&m->logits, c.n_vocab));
    TRY(m->alloc(&m->xs, nb)); TRY(m->alloc(&m->as, nh * hd / 32)); TRY(m->alloc(&m->hs, (size_t)topk * nb)); TRY(m->alloc(&m->wts, 8));
    TRY(m->alloc(&m->xq, d)); TRY(m->alloc(&m->aq, nh * hd)); TRY(m->alloc(&m->hq, (size_t)topk * d));
    TRY(m->alloc(&m->top, 8)); TRY(m->alloc(&m->st, 1));
    TRY(m->alloc(&m->est, (size_t)ne));
    TRY(m->alloc(&m->nq, d)); TRY(m->alloc(&m->ns, nb));
    TRY(m->alloc(&m->dpart, (size_t)topk * ((d + 127) / 128) * 128));
    TRY(m->alloc(&m->dcount, (size_t)(d + 127) / 128));
    CU(cudaMemsetAsync(m->dcount, 0, (size_t)((d + 127) / 128) * 4, m->stream));
    TRY(m->alloc(&m->ximg, (size_t)(nb / 2 + 1) * 768));
    TRY(m->alloc(&m->himg, (size_t)topk * (nb / 2 + 1) * 768));
    CU(cudaMemsetAsync(m->ximg, 0, (size_t)(nb / 2 + 1) * 768, m->stream));      // producers only write the non-zero words
    CU(cudaMemsetAsync(m->himg, 0, (size_t)topk * (nb / 2 + 1) * 768, m->stream));
    CU(cudaMemsetAsync(m->st, 0, sizeof(DevState), m->stream));
    CU(cudaMemsetAsync(m->x, 0, d * 4, m->stream));
    CU(cudaMallocHost(&m->h_in, 16));
    CU(cudaMallocHost(&m->h_out, BRRR_MAXSEQ * sizeof(uint32_t)));
    CU(cudaStreamSynchronize(m->stream));
    if (m->ep) {
        // exchange region: slices [layer][slot][d] | slice flags [layer][slot][d/16] | step counters [8] (+ the local epoch word)
        // ... | tagged row sums of the speculative step [layer][slot][d] x 8 bytes
        const size_t nslice = (size_t)c.n_layer * topk * d, nflag = (size_t)c.n_layer * topk * (d / 16);
        const size_t bytes = nslice * 4 + nflag * 4 + (EP_MAX_WORLD + 8) * 4 + nslice * 8;
        CU(cudaMalloc(&m->ep_buf, bytes));
        CU(cudaMemsetAsync(m->ep_buf, 0, bytes, m->stream));
        CU(cudaStreamSynchronize(m->stream));
        return BRRR_OK;               // the first step needs the peers: brrr_model_ep_attach finishes the build
    }
    return finish_build(m);
}

int parse_dir(const char *dir, brrr_cfg *c, Source *src) {
    std::string p = std::string(dir) + "/config.txt";
    FILE *f = fopen(p.c_str(), "r");
    if (!f) { snprintf(g_cuda_err, sizeof g_cuda_err, "cannot open %s", p.c_str()); return BRRR_ERR_IO; }
    memset(c, 0, sizeof *c);
    c->sliding_window = 1 << 30;                                         // engine_gpt2.rs:78
    char line[512], key[128], val[128];
    std::map<std::string, std::string> kv;
    while (fgets(line, sizeof line, f))
        if (sscanf(line, "%127s %127s", key, val) == 2) kv[key] = val;
    fclose(f);
    const char *need_i[] = {"n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "n_expert", "n_expert_used", "n_ff_exp", "n_vocab"};
    for (const char *k : need_i)
        if (!kv.count(k)) { snprintf(g_cuda_err, sizeof g_cuda_err, "config missing %s", k); return BRRR_ERR_IO; }
    if (!kv.count("rope_freq_base") || !kv.count("rms_eps")) { snprintf(g_cuda_err, sizeof g_cuda_err, "config missing rope_freq_base/rms_eps"); return BRRR_ERR_IO; }
    c->n_embd = atoi(kv["n_embd"].c_str()); c->n_layer = atoi(kv["n_layer"].c_str());
    c->n_head = atoi(kv["n_head"].c_str()); c->n_head_kv = atoi(kv["n_head_kv"].c_str());
    c->head_dim = atoi(kv["head_dim"].c_str()); c->n_expert = atoi(kv["n_expert"].c_str());
    c->n_expert_used = atoi(kv["n_expert_used"].c_str()); c->n_ff_exp = atoi(kv["n_ff_exp"].c_str());
    c->n_vocab = atoi(kv["n_vocab"].c_str());
    if (kv.count("sliding_window")) c->sliding_window = atoi(kv["sliding_window"].c_str());
    c->rope_freq_base = strtof(kv["rope_freq_base"].c_str(), nullptr);
    c->rms_eps = strtof(kv["rms_eps"].c_str(), nullptr);

    p = std::string(dir) + "/manifest.txt";
    f = fopen(p.c_str(), "r");
    if (!f) { snprintf(g_cuda_err, sizeof g_cuda_err, "cannot open %s", p.c_str()); return BRRR_ERR_IO; }
    size_t data_start = 0;
    if (fscanf(f, "%127s %zu", key, &data_start) != 2 || strcmp(key, "data_start")) { fclose(f); snprintf(g_cuda_err, sizeof g_cuda_err, "bad manifest header"); return BRRR_ERR_IO; }
    char nm[256]; unsigned ty; size_t off, nel;
    while (fscanf(f, "%255s %u %zu %zu", nm, &ty, &off, &nel) == 4) src->idx[nm] = Source::Ent{ty, data_start + off, nel};
    fclose(f);
    return BRRR_OK;
}

}  // namespace

extern "C" int brrr_model_open(const char *data_dir, const char *blob_path, int device, brrr_model **out) {
    if (!data_dir || !blob_path || !out) return BRRR_ERR_ARG;
    *out = nullptr;
    brrr_model *m = new brrr_model();
    m->device = device;
    Source src;
    int s = parse_dir(data_dir, &m->cfg, &src);
    if (s == BRRR_OK) s = check_cfg(m->cfg);
    void *map = MAP_FAILED;
    if (s == BRRR_OK) {
        int fd = open(blob_path, O_RDONLY);
        struct stat stt;
        if (fd < 0 || fstat(fd, &stt) != 0) { snprintf(g_cuda_err, sizeof g_cuda_err, "cannot open blob %s", blob_path); s = BRRR_ERR_IO; }
        else {
            src.blob_len = stt.st_size;
            map = mmap(nullptr, src.blob_len, PROT_READ, MAP_PRIVATE, fd, 0);
            if (map == MAP_FAILED) { snprintf(g_cuda_err, sizeof g_cuda_err, "mmap of %s failed", blob_path); s = BRRR_ERR_IO; }
            src.blob = (const uint8_t *)map;
        }
        if (fd >= 0) close(fd);
    }
    if (s == BRRR_OK) s = build_model(m, src);
    if (map != MAP_FAILED) munmap(map, src.blob_len);
    if (s != BRRR_OK) { brrr_model_close(m); return s; }
    *out = m;
    return BRRR_OK;
}

extern "C" int brrr_model_open_synth(const brrr_cfg *cfg, uint64_t seed, int device, brrr_model **out) {
    if (!cfg || !out) return BRRR_ERR_ARG;
    *out = nullptr;
    int s = check_cfg(*cfg);
    if (s != BRRR_OK) return s;
    brrr_model *m = new brrr_model();
    m->cfg = *cfg;
    m->device = device;
    Source src;
    src.synth = true; src.seed = seed;
    s = build_model(m, src);
    if (s != BRRR_OK) { brrr_model_close(m); return s; }
    *out = m;
    return BRRR_OK;
}

// ---------------------------------------------------------------- expert parallelism
static int ep_prepare(brrr_model *m, int rank, int world) {
    const int ne = m->cfg.n_expert;
    if (world < 1 || world > EP_MAX_WORLD || rank < 0 || rank >= world || ne % world) return BRRR_ERR_ARG;
    m->ep = true;
    m->epc.rank = rank; m->epc.world = world;
    m->epc.e_cnt = ne / world; m->epc.e_lo = rank * (ne / world);
    return BRRR_OK;
}

extern "C" int brrr_model_open_synth_ep(const brrr_cfg *cfg, uint64_t seed, int device, int rank, int world, brrr_model **out) {
    if (!cfg || !out) return BRRR_ERR_ARG;
    *out = nullptr;
    int s = check_cfg(*cfg);
    if (s != BRRR_OK) return s;
    brrr_model *m = new brrr_model();
    m->cfg = *cfg;
    m->device = device;
    s = ep_prepare(m, rank, world);
    Source src;
    src.synth = true; src.seed = seed;
    if (s == BRRR_OK) s = build_model(m, src);
    if (s != BRRR_OK) { brrr_model_close(m); return s; }
    *out = m;
    return BRRR_OK;
}

extern "C" int brrr_model_open_ep(const char *data_dir, const char *blob_path, int device, int rank, int world, brrr_model **out) {
    if (!data_dir || !blob_path || !out) return BRRR_ERR_ARG;
    *out = nullptr;
    brrr_model *m = new brrr_model();
    m->device = device;
    Source src;
    int s = parse_dir(data_dir, &m->cfg, &src);
    if (s == BRRR_OK) s = check_cfg(m->cfg);
    if (s == BRRR_OK) s = ep_prepare(m, rank, world);
    void *map = MAP_FAILED;
    if (s == BRRR_OK) {
        int fd = open(blob_path, O_RDONLY);
        struct stat stt;
        if (fd < 0 || fstat(fd, &stt) != 0) { snprintf(g_cuda_err, sizeof g_cuda_err, "cannot open blob %s", blob_path); s = BRRR_ERR_IO; }
        else {
            src.blob_len = stt.st_size;
            map = mmap(nullptr, src.blob_len, PROT_READ, MAP_PRIVATE, fd, 0);
            if (map == MAP_FAILED) { snprintf(g_cuda_err, sizeof g_cuda_err, "mmap of %s failed", blob_path); s = BRRR_ERR_IO; }
            src.blob = (const uint8_t *)map;
        }
        if (fd >= 0) close(fd);
    }
    if (s == BRRR_OK) s = build_model(m, src);
    if (map != MAP_FAILED) munmap(map, src.blob_len);
    if (s != BRRR_OK) { brrr_model_close(m); return s; }
    *out = m;
    return BRRR_OK;
}

extern "C" int brrr_model_ep_handle(brrr_model *m, void *handle64) {
    if (!m || !handle64 || !m->ep || !m->ep_buf) return BRRR_ERR_STATE;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    CU(cudaSetDevice(m->device));
    cudaIpcMemHandle_t h;
    CU(cudaIpcGetMemHandle(&h, m->ep_buf));
    memcpy(handle64, &h, 64);
    return BRRR_OK;
}

extern "C" int brrr_model_ep_attach(brrr_model *m, const void *handles) {
    if (!m || !m->ep || !m->ep_buf || m->ep_attached) return BRRR_ERR_STATE;
    if (!handles && m->epc.world > 1) return BRRR_ERR_ARG;
    CU(cudaSetDevice(m->device));
    const brrr_cfg &c = m->cfg;
    const size_t nslice = (size_t)c.n_layer * c.n_expert_used * c.n_embd, nflag = (size_t)c.n_layer * c.n_expert_used * (c.n_embd / 16);
    m->ep_peers.assign(m->epc.world, nullptr);
    for (int p = 0; p < m->epc.world; p++) {
        void *base = m->ep_buf;
        if (p != m->epc.rank) {
            cudaIpcMemHandle_t h;
            memcpy(&h, (const char *)handles + (size_t)p * 64, 64);
            CU(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
            m->ep_peers[p] = base;
        }
        m->epc.xchg[p] = (float *)base;
        m->epc.flags[p] = (uint32_t *)((char *)base + nslice * 4);
        m->epc.done[p] = m->epc.flags[p] + nflag;
        m->epc.pairs[p] = (unsigned long long *)((char *)base + nslice * 4 + nflag * 4 + (EP_MAX_WORLD + 8) * 4);
    }
    m->epc.epoch = m->epc.done[m->epc.rank] + EP_MAX_WORLD;
    m->ep_attached = true;
    return finish_build(m);
}

extern "C" int brrr_model_ep_info(const brrr_model *m, int *rank, int *world, int *e_lo, int *e_cnt) {
    if (!m) return BRRR_ERR_ARG;
    if (rank) *rank = m->ep ? m->epc.rank : 0;
    if (world) *world = m->ep ? m->epc.world : 1;
    if (e_lo) *e_lo = m->ep ? m->epc.e_lo : 0;
    if (e_cnt) *e_cnt = m->ep ? m->epc.e_cnt : m->cfg.n_expert;
    return BRRR_OK;
}

extern "C" void brrr_model_close(brrr_model *m) {
    if (!m) return;
    cudaSetDevice(m->device);
    if (m->stream) cudaStreamSynchronize(m->stream);
    if (m->g_head) cudaGraphExecDestroy(m->g_head);
    if (m->g_nohead) cudaGraphExecDestroy(m->g_nohead);
    if (m->g_head_safe) cudaGraphExecDestroy(m->g_head_safe);
    if (m->g_nohead_safe) cudaGraphExecDestroy(m->g_nohead_safe);
    if (m->ev_fork) cudaEventDestroy(m->ev_fork);
    if (m->ev_join) cudaEventDestroy(m->ev_join);
    if (m->side) cudaStreamDestroy(m->side);
    for (void *p : m->ep_peers) if (p) cudaIpcCloseMemHandle(p);
    if (m->ep_buf) cudaFree(m->ep_buf);
    for (void *p : m->allocs) cudaFree(p);
    if (m->h_in) cudaFreeHost(m->h_in);
    if (m->h_tile) cudaFreeHost(m->h_tile);
    for (auto &gs : m->g_rows) for (cudaGraphExec_t g : gs) if (g) cudaGraphExecDestroy(g);
    if (m->h_out) cudaFreeHost(m->h_out);
    if (m->stream) cudaStreamDestroy(m->stream);
    delete m;
}

extern "C" int brrr_model_cfg(const brrr_model *m, brrr_cfg *out) {
    if (!m || !out) return BRRR_ERR_ARG;
    *out = m->cfg;
    return BRRR_OK;
}

extern "C" void *brrr_model_stream(brrr_model *m) { return m ? (void *)m->stream : nullptr; }
extern "C" int brrr_model_launches_per_step(const brrr_model *m, int want) { return m ? (want ? m->launches_head : m->launches_nohead) : 0; }

extern "C" uint64_t brrr_model_bytes_per_step(const brrr_model *m, uint32_t pos) {
    if (!m) return 0;
    const brrr_cfg &c = m->cfg;
    const uint64_t d = c.n_embd, nh = c.n_head, nkv = c.n_head_kv, hd = c.head_dim, nb = d / 32, ne = c.n_expert, k = c.n_expert_used;
    auto q8 = [](uint64_t rows, uint64_t cols) { return rows * cols + rows * (cols / 32) * 4; };
    uint64_t per_layer = 0;
    per_layer += k * 3 * d * nb * 17;                       // MXFP4 gate, up, down of the k selected experts
    per_layer += q8((nh + 2 * nkv) * hd, d) + q8(d, nh * hd);
    per_layer += ne * d * 4 + ne * 4;                       // router
    per_layer += ((nh + 2 * nkv) * hd + d) * 4 + k * 3 * d * 4;   // biases
    per_layer += 2 * d * 4 + nh * 4;                        // norms, sinks
    uint64_t total = per_layer * c.n_layer;
    for (int il = 0; il < c.n_layer; il++) {
        uint64_t start = ((il + 1) % 2 != 0 && (uint64_t)c.sliding_window < BRRR_MAXSEQ) ? (pos + 1 > (uint64_t)c.sliding_window ? pos + 1 - c.sliding_window : 0) : 0;
        total += (pos - start + 1) * nkv * hd * 4 * 2;      // f32 K and V
    }
    total += q8(c.n_vocab, d) + d * 4 + d * 2;              // head, output norm, embedding row
    return total;
}

static int run_graph(brrr_model *m, bool want, bool safe = false) {
    if (m->ep && !m->ep_attached) return BRRR_ERR_STATE;
    safe = safe || m->spec_off;
    cudaGraphExec_t g = safe ? (want ? m->g_head_safe : m->g_nohead_safe) : (want ? m->g_head : m->g_nohead);
    CU(cudaGraphLaunch(g, m->stream));
    return BRRR_OK;
}

extern "C" uint64_t brrr_model_spec_redos(const brrr_model *m) { return m ? m->spec_redos : 0; }
extern "C" uint64_t brrr_model_wait_fallbacks(const brrr_model *m) { return m ? m->wait_fallbacks : 0; }

// The fold of the speculative step takes the exact routing from words the router publishes on
// another branch of the graph; nothing guarantees that the two branches run at the same time, so
// its bounded wait can run out.  The kernel then flags the step like a missed speculation (error
// word DEV_ERR_PEER_TIMEOUT, spec_fail_step = the step).  Here: the stream is idle; clear the error,
// bring the fold's sequence number back in line with the router's, and never speculate again on
// this model - the caller re-runs the flagged step with the plain graph.  Returns false when the
// error is not of that kind (the caller reports BRRR_ERR_STATE).
static bool recover_from_router_wait(brrr_model *m, uint32_t err) {
    if (err != (uint32_t)DEV_ERR_PEER_TIMEOUT || !m->use_spec || m->spec_off || m->ep) return false;
    if (cudaMemsetAsync(&m->st->err, 0, 4, m->stream) != cudaSuccess) return false;
    if (cudaMemcpyAsync(&m->st->fold_seq, &m->st->router_seq, 4, cudaMemcpyDeviceToDevice, m->stream) != cudaSuccess) return false;
    m->spec_off = true;
    m->wait_fallbacks++;
    return true;
}

extern "C" int brrr_forward(brrr_model *m, uint32_t tok, uint32_t pos, int want, uint32_t *out_tok) {
    if (!m) return BRRR_ERR_ARG;
    if (tok >= (uint32_t)m->cfg.n_vocab || pos >= BRRR_MAXSEQ) return BRRR_ERR_RANGE;
    CU(cudaSetDevice(m->device));
    m->h_in[0] = tok; m->h_in[1] = pos;
    CU(cudaMemcpyAsync(m->st, m->h_in, 8, cudaMemcpyHostToDevice, m->stream));   // DevState.tok, .pos
    TRY(run_graph(m, want != 0));
    CU(cudaMemcpyAsync(m->h_out, m->st, 32, cudaMemcpyDeviceToHost, m->stream));   // tok .. err
    CU(cudaStreamSynchronize(m->stream));
    if (m->h_out[6] != 0 && !recover_from_router_wait(m, m->h_out[6])) {
        snprintf(g_cuda_err, sizeof g_cuda_err, "device wait timed out (code %u)", m->h_out[6]);
        return BRRR_ERR_STATE;
    }
    if (m->h_out[7] != 0xFFFFFFFFu) {
        // the router estimate missed an expert somewhere in this step (or the fold gave up waiting
        // for the router): run it again without speculation
        m->spec_redos++;
        CU(cudaMemsetAsync(&m->st->spec_fail_step, 0xFF, 4, m->stream));
        CU(cudaMemcpyAsync(m->st, m->h_in, 8, cudaMemcpyHostToDevice, m->stream));
        TRY(run_graph(m, want != 0, true));
        CU(cudaMemcpyAsync(m->h_out, m->st, 32, cudaMemcpyDeviceToHost, m->stream));
        CU(cudaStreamSynchronize(m->stream));
        if (m->h_out[6] != 0) return BRRR_ERR_STATE;
    }
    if (want && out_tok) *out_tok = m->h_out[0];
    return BRRR_OK;
}

static int moe_tile_enqueue(brrr_model *m, int il, const float *d_xn, float *d_x, int ntok);

// Up to BRRR_TILE_MAX token rows walk the layers together (forward_tile_worker, src/bin/engine_gpt2.rs:1011-1250:
// every stage gains a token dimension, weight row outer, tokens inner).  A row is (token, position,
// sequence): consecutive positions of one sequence for a prompt tile, one position each of several
// sequences for batched decode.  Per layer: norm + Q8 of every row, q|k|v for all rows from one pass over
// the weights, RoPE + cache append of every row's k / v, attention of all rows in one launch (causal
// inside a tile: a row sees the rows before it through the cache), o-proj for all rows, FFN norm, and
// the MoE block on the tensor-core tile kernels.  Every value is bit-identical to the token-serial
// schedule.  Everything is read from device arrays (tl_toks, tl_pos, tl_seq), so the enqueue is
// captured once per row count and replayed.
constexpr int ROWS_SLOTS = 64;          // pinned descriptor slots of rows_run
// what the rows of a pass are: a prompt tile on the model's own cache, rows of any sequences of a batch, or a prompt tile of one
// sequence of a batch (rows of one sequence with ascending positions share their K / V tiles in attention)
enum { ROWS_PROMPT = 0, ROWS_BATCH = 1, ROWS_BATCH_PROMPT = 2 };

static int rows_alloc(brrr_model *m) {
    if (m->tl_x) return BRRR_OK;
    const brrr_cfg &c = m->cfg;
    const int d = c.n_embd, nb = d / 32, qkv_rows = (c.n_head + 2 * c.n_head_kv) * c.head_dim, ao = c.n_head * c.head_dim;
    const size_t R = BRRR_TILE_MAX;
    TRY(m->alloc(&m->tl_x, R * d)); TRY(m->alloc(&m->tl_xn, R * d));
    TRY(m->alloc(&m->tl_qkv, R * qkv_rows)); TRY(m->alloc(&m->tl_ao, R * ao));
    TRY(m->alloc(&m->tl_nq, R * d)); TRY(m->alloc(&m->tl_ns, R * nb));
    TRY(m->alloc(&m->tl_aq, R * ao)); TRY(m->alloc(&m->tl_as, R * (ao / 32)));
    TRY(m->alloc(&m->tl_toks, R)); TRY(m->alloc(&m->tl_pos, R)); TRY(m->alloc(&m->tl_seq, R));
    CU(cudaMallocHost(&m->h_tile, (size_t)ROWS_SLOTS * 3 * R * sizeof(uint32_t)));
    return BRRR_OK;
}

static int enqueue_rows(brrr_model *m, int n, int kind, bool pdl) {
    const bool batch = kind != ROWS_PROMPT, one_sequence = kind != ROWS_BATCH;
    const brrr_cfg &c = m->cfg;
    const int d = c.n_embd, nh = c.n_head, nkv = c.n_head_kv, qkv_rows = (nh + 2 * nkv) * c.head_dim;
    cudaStream_t s = m->stream;
    launch_embed_tile(m->tok_embd, d, m->tl_toks, n, m->tl_x, s);
    for (int il = 0; il < c.n_layer; il++) {
        Layer &ly = m->L[il];
        int window = ((il + 1) % 2 != 0) ? c.sliding_window : 0;
        if (window >= BRRR_MAXSEQ) window = 0;
        float *kc = batch ? m->kcb[il] : ly.kc, *vc = batch ? m->vcb[il] : ly.vc;
        const size_t seq_stride = batch ? (size_t)nkv * BRRR_MAXSEQ * c.head_dim : 0;
        // the first kernel after a plain launch takes the full dependency
        CUL(launch_rmsnorm_quant(m->tl_x, ly.attn_norm, c.rms_eps, d, nullptr, m->tl_nq, m->tl_ns, false, s, n));
        CUL(launch_q8_rows(ly.wqkv, m->tl_nq, m->tl_ns, n, ly.bqkv, m->tl_qkv, qkv_rows, Q8_EPI_BIAS, pdl, s, m->st));
        CUL(launch_kv_append_rows(m->tl_qkv, qkv_rows, nh, nkv, kc, vc, seq_stride, m->rope, m->tl_pos, m->tl_seq, n, pdl, s));
        // prompt tiles (rows of one sequence, ascending positions) share their K / V tiles; rows of different sequences cannot
        const int group = nh / nkv;
        if (one_sequence && !m->no_attn_rows && group <= 32 && (group & (group - 1)) == 0)
            CUL(launch_attn_rows(m->tl_qkv, qkv_rows, kc, vc, seq_stride, m->rope, ly.sinks, nh, nkv, window, m->tl_pos, m->tl_seq, n, m->tl_ao, m->tl_aq,
                                 m->tl_as, m->st, pdl, s));
        else
            CUL(launch_attn_decode(m->tl_qkv, kc, vc, m->rope, ly.sinks, nh, nkv, nullptr, 0, window, m->tl_ao, m->tl_aq, m->tl_as, m->st, pdl, s, 0,
                                   m->tl_pos, m->tl_seq, seq_stride, qkv_rows, n));
        CUL(launch_q8_rows(ly.wo, m->tl_aq, m->tl_as, n, ly.bo, m->tl_x, d, Q8_EPI_RESID_BIAS, pdl, s, m->st));
        CUL(launch_rmsnorm_quant(m->tl_x, ly.ffn_norm, c.rms_eps, d, m->tl_xn, m->tl_nq, m->tl_ns, pdl, s, n));
        TRY(moe_tile_enqueue(m, il, m->tl_xn, m->tl_x, n));
    }
    CU(cudaGetLastError());
    return BRRR_OK;
}

// Run the layers for the n rows described by (toks, pos, seq) (host arrays): the descriptors go through a
// pinned slot of their own to the device arrays, then the captured enqueue is replayed (captured at the
// first use of each row count; a direct run comes first so that every kernel has its attributes set).
static int rows_run(brrr_model *m, int n, const uint32_t *toks, const uint32_t *pos, const uint32_t *seq, int kind) {
    TRY(rows_alloc(m));
    const int R = BRRR_TILE_MAX;
    uint32_t *h = m->h_tile + (size_t)(m->h_tile_next++ % ROWS_SLOTS) * 3 * R;
    if (m->h_tile_next % ROWS_SLOTS == 0) CU(cudaStreamSynchronize(m->stream));        // the ring of pinned slots wraps: nothing may still be reading them
    for (int t = 0; t < n; t++) { h[t] = toks[t]; h[R + t] = pos[t]; h[2 * R + t] = seq ? seq[t] : 0u; }
    CU(cudaMemcpyAsync(m->tl_toks, h, (size_t)n * 4, cudaMemcpyHostToDevice, m->stream));
    CU(cudaMemcpyAsync(m->tl_pos, h + R, (size_t)n * 4, cudaMemcpyHostToDevice, m->stream));
    CU(cudaMemcpyAsync(m->tl_seq, h + 2 * R, (size_t)n * 4, cudaMemcpyHostToDevice, m->stream));
    cudaGraphExec_t &g = m->g_rows[kind][n];
    if (g) { CU(cudaGraphLaunch(g, m->stream)); return BRRR_OK; }
    TRY(enqueue_rows(m, n, kind, false));
    if (!m->rows_graph_failed) {
        CU(cudaStreamSynchronize(m->stream));
        cudaGraph_t gr = nullptr;
        CU(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
        int st = enqueue_rows(m, n, kind, m->use_pdl);
        cudaError_t e = cudaStreamEndCapture(m->stream, &gr);
        if (!(st == BRRR_OK && e == cudaSuccess && cudaGraphInstantiate(&g, gr, 0) == cudaSuccess)) { g = nullptr; m->rows_graph_failed = true; (void)cudaGetLastError(); }
        if (gr) cudaGraphDestroy(gr);
    }
    return BRRR_OK;
}

extern "C" int brrr_forward_tile(brrr_model *m, const uint32_t *toks, uint32_t n, uint32_t pos0, int want, uint32_t *out_tok) {
    if (!m || !toks || n == 0) return BRRR_ERR_ARG;
    if (pos0 + n > BRRR_MAXSEQ) return BRRR_ERR_RANGE;
    for (uint32_t i = 0; i < n; i++) if (toks[i] >= (uint32_t)m->cfg.n_vocab) return BRRR_ERR_RANGE;
    CU(cudaSetDevice(m->device));
    // Both schedules give the same bits.  Expert-parallel ranks stay token-serial.
    const bool serial = m->ep || !m->tile_prefill;
    const brrr_cfg &c = m->cfg;
    const int d = c.n_embd;
    bool tiled_last = false;
    const uint32_t T = (uint32_t)m->tile_rows;
    for (uint32_t i0 = 0; i0 < n; i0 += T) {
        const uint32_t cnt = n - i0 < T ? n - i0 : T;
        const bool last = i0 + cnt == n;
        if (serial || cnt == 1) {
            for (uint32_t i = i0; i < i0 + cnt; i++) {
                int st = brrr_forward(m, toks[i], pos0 + i, want && i == n - 1, out_tok);
                if (st != BRRR_OK) return st;
            }
            continue;
        }
        uint32_t pos[BRRR_TILE_MAX];
        for (uint32_t t = 0; t < cnt; t++) pos[t] = pos0 + i0 + t;
        TRY(rows_run(m, (int)cnt, toks + i0, pos, nullptr, ROWS_PROMPT));
        if (last) {
            // leave the engine as the serial schedule would after the tile's last token
            cudaStream_t s = m->stream;
            CU(cudaMemcpyAsync(m->x, m->tl_x + (size_t)(cnt - 1) * d, (size_t)d * sizeof(float), cudaMemcpyDeviceToDevice, s));
            m->h_in[0] = toks[n - 1]; m->h_in[1] = pos0 + n - 1;
            CU(cudaMemcpyAsync(m->st, m->h_in, 8, cudaMemcpyHostToDevice, s));
            if (want) {
                CUL(launch_rmsnorm_quant(m->x, m->out_norm, c.rms_eps, d, nullptr, m->xq, m->xs, false, s));
                CUL(launch_q8_head(m->head, m->xq, m->xs, m->logits, m->st, false, s));
                launch_finish_token(m->st, s);
            }
            CU(cudaGetLastError());
            // (h_in is host-pageable-safe here: the stream is synchronised below before it is reused)
        }
        tiled_last = last;
    }
    if (tiled_last) {
        CU(cudaMemcpyAsync(m->h_out, m->st, 32, cudaMemcpyDeviceToHost, m->stream));   // tok .. err
        CU(cudaStreamSynchronize(m->stream));
        if (m->h_out[6] != 0) { snprintf(g_cuda_err, sizeof g_cuda_err, "device wait timed out (code %u)", m->h_out[6]); return BRRR_ERR_STATE; }
        if (want && out_tok) *out_tok = m->h_out[0];
    }
    return BRRR_OK;
}

// ---- batched decode over independent sequences: one KV cache per sequence, rows = (token, position, sequence)
extern "C" int brrr_batch_open(brrr_model *m, int nseq) {
    if (!m || nseq < 1 || nseq > BRRR_BATCH_MAX) return BRRR_ERR_ARG;
    if (m->ep || m->nseq) return BRRR_ERR_STATE;
    CU(cudaSetDevice(m->device));
    const brrr_cfg &c = m->cfg;
    const size_t per_seq = (size_t)c.n_head_kv * BRRR_MAXSEQ * c.head_dim;
    m->kcb.assign(c.n_layer, nullptr); m->vcb.assign(c.n_layer, nullptr);
    for (int il = 0; il < c.n_layer; il++) { TRY(m->alloc(&m->kcb[il], per_seq * nseq)); TRY(m->alloc(&m->vcb[il], per_seq * nseq)); }
    TRY(m->alloc(&m->bt_logits, (size_t)BRRR_TILE_MAX * c.n_vocab));
    TRY(m->alloc(&m->bt_tok, BRRR_TILE_MAX));
    TRY(rows_alloc(m));
    m->nseq = nseq;
    return BRRR_OK;
}

static int batch_check(brrr_model *m, int n, const uint32_t *toks, const uint32_t *pos, const uint32_t *seq) {
    if (!m || !toks || !pos || !seq || n < 1 || n > BRRR_TILE_MAX) return BRRR_ERR_ARG;
    if (!m->nseq) return BRRR_ERR_STATE;
    for (int t = 0; t < n; t++)
        if (toks[t] >= (uint32_t)m->cfg.n_vocab || pos[t] >= BRRR_MAXSEQ || seq[t] >= (uint32_t)m->nseq) return BRRR_ERR_RANGE;
    return BRRR_OK;
}

// The layers for n rows on the sequences' caches; with out_toks, the vocabulary projection and argmax of every row.
static int batch_rows(brrr_model *m, int n, const uint32_t *toks, const uint32_t *pos, const uint32_t *seq, uint32_t *out_toks, float *out_logits,
                      int kind = ROWS_BATCH) {
    TRY(batch_check(m, n, toks, pos, seq));
    CU(cudaSetDevice(m->device));
    const brrr_cfg &c = m->cfg;
    cudaStream_t s = m->stream;
    TRY(rows_run(m, n, toks, pos, seq, kind));
    if (out_toks || out_logits) {
        CUL(launch_rmsnorm_quant(m->tl_x, m->out_norm, c.rms_eps, c.n_embd, nullptr, m->tl_nq, m->tl_ns, false, s, n));
        // from 8 rows on the vocabulary projection runs on the tensor cores (measured: 3726 against 3564 tok/s at 64 rows, 1790 against
        // 1754 at 16; BRRR_HEAD_TILE_MIN=n moves the threshold, above BRRR_TILE_MAX = never); same bits either way
        static const int head_tile_min = [] { const char *e = getenv("BRRR_HEAD_TILE_MIN"); const int v = e ? atoi(e) : 0; return v >= 1 ? v : 8; }();
        CUL(launch_q8_rows(m->head, m->tl_nq, m->tl_ns, n, nullptr, m->bt_logits, c.n_vocab, Q8_EPI_PLAIN, false, s, m->st, n >= head_tile_min ? 1 : 0));
        launch_rows_argmax(m->bt_logits, c.n_vocab, n, m->bt_tok, s);
        CU(cudaGetLastError());
        CU(cudaMemcpyAsync(m->h_out + 8, m->bt_tok, (size_t)n * 4, cudaMemcpyDeviceToHost, s));
        if (out_logits) CU(cudaMemcpyAsync(out_logits, m->bt_logits, (size_t)n * c.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    CU(cudaMemcpyAsync(m->h_out, m->st, 32, cudaMemcpyDeviceToHost, s));
    CU(cudaStreamSynchronize(s));
    if (m->h_out[6] != 0) { snprintf(g_cuda_err, sizeof g_cuda_err, "device wait timed out (code %u)", m->h_out[6]); return BRRR_ERR_STATE; }
    if (out_toks) for (int t = 0; t < n; t++) out_toks[t] = m->h_out[8 + t];
    return BRRR_OK;
}

extern "C" int brrr_batch_step(brrr_model *m, int n, const uint32_t *toks, const uint32_t *pos, const uint32_t *seq, uint32_t *out_toks) {
    if (!out_toks) return BRRR_ERR_ARG;
    return batch_rows(m, n, toks, pos, seq, out_toks, nullptr);
}

extern "C" int brrr_batch_step_logits(brrr_model *m, int n, const uint32_t *toks, const uint32_t *pos, const uint32_t *seq, uint32_t *out_toks, float *out_logits) {
    if (!out_toks || !out_logits) return BRRR_ERR_ARG;
    return batch_rows(m, n, toks, pos, seq, out_toks, out_logits);
}

extern "C" int brrr_batch_prefill(brrr_model *m, uint32_t seq, const uint32_t *toks, uint32_t n, uint32_t pos0) {
    if (!m || !toks || n == 0) return BRRR_ERR_ARG;
    if (!m->nseq) return BRRR_ERR_STATE;
    if (pos0 + n > BRRR_MAXSEQ || seq >= (uint32_t)m->nseq) return BRRR_ERR_RANGE;
    uint32_t pos[BRRR_TILE_MAX], sq[BRRR_TILE_MAX];
    for (uint32_t i0 = 0; i0 < n; i0 += BRRR_TILE_MAX) {
        const uint32_t cnt = n - i0 < BRRR_TILE_MAX ? n - i0 : BRRR_TILE_MAX;
        for (uint32_t t = 0; t < cnt; t++) { pos[t] = pos0 + i0 + t; sq[t] = seq; }
        TRY(batch_rows(m, (int)cnt, toks + i0, pos, sq, nullptr, nullptr, cnt > 1 ? ROWS_BATCH_PROMPT : ROWS_BATCH));
    }
    return BRRR_OK;
}

extern "C" int brrr_model_set_tile_prefill(brrr_model *m, int on) {
    if (!m) return BRRR_ERR_ARG;
    m->tile_prefill = on != 0;
    return BRRR_OK;
}

extern "C" int brrr_decode_enqueue(brrr_model *m, uint32_t first_tok, uint32_t pos, uint32_t n) {
    if (!m) return BRRR_ERR_ARG;
    if (first_tok >= (uint32_t)m->cfg.n_vocab || n == 0 || n > BRRR_MAXSEQ || pos + n > BRRR_MAXSEQ) return BRRR_ERR_RANGE;
    CU(cudaSetDevice(m->device));
    m->h_in[0] = first_tok; m->h_in[1] = pos; m->h_in[2] = 0;
    m->run_tok = first_tok; m->run_pos = pos;
    CU(cudaMemcpyAsync(m->st, m->h_in, 12, cudaMemcpyHostToDevice, m->stream));  // tok, pos, n_out = 0
    for (uint32_t i = 0; i < n; i++) TRY(run_graph(m, true));
    return BRRR_OK;
}

extern "C" int brrr_decode_wait(brrr_model *m, uint32_t n, uint32_t *out_toks) {
    if (!m || !out_toks || n == 0 || n > BRRR_MAXSEQ) return BRRR_ERR_ARG;
    CU(cudaSetDevice(m->device));
    CU(cudaMemcpyAsync(m->h_out, m->st->out, n * sizeof(uint32_t), cudaMemcpyDeviceToHost, m->stream));
    for (int guard = 0; guard < (int)n + 1; guard++) {
        CU(cudaMemcpyAsync(m->h_in, &m->st->err, 8, cudaMemcpyDeviceToHost, m->stream));   // err, spec_fail_step
        CU(cudaStreamSynchronize(m->stream));
        if (m->h_in[0] != 0 && !recover_from_router_wait(m, m->h_in[0])) {
            snprintf(g_cuda_err, sizeof g_cuda_err, "device wait timed out (code %u)", m->h_in[0]);
            return BRRR_ERR_STATE;
        }
        const uint32_t f = m->h_in[1];
        if (f >= n) break;
        // Step f ran with an expert set the exact router did not confirm: its token and every later
        // one are void.  Resume from step f without speculation (the KV cache entries of the voided
        // steps are simply overwritten).
        m->spec_redos++;
        CU(cudaMemsetAsync(&m->st->spec_fail_step, 0xFF, 4, m->stream));
        m->h_in[0] = f ? m->h_out[f - 1] : m->run_tok; m->h_in[1] = m->run_pos + f; m->h_in[2] = f;
        CU(cudaMemcpyAsync(m->st, m->h_in, 12, cudaMemcpyHostToDevice, m->stream));
        TRY(run_graph(m, true, true));                                  // the failed step, exactly
        for (uint32_t i = f + 1; i < n; i++) TRY(run_graph(m, true));   // the rest speculates again
        CU(cudaMemcpyAsync(m->h_out, m->st->out, n * sizeof(uint32_t), cudaMemcpyDeviceToHost, m->stream));
    }
    memcpy(out_toks, m->h_out, n * sizeof(uint32_t));
    return BRRR_OK;
}

extern "C" int brrr_decode(brrr_model *m, uint32_t first_tok, uint32_t pos, uint32_t n, uint32_t *out_toks) {
    if (!out_toks) return BRRR_ERR_ARG;
    int s = brrr_decode_enqueue(m, first_tok, pos, n);
    if (s != BRRR_OK) return s;
    return brrr_decode_wait(m, n, out_toks);
}

extern "C" int brrr_logits(brrr_model *m, float *out) {
    if (!m || !out) return BRRR_ERR_ARG;
    CU(cudaSetDevice(m->device));
    CU(cudaMemcpyAsync(out, m->logits, (size_t)m->cfg.n_vocab * 4, cudaMemcpyDeviceToHost, m->stream));
    CU(cudaStreamSynchronize(m->stream));
    return BRRR_OK;
}

extern "C" int brrr_hidden(brrr_model *m, float *out) {
    if (!m || !out) return BRRR_ERR_ARG;
    CU(cudaSetDevice(m->device));
    CU(cudaMemcpyAsync(out, m->x, (size_t)m->cfg.n_embd * 4, cudaMemcpyDeviceToHost, m->stream));
    CU(cudaStreamSynchronize(m->stream));
    return BRRR_OK;
}

extern "C" int brrr_forward_trace(brrr_model *m, uint32_t tok, uint32_t pos, float *trace) {
    if (!m || !trace) return BRRR_ERR_ARG;
    if (tok >= (uint32_t)m->cfg.n_vocab || pos >= BRRR_MAXSEQ) return BRRR_ERR_RANGE;
    CU(cudaSetDevice(m->device));
    size_t n = (size_t)(m->cfg.n_layer + 1) * m->cfg.n_embd;
    float *dev = nullptr;
    CU(cudaMalloc(&dev, n * 4));
    m->h_in[0] = tok; m->h_in[1] = pos;
    cudaMemcpyAsync(m->st, m->h_in, 8, cudaMemcpyHostToDevice, m->stream);
    int s = enqueue_step(m, true, dev, nullptr);
    if (s == BRRR_OK && cudaMemcpyAsync(trace, dev, n * 4, cudaMemcpyDeviceToHost, m->stream) != cudaSuccess) s = BRRR_ERR_CUDA;
    if (cudaStreamSynchronize(m->stream) != cudaSuccess) s = BRRR_ERR_CUDA;
    cudaFree(dev);
    return s;
}

extern "C" int brrr_rope_table(const brrr_cfg *cfg, float *out) {
    if (!cfg || !out || cfg->head_dim <= 0 || cfg->head_dim % 2) return BRRR_ERR_ARG;
    rope_table_host(*cfg, out);
    return BRRR_OK;
}

extern "C" int brrr_moe_ffn_step(brrr_model *m, int il, const float *d_xn, float *d_x, int32_t *d_top, float *d_wts) {
    if (!m || !d_xn || !d_x || il < 0 || il >= m->cfg.n_layer) return BRRR_ERR_ARG;
    CU(cudaSetDevice(m->device));
    const brrr_cfg &c = m->cfg;
    const int d = c.n_embd, topk = c.n_expert_used;
    Layer &ly = m->L[il];
    cudaStream_t s = m->stream;
    CUL(launch_ffn_in(d_xn, nullptr, c.rms_eps, d, ly.ginp, ly.ginp_b, c.n_expert, topk, m->rlogits, m->top, m->wts, &m->st->router_done, m->st, false, s));
    CUL(launch_gate_up(ly.gate, ly.up, ly.gate_b, ly.up_b, m->top, topk, d, d_xn, nullptr, c.rms_eps, nullptr, nullptr, m->hq, m->hs, nullptr, m->st, false, s));
    CUL(launch_down_combine(ly.down, ly.down_b, m->top, m->wts, nullptr, 0, topk, d, m->hq, m->hs, d_x, m->st, false, s));
    CU(cudaGetLastError());
    if (d_top) CU(cudaMemcpyAsync(d_top, m->top, topk * sizeof(int32_t), cudaMemcpyDeviceToDevice, s));
    if (d_wts) CU(cudaMemcpyAsync(d_wts, m->wts, topk * sizeof(float), cudaMemcpyDeviceToDevice, s));
    CU(cudaStreamSynchronize(s));
    return BRRR_OK;
}

// The same step through the tensor-core expert kernels (the ones the speculative decode step runs):
// exact router, Q8 of the normalised token, gate/up tiles, down tiles with the last-arriver fold.
// BRRR_ERR_STATE when the model was opened without the tile-unit copy of the experts.
extern "C" int brrr_moe_ffn_step_tc(brrr_model *m, int il, const float *d_xn, float *d_x, int32_t *d_top, float *d_wts) {
    if (!m || !d_xn || !d_x || il < 0 || il >= m->cfg.n_layer) return BRRR_ERR_ARG;
    if (!m->use_mxt || m->ep) return BRRR_ERR_STATE;
    CU(cudaSetDevice(m->device));
    const brrr_cfg &c = m->cfg;
    const int d = c.n_embd, topk = c.n_expert_used;
    Layer &ly = m->L[il];
    cudaStream_t s = m->stream;
    CUL(launch_ffn_in(d_xn, nullptr, c.rms_eps, d, ly.ginp, ly.ginp_b, c.n_expert, topk, m->rlogits, m->top, m->wts, &m->st->router_done, m->st, false, s));
    launch_quant_q8(d_xn, d, m->xq, m->xs, s);
    launch_xt_bimg(m->xq, d / 32, m->ximg, s);
    CUL(launch_gate_up_t(ly.gu_t, ly.gate_b, ly.up_b, m->top, nullptr, 0, topk, d, m->ximg, m->xs, m->hq, m->hs, m->himg, m->st, false, s));
    CUL(launch_down_t(ly.down_t, ly.down_b, m->top, m->wts, nullptr, 0, topk, d, m->himg, m->hs, d_x, m->dpart, m->dcount, m->st, false, s));
    CU(cudaGetLastError());
    if (d_top) CU(cudaMemcpyAsync(d_top, m->top, topk * sizeof(int32_t), cudaMemcpyDeviceToDevice, s));
    if (d_wts) CU(cudaMemcpyAsync(d_wts, m->wts, topk * sizeof(float), cudaMemcpyDeviceToDevice, s));
    CU(cudaStreamSynchronize(s));
    return BRRR_OK;
}

extern "C" int brrr_model_uses_tensor_experts(const brrr_model *m) { return m && m->use_mxt ? 1 : 0; }

// MoE FFN of one layer for a tile of up to BRRR_TILE_MAX (64) normalised tokens: per-token router (one launch),
// routing lists per expert, then three grouped tensor-core matmuls (gate, up, down) that read every
// needed expert matrix once for all its tokens, SwiGLU + Q8 per (token, slot), and the fold in slot
// order.  Bit-identical to brrr_moe_ffn_step applied to the tokens one by one.
// Enqueue only (no synchronisation): the tile's MoE step on m->stream.
static int moe_tile_enqueue(brrr_model *m, int il, const float *d_xn, float *d_x, int ntok) {
    const brrr_cfg &c = m->cfg;
    const int d = c.n_embd, nb = d / 32, topk = c.n_expert_used, ne = c.n_expert, R = BRRR_TILE_MAX, np_ = R * topk;
    if (!m->tl_xq) {
        TRY(m->alloc(&m->tl_xq, (size_t)R * d)); TRY(m->alloc(&m->tl_xs, (size_t)R * nb));
        TRY(m->alloc(&m->tl_logits, (size_t)R * ne)); TRY(m->alloc(&m->tl_top, R * 8)); TRY(m->alloc(&m->tl_wts, R * 8));
        TRY(m->alloc(&m->tl_counter, R)); TRY(m->alloc(&m->tl_cnt, ne)); TRY(m->alloc(&m->tl_list, (size_t)ne * R));
        TRY(m->alloc(&m->tl_gu, (size_t)np_ * 2 * d)); TRY(m->alloc(&m->tl_hq, (size_t)np_ * d)); TRY(m->alloc(&m->tl_hs, (size_t)np_ * nb));
        TRY(m->alloc(&m->tl_part, (size_t)np_ * d));
        CU(cudaMemsetAsync(m->tl_counter, 0, R * sizeof(unsigned int), m->stream));
    }
    Layer &ly = m->L[il];
    cudaStream_t s = m->stream;
    launch_quant_q8(d_xn, ntok * d, m->tl_xq, m->tl_xs, s);
    CUL(launch_ffn_in(d_xn, nullptr, c.rms_eps, d, ly.ginp, ly.ginp_b, ne, topk, m->tl_logits, m->tl_top, m->tl_wts, m->tl_counter, m->st, false, s, ntok));
    launch_tile_route(m->tl_top, ntok, topk, ne, m->tl_cnt, m->tl_list, s);
    CUL(launch_mx_tile_experts(ly.gate, ne, d, m->tl_cnt, m->tl_list, ntok, topk, m->tl_xq, m->tl_xs, ly.gate_b, m->tl_gu, 2 * d, 0, m->st, s));
    CUL(launch_mx_tile_experts(ly.up, ne, d, m->tl_cnt, m->tl_list, ntok, topk, m->tl_xq, m->tl_xs, ly.up_b, m->tl_gu, 2 * d, d, m->st, s));
    launch_swiglu_quant(m->tl_gu, ntok * topk, d, m->tl_hq, m->tl_hs, s);
    CUL(launch_mx_tile_experts(ly.down, ne, d, m->tl_cnt, m->tl_list, ntok, 1, m->tl_hq, m->tl_hs, ly.down_b, m->tl_part, d, 0, m->st, s));
    launch_tile_combine(m->tl_part, m->tl_wts, topk, d, ntok, d_x, s);
    CU(cudaGetLastError());
    return BRRR_OK;
}

extern "C" int brrr_moe_ffn_tile(brrr_model *m, int il, const float *d_xn, float *d_x, int ntok, int32_t *d_top, float *d_wts) {
    if (!m || !d_xn || !d_x || il < 0 || il >= m->cfg.n_layer || ntok < 1 || ntok > BRRR_TILE_MAX) return BRRR_ERR_ARG;
    if (m->ep) return BRRR_ERR_STATE;
    CU(cudaSetDevice(m->device));
    const int topk = m->cfg.n_expert_used;
    cudaStream_t s = m->stream;
    TRY(moe_tile_enqueue(m, il, d_xn, d_x, ntok));
    if (d_top) CU(cudaMemcpy2DAsync(d_top, topk * sizeof(int32_t), m->tl_top, 8 * sizeof(int32_t), topk * sizeof(int32_t), ntok, cudaMemcpyDeviceToDevice, s));
    if (d_wts) CU(cudaMemcpy2DAsync(d_wts, topk * sizeof(float), m->tl_wts, 8 * sizeof(float), topk * sizeof(float), ntok, cudaMemcpyDeviceToDevice, s));
    CU(cudaStreamSynchronize(s));
    uint32_t derr = 0;
    CU(cudaMemcpy(&derr, &m->st->err, 4, cudaMemcpyDeviceToHost));
    if (derr) { snprintf(g_cuda_err, sizeof g_cuda_err, "device wait timed out (code %u)", derr); return BRRR_ERR_STATE; }
    return BRRR_OK;
}

// Algorithmic bytes one launch of a stage class reads (weights in run-time format + f32 KV).
static uint64_t stage_bytes_per_launch(const brrr_model *m, int stage, uint32_t pos) {
    const brrr_cfg &c = m->cfg;
    const uint64_t d = c.n_embd, nh = c.n_head, nkv = c.n_head_kv, hd = c.head_dim, nb = d / 32, ne = c.n_expert, k = c.n_expert_used;
    auto q8 = [](uint64_t rows, uint64_t cols) { return rows * cols + rows * (cols / 32) * 4; };
    switch (stage) {
    case ST_EMBED: return d * 2;
    case ST_QKV: return q8((nh + 2 * nkv) * hd, d) + (nh + 2 * nkv) * hd * 4 + d * 8;
    case ST_ATTN: {
        uint64_t tot = 0;
        for (int il = 0; il < c.n_layer; il++) {
            uint64_t start = ((il + 1) % 2 != 0 && (uint64_t)c.sliding_window < BRRR_MAXSEQ) ? (pos + 1 > (uint64_t)c.sliding_window ? pos + 1 - c.sliding_window : 0) : 0;
            tot += (pos - start + 1) * nkv * hd * 8;
        }
        return tot / c.n_layer;
    }
    case ST_OPROJ: return q8(d, nh * hd) + d * 4;
    case ST_ROUTER: return ne * d * 4 + ne * 4 + d * 8;
    case ST_GATE_UP: return k * 2 * d * nb * 17 + k * 2 * d * 4 + d * 8;
    case ST_DOWN: return k * d * nb * 17 + k * d * 4;
    case ST_FOLD: return 2 * k * d * 4 + 3 * d * 4 + d + nb * 4;       // partial sums, biases, residual in and out, norm weights, Q8 image out
    case ST_HEAD_NORM: return d * 8;
    case ST_HEAD: return q8(c.n_vocab, d);
    }
    return 0;
}

extern "C" int brrr_stage_count(void) { return ST_COUNT; }
extern "C" const char *brrr_stage_name(int stage) { return stage >= 0 && stage < ST_COUNT ? kStageNames[stage] : ""; }

extern "C" int brrr_stage_time(brrr_model *m, int stage, uint32_t pos, int reps, float *ms_per_launch, uint64_t *bytes_per_launch, int *launches_per_step) {
    if (m && m->ep) return BRRR_ERR_STATE;      // per-kernel replays would not be matched by the peers
    if (!m || stage < 0 || stage >= ST_COUNT || stage == ST_FINISH || reps <= 0 || pos >= BRRR_MAXSEQ) return BRRR_ERR_ARG;
    CU(cudaSetDevice(m->device));
    cudaGraphExec_t g = nullptr;
    int n = 0;
    TRY(capture(m, true, &g, &n, 1u << stage));
    uint32_t saved[2];
    CU(cudaMemcpyAsync(saved, m->st, 8, cudaMemcpyDeviceToHost, m->stream));
    CU(cudaStreamSynchronize(m->stream));
    m->h_in[0] = saved[0]; m->h_in[1] = pos;
    CU(cudaMemcpyAsync(m->st, m->h_in, 8, cudaMemcpyHostToDevice, m->stream));
    cudaEvent_t e0, e1;
    CU(cudaEventCreate(&e0)); CU(cudaEventCreate(&e1));
    for (int i = 0; i < 3; i++) CU(cudaGraphLaunch(g, m->stream));
    CU(cudaEventRecord(e0, m->stream));
    for (int i = 0; i < reps; i++) CU(cudaGraphLaunch(g, m->stream));
    CU(cudaEventRecord(e1, m->stream));
    CU(cudaStreamSynchronize(m->stream));
    float ms = 0.0f;
    CU(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaGraphExecDestroy(g);
    m->h_in[0] = saved[0]; m->h_in[1] = saved[1];
    CU(cudaMemcpyAsync(m->st, m->h_in, 8, cudaMemcpyHostToDevice, m->stream));
    CU(cudaStreamSynchronize(m->stream));
    if (ms_per_launch) *ms_per_launch = n ? ms / ((float)reps * n) : 0.0f;
    if (bytes_per_launch) *bytes_per_launch = stage_bytes_per_launch(m, stage, pos);
    if (launches_per_step) *launches_per_step = n;
    return BRRR_OK;
}

#ifdef BRRR_TEST_HOOKS
// Test-hook builds only (not part of the public interface): the in-kernel clock stamps of the last step.
extern "C" int brrr_debug_stamps(brrr_model *m, long long *out256) {
    if (!m || !out256) return BRRR_ERR_ARG;
    CU(cudaSetDevice(m->device));
    CU(cudaMemcpyAsync(out256, m->st->stamps, 256 * sizeof(long long), cudaMemcpyDeviceToHost, m->stream));
    CU(cudaStreamSynchronize(m->stream));
    return BRRR_OK;
}
#endif
