// Host side of the qwen3moe engine: data-directory loader, synthetic-model builder, the decode step
// as one CUDA graph per token, and the model-level C ABI (brrr_qwen_* in include/brrr.h).
//
// It mirrors the reference's host program for this path (src/bin/engine_qwen2.rs): load_cfg
// (27-38), the manifest loader and per-layer tensors (512-545), the activation buffers (552-568)
// and run() (587-595) — with the 12-worker spin-barrier scheduler (302-451, 571-586) replaced by
// one graph launch per token.  K-quant tensors are used in the GGUF byte layout, as the reference
// uses them straight from the mapped blob.
#include "../../include/brrr.h"
#include "brrr_kernels.h"
#include "brrr_kq.cuh"
#include "brrr_synth.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <map>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

using namespace brrr;

#define QERR(...) snprintf(host_err_buf(), 512, __VA_ARGS__)
#define CU(call)                                                                                   \
    do {                                                                                           \
        cudaError_t _e = (call);                                                                   \
        if (_e != cudaSuccess) {                                                                   \
            QERR("%s:%d %s: %s", __FILE__, __LINE__, #call, cudaGetErrorString(_e));               \
            return BRRR_ERR_CUDA;                                                                  \
        }                                                                                          \
    } while (0)
#define TRY(expr) do { int _s = (expr); if (_s != BRRR_OK) return _s; } while (0)

namespace {

struct QLayer {
    float *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr, *ginp = nullptr;
    KMatDev wq{}, wk{}, wv{}, wo{}, gate{}, up{}, down{};
    float *kc = nullptr, *vc = nullptr;      // [kv head][position][head_dim]
};

struct QSource {
    bool synth = false;
    uint64_t seed = 0;
    const uint8_t *blob = nullptr;
    size_t blob_len = 0;
    struct Ent { uint32_t type; size_t off, nel; };
    std::map<std::string, Ent> idx;
};

const char *qkind_name(int kind) {
    switch (kind) {
    case BRRR_T_ATTN_NORM: return "attn_norm.weight"; case BRRR_T_FFN_NORM: return "ffn_norm.weight";
    case BRRR_T_Q_NORM: return "attn_q_norm.weight"; case BRRR_T_K_NORM: return "attn_k_norm.weight";
    case BRRR_T_WQ: return "attn_q.weight"; case BRRR_T_WK: return "attn_k.weight";
    case BRRR_T_WV: return "attn_v.weight"; case BRRR_T_WO: return "attn_output.weight";
    case BRRR_T_ROUTER_W: return "ffn_gate_inp.weight"; case BRRR_T_GATE: return "ffn_gate_exps.weight";
    case BRRR_T_UP: return "ffn_up_exps.weight"; case BRRR_T_DOWN: return "ffn_down_exps.weight";
    case BRRR_T_TOK_EMBD: return "token_embd.weight"; case BRRR_T_OUT_NORM: return "output_norm.weight";
    case BRRR_T_OUTPUT: return "output.weight";
    }
    return "?";
}

size_t ktype_bytes(uint32_t type, size_t nel) { return type == 0 ? nel * 4 : nel / 256 * (type == 12 ? 144 : 210); }

}  // namespace

struct brrr_qwen {
    brrr_qwen_cfg cfg{};
    int device = 0;
    cudaStream_t stream = nullptr;
    std::vector<QLayer> L;
    float *out_norm = nullptr, *rope = nullptr;
    KMatDev head{}, embd{};
    float *x = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *ao = nullptr, *hbuf = nullptr, *rlogits = nullptr,
          *logits = nullptr, *xs = nullptr, *as = nullptr, *hs = nullptr, *wts = nullptr;
    int8_t *xq = nullptr, *aq = nullptr, *hq = nullptr;
    int32_t *xsum = nullptr, *asum = nullptr, *hsum = nullptr, *top = nullptr;
    unsigned int *down_counter = nullptr;      // arrival counter of the down kernel's CTAs (self-resetting)
    DevState *st = nullptr;
    uint32_t *h_in = nullptr, *h_out = nullptr;
    cudaGraphExec_t g_head = nullptr, g_nohead = nullptr;
    int launches_head = 0, launches_nohead = 0;
    bool use_pdl = true;
    std::vector<void *> allocs;

    template <typename T> int alloc(T **p, size_t n) {
        void *vp = nullptr;
        if (cudaMalloc(&vp, n ? n * sizeof(T) : 16) != cudaSuccess) { QERR("cudaMalloc of %zu bytes failed", n * sizeof(T)); return BRRR_ERR_NOMEM; }
        allocs.push_back(vp);
        *p = (T *)vp;
        return BRRR_OK;
    }
    void release(void *vp) {          // give one allocation back early (raw bytes that were re-laid)
        for (size_t i = 0; i < allocs.size(); i++)
            if (allocs[i] == vp) { cudaFree(vp); allocs.erase(allocs.begin() + i); return; }
    }
};

namespace {

// Raw bytes of one tensor into device memory `dst`.  type: 0 (f32) is required exactly; for
// K-quant tensors *type_io names the wanted type on a synthetic source and receives the stored
// type (12 or 14) on a file source.
int qfetch(brrr_qwen *m, const QSource &s, uint32_t layer, int kind, uint32_t *type_io, size_t nel, void **dst_alloc) {
    char name[160];
    if (layer == BRRR_L_GLOBAL) snprintf(name, sizeof name, "%s", qkind_name(kind));
    else snprintf(name, sizeof name, "blk.%u.%s", layer, qkind_name(kind));
    uint32_t type = *type_io;
    const QSource::Ent *ent = nullptr;
    if (!s.synth) {
        auto it = s.idx.find(name);
        if (it == s.idx.end()) { QERR("missing tensor %s", name); return BRRR_ERR_IO; }
        ent = &it->second;
        if (type == 0 ? ent->type != 0 : (ent->type != 12 && ent->type != 14)) { QERR("tensor %s: unsupported type %u", name, ent->type); return BRRR_ERR_IO; }
        if (ent->nel != nel) { QERR("tensor %s: size mismatch", name); return BRRR_ERR_IO; }
        type = ent->type;
        if (ent->off + ktype_bytes(type, nel) > s.blob_len) { QERR("tensor %s exceeds blob", name); return BRRR_ERR_IO; }
    }
    size_t bytes = ktype_bytes(type, nel);
    uint8_t *dst = nullptr;
    TRY(m->alloc(&dst, bytes));
    if (s.synth) {
        launch_synth(s.seed, layer, kind, type, nel, dst, m->stream);
        CU(cudaGetLastError());
    } else {
        CU(cudaMemcpyAsync(dst, s.blob + ent->off, bytes, cudaMemcpyHostToDevice, m->stream));
        CU(cudaStreamSynchronize(m->stream));
    }
    *type_io = type;
    *dst_alloc = dst;
    return BRRR_OK;
}

int qload_f32(brrr_qwen *m, const QSource &s, uint32_t layer, int kind, size_t n, float **out) {
    uint32_t t = 0;
    void *p = nullptr;
    TRY(qfetch(m, s, layer, kind, &t, n, &p));
    *out = (float *)p;
    return BRRR_OK;
}

// Synthetic type scheme: down experts and the output head Q6_K, every other matrix Q4_K.
int qload_k(brrr_qwen *m, const QSource &s, uint32_t layer, int kind, int rows, int cols, KMatDev *out) {
    uint32_t t = (kind == BRRR_T_DOWN || kind == BRRR_T_OUTPUT) ? 14 : 12;
    void *p = nullptr;
    TRY(qfetch(m, s, layer, kind, &t, (size_t)rows * cols, &p));
    if (t == 14 && kind != BRRR_T_TOK_EMBD) {
        // Q6_K rows (210-byte superblocks, 2-byte aligned) are re-laid into aligned planes per row: a byte permutation
        uint8_t *planes = nullptr;
        TRY(m->alloc(&planes, (size_t)rows * q6k_plane_row_bytes(cols / 256)));
        launch_q6k_planes((const uint8_t *)p, (size_t)rows, cols, planes, m->stream);
        CU(cudaGetLastError());
        CU(cudaStreamSynchronize(m->stream));
        m->release(p);
        *out = KMatDev{planes, 14, rows, cols, 1};
        return BRRR_OK;
    }
    *out = KMatDev{(const uint8_t *)p, (int)t, rows, cols, 0};
    return BRRR_OK;
}

// cos/sin of pos * base^(-2i/hd) (engine_qwen2.rs:472-474), single precision host libm
void qrope_table_host(const brrr_qwen_cfg &c, float *tab) {
    const int half = c.head_dim / 2;
    for (int i = 0; i < half; i++) {
        float f = powf(c.rope_freq_base, -(2.0f * (float)i) / (float)c.head_dim);
        for (int pos = 0; pos < BRRR_MAXSEQ; pos++) {
            float theta = (float)pos * f;
            tab[((size_t)pos * half + i) * 2] = cosf(theta);
            tab[((size_t)pos * half + i) * 2 + 1] = sinf(theta);
        }
    }
}

int qcheck_cfg(const brrr_qwen_cfg &c) {
    if (c.n_embd <= 0 || c.n_embd % 256 || c.n_embd > 8192) return BRRR_ERR_ARG;
    if (c.head_dim != 128) return BRRR_ERR_ARG;                 // attention and rope kernels are written for 128
    if (c.n_head <= 0 || c.n_head_kv <= 0 || c.n_head % c.n_head_kv || (c.n_head * c.head_dim) % 256) return BRRR_ERR_ARG;
    if (c.n_ff_exp <= 0 || c.n_ff_exp % 256) return BRRR_ERR_ARG;
    if (c.n_expert <= 0 || c.n_expert > 256 || c.n_expert_used <= 0 || c.n_expert_used > 8 || c.n_expert_used > c.n_expert) return BRRR_ERR_ARG;
    if (c.n_layer <= 0 || c.n_vocab <= 0) return BRRR_ERR_ARG;
    return BRRR_OK;
}

// The decode step (forward_worker, engine_qwen2.rs:302-451), kernel by kernel.
int qenqueue_step(brrr_qwen *m, bool want, float *trace_dev, int *nlaunch) {
    const brrr_qwen_cfg &c = m->cfg;
    const int d = c.n_embd, nh = c.n_head, nkv = c.n_head_kv, hd = c.head_dim, ff = c.n_ff_exp, topk = c.n_expert_used;
    cudaStream_t s = m->stream;
    const bool pdl = m->use_pdl && !trace_dev;
    int n = 0;
    CU(launch_qw_embed(m->embd.p, d, m->st, m->x, false, s)); n++;
    if (trace_dev) CU(cudaMemcpyAsync(trace_dev, m->x, d * sizeof(float), cudaMemcpyDeviceToDevice, s));
    // layer 0 has no down kernel before it: its attention norm + Q8_K is a launch of its own
    CU(launch_qw_norm_quant(m->x, m->L[0].attn_norm, c.rms_eps, d, nullptr, m->xq, m->xs, m->xsum, pdl, s)); n++;
    for (int il = 0; il < c.n_layer; il++) {
        QLayer &ly = m->L[il];
        KMatDev qkv[3] = {ly.wq, ly.wk, ly.wv};
        float *qkv_out[3] = {m->q, m->k, m->v};
        CU(launch_qw_matvec(qkv, qkv_out, 3, false, m->xq, m->xs, m->xsum, pdl, s, ly.kc, ly.vc, nkv, m->st)); n++;
        CU(launch_qw_qknorm_rope(m->q, m->k, m->v, ly.q_norm, ly.k_norm, m->rope, c.rms_eps, nh, nkv, m->st, 0, ly.kc, ly.vc, pdl, s)); n++;
        CU(launch_qw_attn(m->q, ly.kc, ly.vc, nh, nkv, m->st, 0, m->aq, m->as, m->asum, pdl, s)); n++;
        float *xo[1] = {m->x};
        CU(launch_qw_matvec(&ly.wo, xo, 1, true, m->aq, m->as, m->asum, pdl, s)); n++;
        // router: FFN norm (12 slices) and the Q8_K image of the normalised token in its prologue
        CU(launch_ffn_in(m->x, ly.ffn_norm, c.rms_eps, d, ly.ginp, nullptr, c.n_expert, topk, m->rlogits, m->top, m->wts, &m->st->router_done, m->st,
                         pdl, s, 1, nullptr, 1, m->xq, m->xs, m->xsum)); n++;
        CU(launch_qw_gate_up(ly.gate, ly.up, m->top, topk, ff, m->xq, m->xs, m->xsum, m->hbuf, pdl, s)); n++;
        const bool last = il == c.n_layer - 1;
        const float *nw = last ? (want ? m->out_norm : nullptr) : m->L[il + 1].attn_norm;
        CU(launch_qw_down(ly.down, m->top, m->wts, topk, d, ff, m->hbuf, m->x, m->down_counter, nw, c.rms_eps, m->xq, m->xs, m->xsum, pdl, s)); n++;
        if (trace_dev) CU(cudaMemcpyAsync(trace_dev + (size_t)(il + 1) * d, m->x, d * sizeof(float), cudaMemcpyDeviceToDevice, s));
    }
    if (want) {
        CU(launch_qw_head(m->head, m->xq, m->xs, m->xsum, m->logits, m->st, pdl, s)); n++;
        launch_finish_token(m->st, s); n++;
    }
    CU(cudaGetLastError());
    if (nlaunch) *nlaunch = n;
    return BRRR_OK;
}

int qcapture(brrr_qwen *m, bool want, cudaGraphExec_t *out, int *nlaunch) {
    cudaGraph_t g = nullptr;
    CU(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
    int s = qenqueue_step(m, want, nullptr, nlaunch);
    cudaError_t e = cudaStreamEndCapture(m->stream, &g);
    if (s != BRRR_OK) { if (g) cudaGraphDestroy(g); return s; }
    CU(e);
    CU(cudaGraphInstantiate(out, g, 0));
    CU(cudaGraphDestroy(g));
    return BRRR_OK;
}

int qbuild(brrr_qwen *m, const QSource &src) {
    const brrr_qwen_cfg &c = m->cfg;
    const int d = c.n_embd, nh = c.n_head, nkv = c.n_head_kv, hd = c.head_dim, ne = c.n_expert, ff = c.n_ff_exp, topk = c.n_expert_used;
    CU(cudaSetDevice(m->device));
    CU(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
    if (const char *e = getenv("BRRR_NOPDL")) m->use_pdl = !(e[0] && e[0] != '0');
    float *scratch = nullptr;
    if (cudaMalloc(&scratch, (size_t)ne * d * 4) != cudaSuccess) return BRRR_ERR_NOMEM;
    struct Guard { void *p; ~Guard() { cudaFree(p); } } guard{scratch};

    m->L.resize(c.n_layer);
    for (int il = 0; il < c.n_layer; il++) {
        QLayer &ly = m->L[il];
        TRY(qload_f32(m, src, il, BRRR_T_ATTN_NORM, d, &ly.attn_norm));
        TRY(qload_f32(m, src, il, BRRR_T_FFN_NORM, d, &ly.ffn_norm));
        TRY(qload_f32(m, src, il, BRRR_T_Q_NORM, hd, &ly.q_norm));
        TRY(qload_f32(m, src, il, BRRR_T_K_NORM, hd, &ly.k_norm));
        TRY(qload_k(m, src, il, BRRR_T_WQ, nh * hd, d, &ly.wq));
        TRY(qload_k(m, src, il, BRRR_T_WK, nkv * hd, d, &ly.wk));
        TRY(qload_k(m, src, il, BRRR_T_WV, nkv * hd, d, &ly.wv));
        TRY(qload_k(m, src, il, BRRR_T_WO, d, nh * hd, &ly.wo));
        // router: raw f32 [ne][d] -> the tiled layout of the router kernel
        float *raw = nullptr;
        if (src.synth) {
            launch_synth(src.seed, il, BRRR_T_ROUTER_W, 0, (size_t)ne * d, scratch, m->stream);
            CU(cudaGetLastError());
            raw = scratch;
        } else {
            auto it = src.idx.find("blk." + std::to_string(il) + ".ffn_gate_inp.weight");
            if (it == src.idx.end() || it->second.type != 0 || it->second.nel != (size_t)ne * d || it->second.off + (size_t)ne * d * 4 > src.blob_len) {
                QERR("blk.%d.ffn_gate_inp.weight missing or malformed", il);
                return BRRR_ERR_IO;
            }
            CU(cudaMemcpyAsync(scratch, src.blob + it->second.off, (size_t)ne * d * 4, cudaMemcpyHostToDevice, m->stream));
            CU(cudaStreamSynchronize(m->stream));
            raw = scratch;
        }
        TRY(m->alloc(&ly.ginp, router_packed_floats(ne, d)));
        launch_router_pack(raw, ne, d, ly.ginp, m->stream);
        CU(cudaGetLastError());
        TRY(qload_k(m, src, il, BRRR_T_GATE, ne * ff, d, &ly.gate));
        TRY(qload_k(m, src, il, BRRR_T_UP, ne * ff, d, &ly.up));
        TRY(qload_k(m, src, il, BRRR_T_DOWN, ne * d, ff, &ly.down));
        TRY(m->alloc(&ly.kc, (size_t)BRRR_MAXSEQ * nkv * hd));
        TRY(m->alloc(&ly.vc, (size_t)BRRR_MAXSEQ * nkv * hd));
        CU(cudaMemsetAsync(ly.kc, 0, (size_t)BRRR_MAXSEQ * nkv * hd * 4, m->stream));
        CU(cudaMemsetAsync(ly.vc, 0, (size_t)BRRR_MAXSEQ * nkv * hd * 4, m->stream));
    }
    TRY(qload_k(m, src, BRRR_L_GLOBAL, BRRR_T_TOK_EMBD, c.n_vocab, d, &m->embd));
    if (m->embd.type != 12) { QERR("token_embd.weight must be Q4_K"); return BRRR_ERR_IO; }   // engine_qwen2.rs:311
    TRY(qload_f32(m, src, BRRR_L_GLOBAL, BRRR_T_OUT_NORM, d, &m->out_norm));
    TRY(qload_k(m, src, BRRR_L_GLOBAL, BRRR_T_OUTPUT, c.n_vocab, d, &m->head));

    std::vector<float> tab((size_t)BRRR_MAXSEQ * hd);
    qrope_table_host(c, tab.data());
    TRY(m->alloc(&m->rope, tab.size()));
    CU(cudaMemcpyAsync(m->rope, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, m->stream));

    TRY(m->alloc(&m->x, d)); TRY(m->alloc(&m->xn, d)); TRY(m->alloc(&m->q, nh * hd)); TRY(m->alloc(&m->k, nkv * hd)); TRY(m->alloc(&m->v, nkv * hd));
    TRY(m->alloc(&m->ao, nh * hd)); TRY(m->alloc(&m->hbuf, (size_t)topk * ff)); TRY(m->alloc(&m->rlogits, ne)); TRY(m->alloc(&m->logits, c.n_vocab));
    TRY(m->alloc(&m->xs, d / 256)); TRY(m->alloc(&m->as, nh * hd / 256)); TRY(m->alloc(&m->hs, (size_t)topk * ff / 256)); TRY(m->alloc(&m->wts, 8));
    TRY(m->alloc(&m->xq, d)); TRY(m->alloc(&m->aq, nh * hd)); TRY(m->alloc(&m->hq, (size_t)topk * ff));
    TRY(m->alloc(&m->xsum, d / 32)); TRY(m->alloc(&m->asum, nh * hd / 32)); TRY(m->alloc(&m->hsum, (size_t)topk * ff / 32));
    TRY(m->alloc(&m->top, 8)); TRY(m->alloc(&m->st, 1));
    TRY(m->alloc(&m->down_counter, 1));
    CU(cudaMemsetAsync(m->down_counter, 0, sizeof(unsigned int), m->stream));
    CU(cudaMemsetAsync(m->st, 0, sizeof(DevState), m->stream));
    CU(cudaMemsetAsync(m->x, 0, d * 4, m->stream));
    CU(cudaMallocHost(&m->h_in, 16));
    CU(cudaMallocHost(&m->h_out, BRRR_MAXSEQ * sizeof(uint32_t)));
    CU(cudaStreamSynchronize(m->stream));
    // one direct (un-captured) step configures kernel attributes and validates the launches
    TRY(qenqueue_step(m, true, nullptr, nullptr));
    CU(cudaStreamSynchronize(m->stream));
    CU(cudaMemsetAsync(m->st, 0, sizeof(DevState), m->stream));
    TRY(qcapture(m, true, &m->g_head, &m->launches_head));
    TRY(qcapture(m, false, &m->g_nohead, &m->launches_nohead));
    CU(cudaStreamSynchronize(m->stream));
    return BRRR_OK;
}

int qparse_dir(const char *dir, brrr_qwen_cfg *c, QSource *src) {
    std::string p = std::string(dir) + "/config.txt";
    FILE *f = fopen(p.c_str(), "r");
    if (!f) { QERR("cannot open %s", p.c_str()); return BRRR_ERR_IO; }
    char line[512], key[128], val[128];
    std::map<std::string, std::string> kv;
    while (fgets(line, sizeof line, f))
        if (sscanf(line, "%127s %127s", key, val) == 2) kv[key] = val;
    fclose(f);
    const char *need[] = {"n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "n_expert", "n_expert_used", "n_ff_exp", "n_vocab",
                          "rope_freq_base", "rms_eps"};
    for (const char *k : need)
        if (!kv.count(k)) { QERR("config missing %s", k); return BRRR_ERR_IO; }
    memset(c, 0, sizeof *c);
    c->n_embd = atoi(kv["n_embd"].c_str()); c->n_layer = atoi(kv["n_layer"].c_str());
    c->n_head = atoi(kv["n_head"].c_str()); c->n_head_kv = atoi(kv["n_head_kv"].c_str());
    c->head_dim = atoi(kv["head_dim"].c_str()); c->n_expert = atoi(kv["n_expert"].c_str());
    c->n_expert_used = atoi(kv["n_expert_used"].c_str()); c->n_ff_exp = atoi(kv["n_ff_exp"].c_str());
    c->n_vocab = atoi(kv["n_vocab"].c_str());
    c->rope_freq_base = strtof(kv["rope_freq_base"].c_str(), nullptr);
    c->rms_eps = strtof(kv["rms_eps"].c_str(), nullptr);
    p = std::string(dir) + "/manifest.txt";
    f = fopen(p.c_str(), "r");
    if (!f) { QERR("cannot open %s", p.c_str()); return BRRR_ERR_IO; }
    size_t data_start = 0;
    if (fscanf(f, "%127s %zu", key, &data_start) != 2 || strcmp(key, "data_start")) { fclose(f); QERR("bad manifest header"); return BRRR_ERR_IO; }
    char nm[256]; unsigned ty; size_t off, nel;
    while (fscanf(f, "%255s %u %zu %zu", nm, &ty, &off, &nel) == 4) src->idx[nm] = QSource::Ent{ty, data_start + off, nel};
    fclose(f);
    return BRRR_OK;
}

}  // namespace

extern "C" void brrr_qwen_close(brrr_qwen *m) {
    if (!m) return;
    cudaSetDevice(m->device);
    if (m->stream) cudaStreamSynchronize(m->stream);
    if (m->g_head) cudaGraphExecDestroy(m->g_head);
    if (m->g_nohead) cudaGraphExecDestroy(m->g_nohead);
    for (void *p : m->allocs) cudaFree(p);
    if (m->h_in) cudaFreeHost(m->h_in);
    if (m->h_out) cudaFreeHost(m->h_out);
    if (m->stream) cudaStreamDestroy(m->stream);
    delete m;
}

extern "C" int brrr_qwen_open(const char *data_dir, const char *blob_path, int device, brrr_qwen **out) {
    if (!data_dir || !blob_path || !out) return BRRR_ERR_ARG;
    *out = nullptr;
    brrr_qwen *m = new brrr_qwen();
    m->device = device;
    QSource src;
    int s = qparse_dir(data_dir, &m->cfg, &src);
    if (s == BRRR_OK) s = qcheck_cfg(m->cfg);
    void *map = MAP_FAILED;
    if (s == BRRR_OK) {
        int fd = open(blob_path, O_RDONLY);
        struct stat stt;
        if (fd < 0 || fstat(fd, &stt) != 0) { QERR("cannot open blob %s", blob_path); s = BRRR_ERR_IO; }
        else {
            src.blob_len = stt.st_size;
            map = mmap(nullptr, src.blob_len, PROT_READ, MAP_PRIVATE, fd, 0);
            if (map == MAP_FAILED) { QERR("mmap of %s failed", blob_path); s = BRRR_ERR_IO; }
            src.blob = (const uint8_t *)map;
        }
        if (fd >= 0) close(fd);
    }
    if (s == BRRR_OK) s = qbuild(m, src);
    if (map != MAP_FAILED) munmap(map, src.blob_len);
    if (s != BRRR_OK) { brrr_qwen_close(m); return s; }
    *out = m;
    return BRRR_OK;
}

extern "C" int brrr_qwen_open_synth(const brrr_qwen_cfg *cfg, uint64_t seed, int device, brrr_qwen **out) {
    if (!cfg || !out) return BRRR_ERR_ARG;
    *out = nullptr;
    int s = qcheck_cfg(*cfg);
    if (s != BRRR_OK) return s;
    brrr_qwen *m = new brrr_qwen();
    m->cfg = *cfg;
    m->device = device;
    QSource src;
    src.synth = true; src.seed = seed;
    s = qbuild(m, src);
    if (s != BRRR_OK) { brrr_qwen_close(m); return s; }
    *out = m;
    return BRRR_OK;
}

extern "C" int brrr_qwen_cfg_get(const brrr_qwen *m, brrr_qwen_cfg *out) {
    if (!m || !out) return BRRR_ERR_ARG;
    *out = m->cfg;
    return BRRR_OK;
}

extern "C" int brrr_qwen_launches_per_step(const brrr_qwen *m, int want) { return m ? (want ? m->launches_head : m->launches_nohead) : 0; }

// Algorithmic bytes one decode step at position pos must read: the K-quant rows it touches, the
// router, the norms, K and V of positions 0..pos, the embedding row.
extern "C" uint64_t brrr_qwen_bytes_per_step(const brrr_qwen *m, uint32_t pos) {
    if (!m) return 0;
    const brrr_qwen_cfg &c = m->cfg;
    const uint64_t d = c.n_embd, nkv = c.n_head_kv, hd = c.head_dim, ne = c.n_expert, k = c.n_expert_used, ff = c.n_ff_exp;
    auto rb = [](const KMatDev &w) { return (uint64_t)kq_gguf_row_bytes(w.type, w.cols); };      // GGUF density, whatever the device layout
    uint64_t total = 0;
    for (const QLayer &ly : m->L) {
        total += (uint64_t)ly.wq.rows * rb(ly.wq) + (uint64_t)ly.wk.rows * rb(ly.wk) + (uint64_t)ly.wv.rows * rb(ly.wv) + (uint64_t)ly.wo.rows * rb(ly.wo);
        total += k * ff * (rb(ly.gate) + rb(ly.up)) + k * d * rb(ly.down);
        total += ne * d * 4 + 2 * d * 4 + 2 * hd * 4;
        total += ((uint64_t)pos + 1) * nkv * hd * 4 * 2;
    }
    total += (uint64_t)m->head.rows * rb(m->head) + d * 4 + rb(m->embd);
    return total;
}

static int qrun_graph(brrr_qwen *m, bool want) {
    CU(cudaGraphLaunch(want ? m->g_head : m->g_nohead, m->stream));
    return BRRR_OK;
}

extern "C" int brrr_qwen_forward(brrr_qwen *m, uint32_t tok, uint32_t pos, int want, uint32_t *out_tok) {
    if (!m) return BRRR_ERR_ARG;
    if (tok >= (uint32_t)m->cfg.n_vocab || pos >= BRRR_MAXSEQ) return BRRR_ERR_RANGE;
    CU(cudaSetDevice(m->device));
    m->h_in[0] = tok; m->h_in[1] = pos;
    CU(cudaMemcpyAsync(m->st, m->h_in, 8, cudaMemcpyHostToDevice, m->stream));   // DevState.tok, .pos
    TRY(qrun_graph(m, want != 0));
    CU(cudaMemcpyAsync(m->h_out, m->st, 32, cudaMemcpyDeviceToHost, m->stream));
    CU(cudaStreamSynchronize(m->stream));
    if (m->h_out[6] != 0) { QERR("device wait timed out (code %u)", m->h_out[6]); return BRRR_ERR_STATE; }
    if (want && out_tok) *out_tok = m->h_out[0];
    return BRRR_OK;
}

extern "C" int brrr_qwen_decode_enqueue(brrr_qwen *m, uint32_t first_tok, uint32_t pos, uint32_t n) {
    if (!m) return BRRR_ERR_ARG;
    if (first_tok >= (uint32_t)m->cfg.n_vocab || n == 0 || n > BRRR_MAXSEQ || pos + n > BRRR_MAXSEQ) return BRRR_ERR_RANGE;
    CU(cudaSetDevice(m->device));
    m->h_in[0] = first_tok; m->h_in[1] = pos; m->h_in[2] = 0;
    CU(cudaMemcpyAsync(m->st, m->h_in, 12, cudaMemcpyHostToDevice, m->stream));  // tok, pos, n_out = 0
    for (uint32_t i = 0; i < n; i++) TRY(qrun_graph(m, true));
    return BRRR_OK;
}

extern "C" int brrr_qwen_decode_wait(brrr_qwen *m, uint32_t n, uint32_t *out_toks) {
    if (!m || !out_toks || n == 0 || n > BRRR_MAXSEQ) return BRRR_ERR_ARG;
    CU(cudaSetDevice(m->device));
    CU(cudaMemcpyAsync(m->h_out, m->st->out, n * sizeof(uint32_t), cudaMemcpyDeviceToHost, m->stream));
    CU(cudaMemcpyAsync(m->h_in, &m->st->err, 4, cudaMemcpyDeviceToHost, m->stream));
    CU(cudaStreamSynchronize(m->stream));
    if (m->h_in[0] != 0) { QERR("device wait timed out (code %u)", m->h_in[0]); return BRRR_ERR_STATE; }
    memcpy(out_toks, m->h_out, n * sizeof(uint32_t));
    return BRRR_OK;
}

extern "C" int brrr_qwen_decode(brrr_qwen *m, uint32_t first_tok, uint32_t pos, uint32_t n, uint32_t *out_toks) {
    if (!out_toks) return BRRR_ERR_ARG;
    int s = brrr_qwen_decode_enqueue(m, first_tok, pos, n);
    if (s != BRRR_OK) return s;
    return brrr_qwen_decode_wait(m, n, out_toks);
}

extern "C" int brrr_qwen_logits(brrr_qwen *m, float *out) {
    if (!m || !out) return BRRR_ERR_ARG;
    CU(cudaSetDevice(m->device));
    CU(cudaMemcpyAsync(out, m->logits, (size_t)m->cfg.n_vocab * 4, cudaMemcpyDeviceToHost, m->stream));
    CU(cudaStreamSynchronize(m->stream));
    return BRRR_OK;
}

extern "C" int brrr_qwen_hidden(brrr_qwen *m, float *out) {
    if (!m || !out) return BRRR_ERR_ARG;
    CU(cudaSetDevice(m->device));
    CU(cudaMemcpyAsync(out, m->x, (size_t)m->cfg.n_embd * 4, cudaMemcpyDeviceToHost, m->stream));
    CU(cudaStreamSynchronize(m->stream));
    return BRRR_OK;
}

extern "C" int brrr_qwen_forward_trace(brrr_qwen *m, uint32_t tok, uint32_t pos, float *trace) {
    if (!m || !trace) return BRRR_ERR_ARG;
    if (tok >= (uint32_t)m->cfg.n_vocab || pos >= BRRR_MAXSEQ) return BRRR_ERR_RANGE;
    CU(cudaSetDevice(m->device));
    size_t n = (size_t)(m->cfg.n_layer + 1) * m->cfg.n_embd;
    float *dev = nullptr;
    CU(cudaMalloc(&dev, n * 4));
    m->h_in[0] = tok; m->h_in[1] = pos;
    cudaMemcpyAsync(m->st, m->h_in, 8, cudaMemcpyHostToDevice, m->stream);
    int s = qenqueue_step(m, true, dev, nullptr);
    if (s == BRRR_OK && cudaMemcpyAsync(trace, dev, n * 4, cudaMemcpyDeviceToHost, m->stream) != cudaSuccess) s = BRRR_ERR_CUDA;
    if (cudaStreamSynchronize(m->stream) != cudaSuccess) s = BRRR_ERR_CUDA;
    cudaFree(dev);
    return s;
}

extern "C" void *brrr_qwen_stream(brrr_qwen *m) { return m ? (void *)m->stream : nullptr; }
