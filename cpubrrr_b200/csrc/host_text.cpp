// Host text layer of the gpt-oss engine: tokenizer (tokens.bin, greedy longest match), the
// temperature / top-k sampler, the harmony chat prompt, generate() and the line-oriented serve
// loop.  It mirrors the part of the reference's host program that surrounds the forward pass
// (src/bin/engine_gpt2.rs): tokenizer 1261-1274, sample_logits 82-126, generate 1400-1440, the
// --serve protocol 1442-1488.  Pure host code; the forward pass goes through brrr_forward /
// brrr_decode.
#include "../../include/brrr.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <chrono>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

// exp as the engine defines it (same fixed IEEE sequence as the device code and the oracle), so a
// sampled sequence does not depend on the host's libm.
float host_expf(float x) {
    if (x != x) return x + x;
    if (x > 88.72283935546875f) return INFINITY;
    if (x < -104.0f) return 0.0f;
    float kf = rintf(x * 1.44269504088896341f);
    float r = fmaf(kf, -0.693145751953125f, x);
    r = fmaf(kf, -1.42860682030941723212e-6f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float r2 = r * r;
    float y = fmaf(p, r2, r);
    y = y + 1.0f;
    int k = (int)kf, k1 = k >> 1, k2 = k - k1;
    uint32_t b1 = (uint32_t)(k1 + 127) << 23, b2 = (uint32_t)(k2 + 127) << 23;
    float s1, s2;
    memcpy(&s1, &b1, 4);
    memcpy(&s2, &b2, 4);
    return (y * s1) * s2;
}

}  // namespace

struct brrr_tokenizer {
    std::vector<std::string> toks;                       // id -> bytes
    std::unordered_map<std::string, uint32_t> lookup;    // ordinary tokens, first id wins
    std::unordered_map<std::string, uint32_t> special;   // tokens spelled "<|...", by text
};

// tokens.bin: u32 count, then per token u16 length + bytes (scripts/dump_tokenizer.py:59-64).
extern "C" int brrr_tokenizer_open(const char *data_dir, brrr_tokenizer **out) {
    if (!data_dir || !out) return BRRR_ERR_ARG;
    *out = nullptr;
    std::string path = std::string(data_dir) + "/tokens.bin";
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return BRRR_ERR_IO;
    uint32_t n = 0;
    if (fread(&n, 4, 1, f) != 1 || n > (1u << 24)) { fclose(f); return BRRR_ERR_IO; }
    brrr_tokenizer *t = new brrr_tokenizer();
    t->toks.resize(n);
    for (uint32_t i = 0; i < n; i++) {
        uint16_t len = 0;
        if (fread(&len, 2, 1, f) != 1) { fclose(f); delete t; return BRRR_ERR_IO; }
        t->toks[i].resize(len);
        if (len && fread(&t->toks[i][0], 1, len, f) != len) { fclose(f); delete t; return BRRR_ERR_IO; }
    }
    fclose(f);
    for (uint32_t i = 0; i < n; i++) {
        const std::string &s = t->toks[i];
        if (s.empty()) continue;
        if (s.compare(0, 2, "<|") == 0) t->special.emplace(s, i);     // engine_qwen2.rs:499
        else t->lookup.emplace(s, i);                                 // or_insert: the first id wins (engine_gpt2.rs:1268)
    }
    *out = t;
    return BRRR_OK;
}

extern "C" void brrr_tokenizer_close(brrr_tokenizer *t) { delete t; }
extern "C" uint32_t brrr_tokenizer_size(const brrr_tokenizer *t) { return t ? (uint32_t)t->toks.size() : 0; }

extern "C" int brrr_tokenizer_token(const brrr_tokenizer *t, uint32_t id, const char **bytes, uint32_t *len) {
    if (!t || !bytes || !len || id >= t->toks.size()) return BRRR_ERR_RANGE;
    *bytes = t->toks[id].data();
    *len = (uint32_t)t->toks[id].size();
    return BRRR_OK;
}

extern "C" int brrr_tokenizer_special(const brrr_tokenizer *t, const char *text, uint32_t *id) {
    if (!t || !text || !id) return BRRR_ERR_ARG;
    auto it = t->special.find(text);
    if (it == t->special.end()) return BRRR_ERR_RANGE;
    *id = it->second;
    return BRRR_OK;
}

// Greedy longest match, at most max_piece bytes per token (32 in engine_gpt2.rs:1270, 48 in
// engine_qwen2.rs:503).  A byte no token covers is BRRR_ERR_RANGE (the reference asserts).
extern "C" int brrr_tokenizer_encode(const brrr_tokenizer *t, const char *text, size_t len, uint32_t max_piece, uint32_t *out, size_t cap,
                                     size_t *n_out) {
    if (!t || (!text && len) || !n_out || max_piece == 0) return BRRR_ERR_ARG;
    size_t n = 0, i = 0;
    std::string key;
    while (i < len) {
        size_t l = len - i < max_piece ? len - i : max_piece;
        for (;; l--) {
            if (l == 0) return BRRR_ERR_RANGE;
            key.assign(text + i, l);
            auto it = t->lookup.find(key);
            if (it != t->lookup.end()) {
                if (out && n < cap) out[n] = it->second;
                n++;
                i += l;
                break;
            }
        }
    }
    *n_out = n;
    return (out && n > cap) ? BRRR_ERR_RANGE : BRRR_OK;
}

// ---------------------------------------------------------------- sampler (engine_gpt2.rs:82-126)
extern "C" uint64_t brrr_rng_seed(uint64_t seed) {          // splitmix64 scramble, never zero (engine_gpt2.rs:1462-1466)
    uint64_t z = seed + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return (z ^ (z >> 31)) | 1ull;
}

static uint64_t rng_next(uint64_t *state) {                 // xorshift64 (engine_gpt2.rs:87-92)
    uint64_t x = *state;
    x ^= x << 13; x ^= x >> 7; x ^= x << 17;
    *state = x;
    return x;
}

extern "C" uint32_t brrr_sample_logits(const float *logits, uint32_t n, uint32_t temp_milli, uint32_t top_k, uint64_t *rng_state) {
    if (!logits || n == 0) return 0;
    if (temp_milli == 0 || !rng_state) {                    // greedy: first strict maximum
        float best = -3.402823466e+38f;
        uint32_t bi = 0;
        for (uint32_t i = 0; i < n; i++) if (logits[i] > best) { best = logits[i]; bi = i; }
        return bi;
    }
    const float temp = (float)temp_milli / 1000.0f;
    size_t k = top_k < 1 ? 1 : (top_k > 64 ? 64 : top_k);
    std::vector<std::pair<float, uint32_t>> top;
    top.reserve(k + 1);
    for (uint32_t i = 0; i < n; i++) {
        float l = logits[i];
        if (top.size() < k || l > top.back().first) {
            size_t pos = 0;                                 // partition_point(|v| v > l)
            while (pos < top.size() && top[pos].first > l) pos++;
            top.insert(top.begin() + pos, std::make_pair(l, i));
            if (top.size() > k) top.pop_back();
        }
    }
    const float mx = top[0].first;
    std::vector<float> probs(top.size());
    float sum = 0.0f;
    for (size_t i = 0; i < top.size(); i++) { probs[i] = host_expf((top[i].first - mx) / temp); sum += probs[i]; }
    for (float &p : probs) p /= sum;
    const float r = (float)(rng_next(rng_state) >> 11) / (float)(1ull << 53);
    float acc = 0.0f;
    for (size_t i = 0; i < top.size(); i++) {
        acc += probs[i];
        if (r <= acc) return top[i].second;
    }
    return top.back().second;
}

// ---------------------------------------------------------------- chat prompt (engine_gpt2.rs:1401-1414)
static const char *kSystem =
    "You are ChatGPT, a large language model trained by OpenAI.\nKnowledge cutoff: 2024-06\nCurrent date: 2026-07-03\n\nReasoning: low\n\n"
    "# Valid channels: analysis, commentary, final. Channel must be included for every message.";
enum { TOK_START = 200006, TOK_END = 200007, TOK_MESSAGE = 200008, TOK_RETURN = 200002, TOK_EOT = 199999 };

extern "C" int brrr_chat_prompt(const brrr_tokenizer *t, const char *user_text, uint32_t *out, size_t cap, size_t *n_out) {
    if (!t || !user_text || !n_out) return BRRR_ERR_ARG;
    std::vector<uint32_t> ids;
    auto enc = [&](const char *s) -> int {
        size_t n = 0, l = strlen(s);
        int st = brrr_tokenizer_encode(t, s, l, 32, nullptr, 0, &n);
        if (st != BRRR_OK) return st;
        size_t at = ids.size();
        ids.resize(at + n);
        return brrr_tokenizer_encode(t, s, l, 32, ids.data() + at, n, &n);
    };
    int st;
    ids.push_back(TOK_START);
    if ((st = enc("system")) != BRRR_OK) return st;
    ids.push_back(TOK_MESSAGE);
    if ((st = enc(kSystem)) != BRRR_OK) return st;
    ids.push_back(TOK_END);
    ids.push_back(TOK_START);
    if ((st = enc("user")) != BRRR_OK) return st;
    ids.push_back(TOK_MESSAGE);
    if ((st = enc(user_text)) != BRRR_OK) return st;
    ids.push_back(TOK_END);
    ids.push_back(TOK_START);
    if ((st = enc("assistant")) != BRRR_OK) return st;
    *n_out = ids.size();
    if (out) {
        if (ids.size() > cap) return BRRR_ERR_RANGE;
        memcpy(out, ids.data(), ids.size() * 4);
    }
    return BRRR_OK;
}

// ---------------------------------------------------------------- generate (engine_gpt2.rs:1400-1440)
// Prefill the ids, then decode until a stop token (200002, 199999), ngen tokens or the context
// limit.  Greedy decoding runs on the device in bursts (brrr_decode) and is cut at the first stop
// token; with a temperature every step fetches the logits and samples on the host like the
// reference.  emit (nullable) receives the bytes of every produced token.
extern "C" int brrr_generate(brrr_model *m, const brrr_tokenizer *t, const uint32_t *ids, size_t n_ids, uint32_t ngen, uint32_t temp_milli,
                             uint32_t top_k, uint64_t *rng_state, void (*emit)(const char *, uint32_t, void *), void *emit_arg,
                             uint32_t *out_ids, size_t out_cap, brrr_gen_stats *stats) {
    if (!m || !ids || n_ids == 0) return BRRR_ERR_ARG;
    brrr_cfg cfg;
    int st = brrr_model_cfg(m, &cfg);
    if (st != BRRR_OK) return st;
    if (n_ids >= BRRR_MAXSEQ) return BRRR_ERR_RANGE;
    const bool greedy = temp_milli == 0 || !rng_state;
    std::vector<float> logits(greedy ? 0 : (size_t)cfg.n_vocab);
    auto t0 = std::chrono::steady_clock::now();
    uint32_t next = 0;
    st = brrr_forward_tile(m, ids, (uint32_t)n_ids, 0, 1, &next);
    if (st != BRRR_OK) return st;
    if (!greedy) {
        if ((st = brrr_logits(m, logits.data())) != BRRR_OK) return st;
        next = brrr_sample_logits(logits.data(), (uint32_t)cfg.n_vocab, temp_milli, top_k, rng_state);
    }
    auto t1 = std::chrono::steady_clock::now();
    size_t pos = n_ids;
    uint32_t n = 0;
    auto put = [&](uint32_t tok) {
        if (out_ids && n < out_cap) out_ids[n] = tok;
        if (emit && t) {
            const char *b; uint32_t l;
            if (brrr_tokenizer_token(t, tok, &b, &l) == BRRR_OK) emit(b, l, emit_arg);
        }
        n++;
    };
    auto stop = [&](uint32_t tok) { return tok == TOK_RETURN || tok == TOK_EOT; };
    if (greedy) {
        std::vector<uint32_t> burst(32);
        while (n < ngen && !stop(next) && pos + 1 < BRRR_MAXSEQ) {
            uint32_t want = ngen - n < 32 ? ngen - n : 32;
            if (pos + want >= BRRR_MAXSEQ) want = (uint32_t)(BRRR_MAXSEQ - 1 - pos);
            if (want == 0) break;
            // burst[i] = token produced by feeding the chain's token i at position pos + i
            if ((st = brrr_decode(m, next, (uint32_t)pos, want, burst.data())) != BRRR_OK) return st;
            for (uint32_t used = 0; used < want; used++) {
                put(next);                                   // the token that was fed is the one shown
                pos++;
                next = burst[used];
                if (n >= ngen || stop(next) || pos + 1 >= BRRR_MAXSEQ) break;   // steps the device ran beyond this one are discarded
            }
        }
    } else {
        while (n < ngen && !stop(next) && pos + 1 < BRRR_MAXSEQ) {
            put(next);
            uint32_t dummy = 0;
            if ((st = brrr_forward(m, next, (uint32_t)pos, 1, &dummy)) != BRRR_OK) return st;
            if ((st = brrr_logits(m, logits.data())) != BRRR_OK) return st;
            next = brrr_sample_logits(logits.data(), (uint32_t)cfg.n_vocab, temp_milli, top_k, rng_state);
            pos++;
        }
    }
    auto t2 = std::chrono::steady_clock::now();
    if (stats) {
        stats->prefill_tokens = (uint32_t)n_ids;
        stats->decode_tokens = n;
        stats->prefill_seconds = std::chrono::duration<double>(t1 - t0).count();
        stats->decode_seconds = std::chrono::duration<double>(t2 - t1).count();
    }
    return BRRR_OK;
}

// ---------------------------------------------------------------- serve protocol (engine_gpt2.rs:1442-1488)
// One request line: either a bare prompt, or TSV `temp \t seed \t ngen \t prompt` with \n, \t and
// \\ backslash-escaped in the prompt.  Returns 1 for the TSV form, 0 for a bare prompt.
extern "C" int brrr_serve_parse(const char *line, float *temp, uint64_t *seed, uint32_t *ngen, char *prompt, size_t prompt_cap) {
    if (!line || !prompt || prompt_cap == 0) return -1;
    std::string s(line);
    while (!s.empty() && (s.back() == '\n' || s.back() == '\r' || s.back() == ' ' || s.back() == '\t')) s.pop_back();
    size_t b = 0;
    while (b < s.size() && (s[b] == ' ' || s[b] == '\t' || s[b] == '\n' || s[b] == '\r')) b++;
    s = s.substr(b);
    auto bare = [&]() { snprintf(prompt, prompt_cap, "%s", s.c_str()); return 0; };
    size_t p1 = s.find('\t');
    if (p1 == std::string::npos) return bare();
    size_t p2 = s.find('\t', p1 + 1);
    if (p2 == std::string::npos) return bare();
    size_t p3 = s.find('\t', p2 + 1);
    if (p3 == std::string::npos) return bare();
    std::string f0 = s.substr(0, p1), f1 = s.substr(p1 + 1, p2 - p1 - 1), f2 = s.substr(p2 + 1, p3 - p2 - 1), f3 = s.substr(p3 + 1);
    char *end = nullptr;
    float tv = strtof(f0.c_str(), &end);
    if (f0.empty() || *end) return bare();
    unsigned long long sv = strtoull(f1.c_str(), &end, 10);
    if (f1.empty() || *end || f1[0] == '-') return bare();
    unsigned long long nv = strtoull(f2.c_str(), &end, 10);
    if (f2.empty() || *end || f2[0] == '-') return bare();
    std::string un;
    for (size_t i = 0; i < f3.size(); i++) {
        if (f3[i] == '\\') {
            if (i + 1 < f3.size()) {
                char o = f3[++i];
                if (o == 'n') un.push_back('\n');
                else if (o == 't') un.push_back('\t');
                else if (o == '\\') un.push_back('\\');
                else { un.push_back('\\'); un.push_back(o); }
            } else un.push_back('\\');
        } else un.push_back(f3[i]);
    }
    if (temp) *temp = tv < 0.0f ? 0.0f : tv;
    if (seed) *seed = sv;
    if (ngen) *ngen = (uint32_t)(nv < 1 ? 1 : (nv > BRRR_MAXSEQ ? BRRR_MAXSEQ : nv));
    snprintf(prompt, prompt_cap, "%s", un.c_str());
    return 1;
}

// ---------------------------------------------------------------- qwen3moe: ChatML prompt, generate, serve line (engine_qwen2.rs:622-683)
// Prompt ids: <|im_start|> "system\nYou are a helpful assistant." <|im_end|> <|im_start|> "\nuser\n" + text
// <|im_end|> <|im_start|> "\nassistant\n"; text pieces go through the greedy longest-match encoder with a
// 48-byte window (engine_qwen2.rs:500-505); the special tokens are looked up by their literal spelling.
extern "C" int brrr_qwen_chat_prompt(const brrr_tokenizer *t, const char *user_text, uint32_t *out, size_t cap, size_t *n_out) {
    if (!t || !user_text || !n_out) return BRRR_ERR_ARG;
    uint32_t im_start = 0, im_end = 0;
    if (brrr_tokenizer_special(t, "<|im_start|>", &im_start) != BRRR_OK || brrr_tokenizer_special(t, "<|im_end|>", &im_end) != BRRR_OK) return BRRR_ERR_IO;
    std::vector<uint32_t> ids;
    auto enc = [&](const std::string &s) -> int {
        size_t n = 0;
        int st = brrr_tokenizer_encode(t, s.data(), s.size(), 48, nullptr, 0, &n);
        if (st != BRRR_OK) return st;
        size_t at = ids.size();
        ids.resize(at + n);
        return brrr_tokenizer_encode(t, s.data(), s.size(), 48, ids.data() + at, n, &n);
    };
    int st;
    ids.push_back(im_start);
    if ((st = enc("system\nYou are a helpful assistant.")) != BRRR_OK) return st;
    ids.push_back(im_end);
    ids.push_back(im_start);
    if ((st = enc(std::string("\nuser\n") + user_text)) != BRRR_OK) return st;
    ids.push_back(im_end);
    ids.push_back(im_start);
    if ((st = enc("\nassistant\n")) != BRRR_OK) return st;
    *n_out = ids.size();
    if (out) {
        if (ids.size() > cap) return BRRR_ERR_RANGE;
        memcpy(out, ids.data(), ids.size() * 4);
    }
    return BRRR_OK;
}

// Token-by-token prefill, then greedy decode until <|im_end|>, a token id beyond the vocabulary file,
// ngen tokens or the context limit (engine_qwen2.rs:632-650).  Decoding runs on the device in bursts.
extern "C" int brrr_qwen_generate(brrr_qwen *m, const brrr_tokenizer *t, const uint32_t *ids, size_t n_ids, uint32_t ngen,
                                  void (*emit)(const char *, uint32_t, void *), void *emit_arg, uint32_t *out_ids, size_t out_cap,
                                  brrr_gen_stats *stats) {
    if (!m || !t || !ids || n_ids == 0) return BRRR_ERR_ARG;
    if (n_ids >= BRRR_MAXSEQ) return BRRR_ERR_RANGE;
    uint32_t im_end = 0;
    if (brrr_tokenizer_special(t, "<|im_end|>", &im_end) != BRRR_OK) return BRRR_ERR_IO;
    const uint32_t ntok = brrr_tokenizer_size(t);
    auto t0 = std::chrono::steady_clock::now();
    uint32_t next = 0;
    int st;
    for (size_t i = 0; i < n_ids; i++)
        if ((st = brrr_qwen_forward(m, ids[i], (uint32_t)i, i + 1 == n_ids, &next)) != BRRR_OK) return st;
    auto t1 = std::chrono::steady_clock::now();
    size_t pos = n_ids;
    uint32_t n = 0;
    auto stop = [&](uint32_t tok) { return tok == im_end || tok >= ntok; };
    std::vector<uint32_t> burst(32);
    while (n < ngen && !stop(next) && pos + 1 < BRRR_MAXSEQ) {
        uint32_t want = ngen - n < 32 ? ngen - n : 32;
        if (pos + want >= BRRR_MAXSEQ) want = (uint32_t)(BRRR_MAXSEQ - 1 - pos);
        if (want == 0) break;
        if ((st = brrr_qwen_decode(m, next, (uint32_t)pos, want, burst.data())) != BRRR_OK) return st;
        for (uint32_t used = 0; used < want; used++) {
            if (out_ids && n < out_cap) out_ids[n] = next;
            if (emit) {
                const char *b; uint32_t l;
                if (brrr_tokenizer_token(t, next, &b, &l) == BRRR_OK) emit(b, l, emit_arg);
            }
            n++; pos++;
            next = burst[used];
            if (n >= ngen || stop(next) || pos + 1 >= BRRR_MAXSEQ) break;      // steps the device ran beyond this one are discarded
        }
    }
    auto t2 = std::chrono::steady_clock::now();
    if (stats) {
        stats->prefill_tokens = (uint32_t)n_ids;
        stats->decode_tokens = n;
        stats->prefill_seconds = std::chrono::duration<double>(t1 - t0).count();
        stats->decode_seconds = std::chrono::duration<double>(t2 - t1).count();
    }
    return BRRR_OK;
}

static void emit_stdout(const char *b, uint32_t l, void *) {
    fwrite(b, 1, l, stdout);
    fflush(stdout);
}

// The reference binary's command line: <data-dir> <blob> [prompt|--serve] [ngen].
extern "C" int brrr_cli_main(int argc, char **argv) {
    if (argc < 3) { fprintf(stderr, "usage: %s <data-dir> <blob> [prompt|--serve] [ngen]\n", argv[0]); return 2; }
    const char *dir = argv[1], *blob = argv[2];
    std::string prompt = argc > 3 ? argv[3] : "Why is the sky blue?";
    brrr_tokenizer *tok = nullptr;
    if (brrr_tokenizer_open(dir, &tok) != BRRR_OK) { fprintf(stderr, "cannot read %s/tokens.bin\n", dir); return 1; }
    fprintf(stderr, "loading model blob...\n");
    brrr_model *m = nullptr;
    int st = brrr_model_open(dir, blob, 0, &m);
    if (st != BRRR_OK) { fprintf(stderr, "model open failed: %s (%s)\n", brrr_strerror(st), brrr_last_cuda_error()); return 1; }
    uint64_t rng = 0x9E3779B97F4A7C15ull;
    auto run = [&](const std::string &text, uint32_t ngen, uint32_t temp_milli, bool serve) -> int {
        size_t n = 0;
        int s2 = brrr_chat_prompt(tok, text.c_str(), nullptr, 0, &n);
        if (s2 != BRRR_OK) { fprintf(stderr, "prompt not encodable\n"); return s2; }
        std::vector<uint32_t> ids(n);
        brrr_chat_prompt(tok, text.c_str(), ids.data(), n, &n);
        brrr_gen_stats gs{};
        s2 = brrr_generate(m, tok, ids.data(), n, ngen, temp_milli, 40, &rng, emit_stdout, nullptr, nullptr, 0, &gs);
        if (s2 != BRRR_OK) { fprintf(stderr, "generate failed: %s (%s)\n", brrr_strerror(s2), brrr_last_cuda_error()); return s2; }
        printf("\n[STATS] prefill_tok=%u prefill_s=%.2f decode_tok=%u decode_s=%.2f tok_s=%.1f\n%s", gs.prefill_tokens, gs.prefill_seconds,
               gs.decode_tokens, gs.decode_seconds, gs.decode_seconds > 0 ? gs.decode_tokens / gs.decode_seconds : 0.0, serve ? "[DONE]\n" : "");
        fflush(stdout);
        return BRRR_OK;
    };
    int rc = 0;
    if (prompt == "--serve") {
        fprintf(stderr, "[READY]\n");
        // Temperature and random state belong to the process, as the reference's TEMP_MILLI /
        // RNG_STATE globals (src/bin/engine_gpt2.rs:1456-1466): a bare-prompt line after a
        // temp/seed/ngen/prompt line keeps that line's temperature and continues its random stream.
        uint32_t temp_milli = 0;
        char *line = nullptr;
        size_t cap = 0;
        std::vector<char> ptext;
        ssize_t got;
        while ((got = getline(&line, &cap, stdin)) >= 0) {       // whole lines, whatever their length
            float temp = 0.0f; uint64_t seed = 0; uint32_t ngen = 0;
            ptext.assign((size_t)got + 2, 0);
            int form = brrr_serve_parse(line, &temp, &seed, &ngen, ptext.data(), ptext.size());
            if (form < 0 || ptext[0] == 0) continue;
            if (form == 1) { temp_milli = (uint32_t)(temp * 1000.0f); rng = brrr_rng_seed(seed); }
            if (run(ptext.data(), form == 1 ? ngen : 256, temp_milli, true) != BRRR_OK) { rc = 1; break; }
        }
        free(line);
    } else {
        uint32_t ngen = argc > 4 ? (uint32_t)strtoul(argv[4], nullptr, 10) : 96;
        rc = run(prompt, ngen ? ngen : 96, 0, false) == BRRR_OK ? 0 : 1;
    }
    brrr_model_close(m);
    brrr_tokenizer_close(tok);
    return rc;
}

// One request line of the qwen3moe serve loop (engine_qwen2.rs:664-673): the line is trimmed; if it
// splits into four tab-separated fields and the third is a count, that is ngen and the fourth is the
// prompt with every "\\n" and "\\t" turned into a SPACE (temperature and seed are accepted and ignored:
// this engine is greedy only); otherwise the whole line is the prompt.  Returns 1 / 0, -1 for an empty line.
extern "C" int brrr_qwen_serve_parse(const char *line, uint32_t *ngen, char *prompt, size_t prompt_cap) {
    if (!line || !prompt || prompt_cap == 0) return -1;
    std::string s(line);
    auto ws = [](char c) { return c == ' ' || c == '\t' || c == '\n' || c == '\r' || c == '\f' || c == '\v'; };
    while (!s.empty() && ws(s.back())) s.pop_back();
    size_t b = 0;
    while (b < s.size() && ws(s[b])) b++;
    s = s.substr(b);
    if (s.empty()) return -1;
    size_t p1 = s.find('\t'), p2 = p1 == std::string::npos ? p1 : s.find('\t', p1 + 1), p3 = p2 == std::string::npos ? p2 : s.find('\t', p2 + 1);
    if (p3 != std::string::npos) {
        std::string f2 = s.substr(p2 + 1, p3 - p2 - 1);
        size_t i = !f2.empty() && f2[0] == '+' ? 1 : 0;
        bool num = i < f2.size();
        unsigned long long v = 0;
        for (size_t k = i; k < f2.size() && num; k++) {
            if (f2[k] < '0' || f2[k] > '9') num = false;
            else if ((v = v * 10 + (unsigned)(f2[k] - '0')) > (1ull << 40)) v = 1ull << 40;
        }
        if (num) {
            std::string f3 = s.substr(p3 + 1), un;
            for (size_t k = 0; k < f3.size(); k++) {
                if (f3[k] == '\\' && k + 1 < f3.size() && (f3[k + 1] == 'n' || f3[k + 1] == 't')) { un.push_back(' '); k++; }
                else un.push_back(f3[k]);
            }
            if (ngen) *ngen = (uint32_t)(v > BRRR_MAXSEQ ? BRRR_MAXSEQ : v);
            snprintf(prompt, prompt_cap, "%s", un.c_str());
            return 1;
        }
    }
    snprintf(prompt, prompt_cap, "%s", s.c_str());
    return 0;
}

// The qwen3moe reference binary's command line (engine_qwen2.rs:486-489, 622-683):
// <data-dir> <blob> [prompt|--serve] [ngen]; default ngen 64 (256 when serving).
extern "C" int brrr_qwen_cli_main(int argc, char **argv) {
    if (argc < 3) { fprintf(stderr, "usage: %s <data-dir> <blob> [prompt|--serve] [ngen]\n", argv[0]); return 2; }
    const char *dir = argv[1], *blob = argv[2];
    std::string prompt = argc > 3 ? argv[3] : "Write a haiku about CPUs.";
    const bool serve = prompt == "--serve";
    uint32_t ngen_default = serve ? 256 : 64;
    if (argc > 4) { char *end = nullptr; unsigned long v = strtoul(argv[4], &end, 10); if (end && *end == 0 && argv[4][0]) ngen_default = (uint32_t)v; }
    brrr_tokenizer *tok = nullptr;
    if (brrr_tokenizer_open(dir, &tok) != BRRR_OK) { fprintf(stderr, "cannot read %s/tokens.bin\n", dir); return 1; }
    fprintf(stderr, "loading blob...\n");
    brrr_qwen *m = nullptr;
    int st = brrr_qwen_open(dir, blob, 0, &m);
    if (st != BRRR_OK) { fprintf(stderr, "model open failed: %s (%s)\n", brrr_strerror(st), brrr_last_cuda_error()); return 1; }
    auto run = [&](const std::string &text, uint32_t ngen, brrr_gen_stats *gs) -> int {
        size_t n = 0;
        int s2 = brrr_qwen_chat_prompt(tok, text.c_str(), nullptr, 0, &n);
        if (s2 != BRRR_OK) { fprintf(stderr, "prompt not encodable\n"); return s2; }
        std::vector<uint32_t> ids(n);
        brrr_qwen_chat_prompt(tok, text.c_str(), ids.data(), n, &n);
        fprintf(stderr, "prompt: %zu tokens\n", n);
        s2 = brrr_qwen_generate(m, tok, ids.data(), n, ngen, emit_stdout, nullptr, nullptr, 0, gs);
        if (s2 != BRRR_OK) fprintf(stderr, "generate failed: %s (%s)\n", brrr_strerror(s2), brrr_last_cuda_error());
        return s2;
    };
    int rc = 0;
    if (serve) {
        fprintf(stderr, "[READY]\n");
        char *line = nullptr;
        size_t cap = 0;
        ssize_t got;
        std::vector<char> ptext;
        while ((got = getline(&line, &cap, stdin)) >= 0) {
            uint32_t ngen = 0;
            ptext.assign((size_t)got + 2, 0);
            int form = brrr_qwen_serve_parse(line, &ngen, ptext.data(), ptext.size());
            if (form < 0) continue;
            brrr_gen_stats gs{};
            if (run(ptext.data(), form == 1 ? ngen : ngen_default, &gs) != BRRR_OK) { rc = 1; break; }
            // the reference prints prefill_tok=0 here (engine_qwen2.rs:677)
            printf("\n[STATS] prefill_tok=0 prefill_s=%.3f decode_tok=%u decode_s=%.3f tok_s=%.1f\n[DONE]\n", gs.prefill_seconds, gs.decode_tokens,
                   gs.decode_seconds, gs.decode_seconds > 0 ? gs.decode_tokens / gs.decode_seconds : 0.0);
            fflush(stdout);
        }
        free(line);
    } else {
        brrr_gen_stats gs{};
        rc = run(prompt, ngen_default, &gs) == BRRR_OK ? 0 : 1;
        if (rc == 0)
            printf("\n---\ndecode: %u tokens in %.2fs = %.1f tok/s\n", gs.decode_tokens, gs.decode_seconds,
                   gs.decode_seconds > 0 ? gs.decode_tokens / gs.decode_seconds : 0.0);
    }
    brrr_qwen_close(m);
    brrr_tokenizer_close(tok);
    return rc;
}
