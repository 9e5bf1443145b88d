/* brrr.h — C ABI of the B200 decode engine.
 *
 * This is the boundary a host program links against (the reference host is Rust: an
 * `unsafe extern "C"` block binds these symbols unchanged).  Plain pointers and sizes only; every
 * function returns an int status (0 = BRRR_OK), never aborts and never throws.  A model handle
 * owns all of its device memory; use one host thread per handle.
 *
 * The reference (arizqi/cpubrrr) has no FFI: its engines are monolithic binaries.  Each entry
 * point below names the reference function or code region it replaces, by file:line within the
 * reference project.
 *
 * Pointers named d_* are CUDA device pointers; everything else is host memory.
 * `stream` arguments are a cudaStream_t passed as void* (NULL = the default stream).
 */
#ifndef BRRR_H
#define BRRR_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    BRRR_OK = 0,
    BRRR_ERR_ARG = 1,        /* bad argument / unsupported shape */
    BRRR_ERR_IO = 2,         /* data directory or blob unreadable / malformed */
    BRRR_ERR_CUDA = 3,       /* a CUDA call failed; brrr_last_cuda_error() has the text */
    BRRR_ERR_NOMEM = 4,
    BRRR_ERR_RANGE = 5,      /* position / token / count out of range */
    BRRR_ERR_STATE = 6       /* call not valid in the handle's current state */
};

#define BRRR_MAXSEQ 4096     /* src/bin/engine_gpt2.rs:16 */
#ifndef BRRR_TILE_MAX
#define BRRR_TILE_MAX 512    /* most token rows one pass over the layers takes (the reference's TILE is 16, src/bin/engine_gpt2.rs:19;
                              * every row's result is independent of the tile size) */
#endif

/* Model hyper-parameters: the keys of the data directory's config.txt
 * (scripts/setup_model.sh:71-89, parsed at src/bin/engine_gpt2.rs:58-80). */
typedef struct brrr_cfg {
    int32_t n_embd, n_layer, n_head, n_head_kv, head_dim;
    int32_t n_expert, n_expert_used, n_ff_exp, sliding_window, n_vocab;
    float rope_freq_base, rms_eps;
} brrr_cfg;

typedef struct brrr_model brrr_model;

const char *brrr_strerror(int status);
const char *brrr_last_cuda_error(void);

/* ---------------------------------------------------------------- model lifetime */

/* Load a model from a data directory (config.txt, manifest.txt) and its GGUF blob: mmap, upload,
 * quantise attention/head weights from bf16 to Q8 and re-lay the MXFP4 experts, all on `device`.
 * Replaces load_cfg + the loader in main (src/bin/engine_gpt2.rs:64-80, 1276-1352):
 * Q8Mat::from_bf16 (464-494), repack_mx (439-461), rope_init (536-550). */
int brrr_model_open(const char *data_dir, const char *blob_path, int device, brrr_model **out);

/* Same model container filled with seeded synthetic tensors generated on the device in the GGUF
 * tensor formats (no file involved), then converted exactly as brrr_model_open converts a blob.
 * No counterpart in the reference: it stands in for a checkpoint where none is available. */
int brrr_model_open_synth(const brrr_cfg *cfg, uint64_t seed, int device, brrr_model **out);

int brrr_model_cfg(const brrr_model *m, brrr_cfg *out);
void brrr_model_close(brrr_model *m);

/* ---------------------------------------------------------------- forward pass */

/* One token through the whole network at position `pos`; with want_logits != 0 the vocabulary
 * projection runs and *out_tok receives the greedy token (first strict maximum).  Host token in,
 * host token out.  Replaces the closure `run(tok, pos, want) -> u32` and the worker dispatch
 * behind it (src/bin/engine_gpt2.rs:1373-1385; forward_worker 751-934; head 936-1002).  The
 * whole step is one CUDA graph launch. */
int brrr_forward(brrr_model *m, uint32_t tok, uint32_t pos, int want_logits, uint32_t *out_tok);

/* A tile of tokens at positions pos0.. (prefill); the result equals feeding them one by one, as
 * the reference guarantees for run_tile (src/bin/engine_gpt2.rs:1004-1010, 1387-1393). */
int brrr_forward_tile(brrr_model *m, const uint32_t *toks, uint32_t n, uint32_t pos0, int want_logits, uint32_t *out_tok);

/* Schedule of brrr_forward_tile.  on != 0 (default): tiles of up to BRRR_TILE_MAX tokens walk the layers
 * together as in forward_tile_worker (src/bin/engine_gpt2.rs:1011-1250, where TILE = 16): q/k/v and the
 * output projection once per 16 rows, attention for all rows in one launch, the MoE block once per layer
 * and tile on the tensor-core tile kernels.  on = 0: one graph launch per token.  Same bits either way;
 * the environment variables BRRR_TILE_PREFILL=0/1 and BRRR_TILE_ROWS=n (2..BRRR_TILE_MAX) set the initial
 * values.  Ignored by expert-parallel ranks (always token-serial). */
int brrr_model_set_tile_prefill(brrr_model *m, int on);

/* Batched decode over independent sequences.  The reference decodes one sequence; its tile path
 * (forward_tile_worker, src/bin/engine_gpt2.rs:1011-1250) already walks several token rows through a
 * layer together and groups them by routed expert (the `subs` / `active` lists, :1160-1172).  Here a
 * row is (token, position, sequence): every sequence has its own KV cache, the dense projections and
 * the vocabulary projection read their weights once per 8 rows, each selected expert is read once
 * for all the rows routed to it.  Every row's result is bit-identical to brrr_forward on that
 * sequence alone.
 *   brrr_batch_open     allocates nseq (1..BRRR_BATCH_MAX) caches; once per model, not with expert-parallel ranks
 *   brrr_batch_prefill  feeds n prompt tokens of one sequence from position pos0 (tiles, no logits)
 *   brrr_batch_step     n rows (1..BRRR_TILE_MAX) in one pass; out_toks[i] = greedy next token of row i.
 *                       A row attends over its sequence's cache up to pos[i] - 1 plus itself; rows of one
 *                       sequence must carry ascending positions
 *   brrr_batch_step_logits  the same, and the rows' logits [n][n_vocab] to host memory */
#define BRRR_BATCH_MAX 256
int brrr_batch_open(brrr_model *m, int nseq);
int brrr_batch_prefill(brrr_model *m, uint32_t seq, const uint32_t *toks, uint32_t n, uint32_t pos0);
int brrr_batch_step(brrr_model *m, int n, const uint32_t *toks, const uint32_t *pos, const uint32_t *seq, uint32_t *out_toks);
int brrr_batch_step_logits(brrr_model *m, int n, const uint32_t *toks, const uint32_t *pos, const uint32_t *seq, uint32_t *out_toks, float *out_logits);

/* n greedy decode steps starting from `first_tok` at position `pos`, the token id staying on the
 * device between steps (one graph launch per step, no host round trip); out_toks[i] is the token
 * produced by step i.  Replaces the decode loop of generate (src/bin/engine_gpt2.rs:1431-1438)
 * without its stop-token test, which the caller applies to out_toks. */
int brrr_decode(brrr_model *m, uint32_t first_tok, uint32_t pos, uint32_t n, uint32_t *out_toks);

/* Same loop, asynchronous: enqueue n steps on the model's stream and return; the tokens are
 * collected by brrr_decode_wait.  Lets a caller time the device work with its own events. */
int brrr_decode_enqueue(brrr_model *m, uint32_t first_tok, uint32_t pos, uint32_t n);
int brrr_decode_wait(brrr_model *m, uint32_t n, uint32_t *out_toks);

/* Full-vocabulary Q8 logits of the last want_logits step (host buffer of n_vocab floats); the
 * values `CPBRR_HEADCHK` materialises at src/bin/engine_gpt2.rs:973-976. */
int brrr_logits(brrr_model *m, float *out);
/* Residual stream x after the last step (host buffer of n_embd floats); the vector the
 * reference's DUMP / CPBRR_DBG taps summarise (src/bin/engine_gpt2.rs:924-928). */
int brrr_hidden(brrr_model *m, float *out);
/* Debug forward that runs the same kernels un-graphed and copies x after the embedding and after
 * every layer into trace[(n_layer+1)][n_embd] (host). */
int brrr_forward_trace(brrr_model *m, uint32_t tok, uint32_t pos, float *trace);
/* The model's CUDA stream (cudaStream_t as void*), for callers that record their own events. */
void *brrr_model_stream(brrr_model *m);
/* Number of kernel launches one decode step performs (graph kernel nodes). */
int brrr_model_launches_per_step(const brrr_model *m, int want_logits);
/* How many steps had to be re-run because the fast router estimate that starts the expert weight
 * stream early missed an expert the exact router chose (results are unaffected; this is a
 * performance counter).  No counterpart in the reference. */
uint64_t brrr_model_spec_redos(const brrr_model *m);
/* How many times a bounded device wait of the speculative step ran out (the exact router, which
 * runs on its own branch of the step's graph, had not published its routing within about a
 * second).  The step concerned was re-run without speculation and the model has used the plain
 * step since; results are unaffected.  0 or 1.  No counterpart in the reference. */
uint64_t brrr_model_wait_fallbacks(const brrr_model *m);
/* Weight + KV bytes one decode step at position `pos` must read in the run-time formats. */
uint64_t brrr_model_bytes_per_step(const brrr_model *m, uint32_t pos);

/* Stage timing for roofline reports.  The decode step is made of brrr_stage_count() kernel
 * classes (brrr_stage_name(i)); brrr_stage_time replays, as one CUDA graph, every launch of one
 * class that a step at position `pos` performs (all layers, real weights, so the working set
 * exceeds L2 for the streaming classes), `reps` times between two events on the model's stream,
 * and returns the mean duration of one launch, the algorithmic bytes one launch reads and the
 * launches per step.  Counterpart of the reference's per-stage timers TM[5]
 * (src/bin/engine_gpt2.rs:56, 843-929, 1496-1497). */
int brrr_stage_count(void);
const char *brrr_stage_name(int stage);
int brrr_stage_time(brrr_model *m, int stage, uint32_t pos, int reps, float *ms_per_launch, uint64_t *bytes_per_launch, int *launches_per_step);


/* ---------------------------------------------------------------- expert parallelism (one process per GPU)
 * Rank r of `world` (<= 8, dividing n_expert) loads the experts [r * n_expert / world, (r + 1) *
 * n_expert / world) only; attention, router, norms, embedding and head are replicated and computed
 * redundantly, so every rank produces the same token.  Per layer the ranks exchange the selected
 * experts' down-projection slices through peer memory inside the down-projection kernel and fold
 * them in slot order: results equal the single-GPU model bit for bit.  Every rank must issue the
 * same sequence of forward / decode calls.  No counterpart in the reference (single process, CPU);
 * it serves the gpt-oss-120b configuration, whose experts are sharded by index over the GPUs of a node.
 *
 * Set-up: open on every rank, exchange the 64-byte handles (any host-side all-gather), make sure
 * every rank has opened (a host barrier), then attach on every rank at the same time: attach runs
 * the first step, which already synchronises with the peers (a rank whose peers do not show up
 * within about ten seconds fails with BRRR_ERR_STATE on its next call instead of hanging). */
int brrr_model_open_synth_ep(const brrr_cfg *cfg, uint64_t seed, int device, int rank, int world, brrr_model **out);
int brrr_model_open_ep(const char *data_dir, const char *blob_path, int device, int rank, int world, brrr_model **out);
int brrr_model_ep_handle(brrr_model *m, void *handle64);          /* IPC handle of this rank's exchange region */
int brrr_model_ep_attach(brrr_model *m, const void *handles);     /* world x 64 bytes in rank order (own entry ignored) */
int brrr_model_ep_info(const brrr_model *m, int *rank, int *world, int *first_expert, int *n_local_experts);

/* ---------------------------------------------------------------- host text layer (gpt-oss engine)
 * Pure host code around the forward pass: tokenizer, sampler, chat prompt, generate, serve. */
typedef struct brrr_tokenizer brrr_tokenizer;
/* Reads <data_dir>/tokens.bin (u32 count, then u16 length + bytes per token).  Tokens spelled
 * "<|...|>" are special (never matched by encode); among equal byte strings the lowest id wins.
 * Replaces the tokenizer set-up of main (src/bin/engine_gpt2.rs:1261-1268). */
int brrr_tokenizer_open(const char *data_dir, brrr_tokenizer **out);
void brrr_tokenizer_close(brrr_tokenizer *t);
uint32_t brrr_tokenizer_size(const brrr_tokenizer *t);
int brrr_tokenizer_token(const brrr_tokenizer *t, uint32_t id, const char **bytes, uint32_t *len);
int brrr_tokenizer_special(const brrr_tokenizer *t, const char *text, uint32_t *id);
/* Greedy longest match with pieces of at most max_piece bytes (32 for gpt-oss, 48 for qwen3moe).
 * out nullable (count only); *n_out receives the number of ids; BRRR_ERR_RANGE when a byte is
 * not encodable or cap is too small.  Replaces the closure `encode`
 * (src/bin/engine_gpt2.rs:1269-1274, src/bin/engine_qwen2.rs:501-506). */
int brrr_tokenizer_encode(const brrr_tokenizer *t, const char *text, size_t len, uint32_t max_piece, uint32_t *out, size_t cap, size_t *n_out);

/* Sampler state from a request seed (splitmix64 scramble, never zero; src/bin/engine_gpt2.rs:1462-1466). */
uint64_t brrr_rng_seed(uint64_t seed);
/* Temperature + top-k sampling over host logits; greedy (first strict maximum) when temp_milli == 0
 * or rng_state == NULL.  top_k is clamped to 1..64; the random draw is one xorshift64 step of
 * *rng_state.  Replaces sample_logits (src/bin/engine_gpt2.rs:82-126); exp is the engine's fixed
 * operation sequence instead of the platform's libm. */
uint32_t brrr_sample_logits(const float *logits, uint32_t n, uint32_t temp_milli, uint32_t top_k, uint64_t *rng_state);

/* Token ids of the harmony chat prompt for one user turn (src/bin/engine_gpt2.rs:1401-1414). */
int brrr_chat_prompt(const brrr_tokenizer *t, const char *user_text, uint32_t *out, size_t cap, size_t *n_out);

typedef struct brrr_gen_stats {
    uint32_t prefill_tokens, decode_tokens;
    double prefill_seconds, decode_seconds;
} brrr_gen_stats;
/* Prefill ids, then decode until a stop token (200002, 199999), ngen tokens or the context limit;
 * emit (nullable) gets the bytes of every produced token, out_ids (nullable) the ids.  Greedy
 * decoding runs on the device in bursts.  Replaces generate (src/bin/engine_gpt2.rs:1400-1440). */
int brrr_generate(brrr_model *m, const brrr_tokenizer *t, const uint32_t *ids, size_t n_ids, uint32_t ngen, uint32_t temp_milli,
                  uint32_t top_k, uint64_t *rng_state, void (*emit)(const char *, uint32_t, void *), void *emit_arg,
                  uint32_t *out_ids, size_t out_cap, brrr_gen_stats *stats);
/* One request line of the serve protocol: bare prompt (returns 0) or `temp \t seed \t ngen \t prompt`
 * with \n, \t, \\ escapes (returns 1); -1 on bad arguments (src/bin/engine_gpt2.rs:1454-1482). */
int brrr_serve_parse(const char *line, float *temp, uint64_t *seed, uint32_t *ngen, char *prompt, size_t prompt_cap);
/* main() of the engine binary: <data-dir> <blob> [prompt|--serve] [ngen]; [READY] on stderr, streamed
 * tokens, "[STATS] ..." and "[DONE]" lines on stdout (src/bin/engine_gpt2.rs:1252-1500). */
int brrr_cli_main(int argc, char **argv);

/* ---------------------------------------------------------------- qwen3moe engine
 * The reference's second engine binary (src/bin/engine_qwen2.rs): Qwen3-MoE models with Q4_K / Q6_K
 * weights used straight in the GGUF byte layout, Q8_K activations, QK-norm, NeoX RoPE, full
 * causal attention (head_dim 128), top-k-of-n experts with SiLU-GLU.  Same conventions as the
 * brrr_model_* functions above. */
typedef struct brrr_qwen_cfg {          /* config.txt keys, src/bin/engine_qwen2.rs:27-38 */
    int32_t n_embd, n_layer, n_head, n_head_kv, head_dim;
    int32_t n_expert, n_expert_used, n_ff_exp, n_vocab;
    float rope_freq_base, rms_eps;
} brrr_qwen_cfg;
typedef struct brrr_qwen brrr_qwen;

/* Load from a data directory and its GGUF blob.  Replaces load_cfg and the loader in main
 * (src/bin/engine_qwen2.rs:27-38, 512-545); token_embd must be Q4_K, matrices Q4_K or Q6_K. */
int brrr_qwen_open(const char *data_dir, const char *blob_path, int device, brrr_qwen **out);
/* Seeded synthetic model generated on the device in the GGUF formats (down experts and the output
 * head Q6_K, every other matrix Q4_K).  No counterpart in the reference. */
int brrr_qwen_open_synth(const brrr_qwen_cfg *cfg, uint64_t seed, int device, brrr_qwen **out);
int brrr_qwen_cfg_get(const brrr_qwen *m, brrr_qwen_cfg *out);
void brrr_qwen_close(brrr_qwen *m);
/* One token at position pos; with want_logits != 0 the vocabulary projection runs and *out_tok is
 * the greedy token (first strict maximum).  Replaces run(t, pos) and the worker pool
 * (src/bin/engine_qwen2.rs:302-451, 571-595). */
int brrr_qwen_forward(brrr_qwen *m, uint32_t tok, uint32_t pos, int want_logits, uint32_t *out_tok);
/* n greedy steps starting from first_tok at position pos with the token fed back on the device;
 * out_toks[i] is the token produced by step i.  Replaces the decode loop of generate
 * (src/bin/engine_qwen2.rs:613-619) without its stop test. */
int brrr_qwen_decode(brrr_qwen *m, uint32_t first_tok, uint32_t pos, uint32_t n, uint32_t *out_toks);
/* The same in two halves: enqueue returns as soon as the n steps are queued on the model's stream,
 * wait blocks and fetches the tokens. */
int brrr_qwen_decode_enqueue(brrr_qwen *m, uint32_t first_tok, uint32_t pos, uint32_t n);
int brrr_qwen_decode_wait(brrr_qwen *m, uint32_t n, uint32_t *out_toks);
int brrr_qwen_logits(brrr_qwen *m, float *out);               /* [n_vocab], of the last want_logits step */
int brrr_qwen_hidden(brrr_qwen *m, float *out);               /* [n_embd], residual stream after the last step */
/* One step run kernel by kernel, recording the residual stream after the embedding and after each
 * layer: trace is host memory [(n_layer + 1)][n_embd]. */
int brrr_qwen_forward_trace(brrr_qwen *m, uint32_t tok, uint32_t pos, float *trace);
void *brrr_qwen_stream(brrr_qwen *m);
int brrr_qwen_launches_per_step(const brrr_qwen *m, int want_logits);
uint64_t brrr_qwen_bytes_per_step(const brrr_qwen *m, uint32_t pos);

/* ChatML prompt ids of the qwen3moe engine: im_start "system\nYou are a helpful assistant." im_end im_start
 * "\nuser\n" + text im_end im_start "\nassistant\n", text pieces through brrr_tokenizer_encode with a 48-byte
 * window, the two special tokens looked up by spelling (BRRR_ERR_IO when the vocabulary lacks them).
 * Replaces the prompt builder of generate (src/bin/engine_qwen2.rs:627-631, 500-505). */
int brrr_qwen_chat_prompt(const brrr_tokenizer *t, const char *user_text, uint32_t *out, size_t cap, size_t *n_out);
/* Token-by-token prefill, then greedy decode until <|im_end|>, an id beyond the vocabulary file, ngen tokens
 * or the context limit; emit (nullable) gets the bytes of every produced token, out_ids (nullable) the ids.
 * Replaces generate (src/bin/engine_qwen2.rs:626-650). */
int brrr_qwen_generate(brrr_qwen *m, const brrr_tokenizer *t, const uint32_t *ids, size_t n_ids, uint32_t ngen,
                       void (*emit)(const char *, uint32_t, void *), void *emit_arg, uint32_t *out_ids, size_t out_cap,
                       brrr_gen_stats *stats);
/* One request line of the qwen3moe serve loop: trimmed; `temp \t seed \t ngen \t prompt` (returns 1: ngen taken,
 * "\n" and "\t" escapes of the prompt become spaces, temp and seed ignored - the engine is greedy only) or a
 * bare prompt (returns 0); -1 for an empty line (src/bin/engine_qwen2.rs:659-673). */
int brrr_qwen_serve_parse(const char *line, uint32_t *ngen, char *prompt, size_t prompt_cap);
/* main() of the qwen3moe engine binary: <data-dir> <blob> [prompt|--serve] [ngen] (default 64, 256 when
 * serving); [READY] on stderr, streamed tokens, "[STATS] prefill_tok=0 ..." and "[DONE]" on stdout
 * (src/bin/engine_qwen2.rs:486-489, 622-683). */
int brrr_qwen_cli_main(int argc, char **argv);

/* ---------------------------------------------------------------- stage-level entry points
 * Device pointers in, device pointers out.  They launch the same kernels the forward pass uses. */

/* Per-32-block int8 quantiser: q[i] = round_half_away(x[i] / s[b]), s[b] = max(1e-12, amax)/127.
 * Replaces qblock32 / quant_i8 (src/bin/engine_gpt2.rs:689-699; src/bin/engine.rs:264-279). */
int brrr_quant_q8(const float *d_x, int n, int8_t *d_q, float *d_s, void *stream);

/* Q8_K activation quantiser of the qwen3moe engine: one scale per 256 values
 * (max(1e-12, amax)/127), int8 quants rounded half away from zero, and the int32 sum of every 32
 * quants (d_bsum [n/32]).  n % 256 == 0; d_x 16-byte, d_q 8-byte aligned.
 * Replaces qblock (src/bin/engine_qwen2.rs:287-300). */
int brrr_quant_q8k(const float *d_x, int n, int8_t *d_q, float *d_s, int32_t *d_bsum, void *stream);

/* y[r] = Q4_K row r . Q8_K activation, rows in the GGUF Q4_K byte layout (144 bytes per 256
 * values, rows contiguous).  d_sbdots (nullable) receives the exact integers of every superblock
 * as [rows][cols/256][2] = {scaled quant sum, min sum}.  cols % 256 == 0; d_w and d_xq 4-byte
 * aligned.  Replaces q4k_dot (src/bin/engine_qwen2.rs:84-114). */
int brrr_q4k_matvec(const uint8_t *d_w, int rows, int cols, const int8_t *d_xq, const float *d_ys, const int32_t *d_bsum,
                    float *d_y, int32_t *d_sbdots, void *stream);

/* y[r] = Q6_K row r . Q8_K activation, rows in the GGUF Q6_K byte layout (210 bytes per 256
 * values).  d_sbdots (nullable): [rows][cols/256] integer accumulators.  d_w and d_xq 2-byte
 * aligned.  Replaces q6k_dot (src/bin/engine_qwen2.rs:164-200). */
int brrr_q6k_matvec(const uint8_t *d_w, int rows, int cols, const int8_t *d_xq, const float *d_ys, float *d_y,
                    int32_t *d_sbdots, void *stream);

/* RMSNorm then brrr_quant_q8; d_xn (nullable) receives the normalised floats.
 * Replaces ssq + rmsnorm_quant_par (src/bin/engine_gpt2.rs:709-738). */
int brrr_rmsnorm_quant(const float *d_x, const float *d_w, float eps, int n, float *d_xn, int8_t *d_q, float *d_s, void *stream);

/* x[r] += sum over k ascending of wts[k] * (part[k][r] + down_b[top[k]][r]) (multiply, then add), then
 * brrr_rmsnorm_quant of the new x with d_norm_w (nullable: fold only) into d_q / d_s: the combine of
 * src/bin/engine_gpt2.rs:908-923 together with the norm + quantiser that opens the next layer
 * (709-738), as the decode step's last kernel of a layer runs them.  d_part: [topk][ceil(d / 128) * 128]
 * row sums of the down projection before bias, 16-byte aligned like d_x and d_down_b ([experts][d]).
 * wait_for_router != 0: the kernel first polls (bounded, about a second) for routing words that the
 * router of the decode step would publish; this call publishes none, so the wait runs out and the call
 * returns BRRR_ERR_STATE with the CUDA context intact (the test of that bounded wait).  Synchronous. */
int brrr_fold_norm(const int32_t *d_top, const float *d_wts, int topk, int d, const float *d_part, const float *d_down_b, float *d_x,
                   const float *d_norm_w, float eps, int8_t *d_q, float *d_s, int wait_for_router, void *stream);

/* Opaque device matrices in the engine's streaming layouts. */
typedef struct brrr_q8mat brrr_q8mat;
typedef struct brrr_mxmat brrr_mxmat;

/* bf16 [rows][cols] (device) -> Q8 matrix, quantised per 32-block as Q8Mat::from_bf16
 * (src/bin/engine_gpt2.rs:464-494). cols % 64 == 0. */
int brrr_q8mat_from_bf16(const uint16_t *d_w, int rows, int cols, brrr_q8mat **out, void *stream);
/* copies back the quantised values in natural order: q[rows][cols], s[rows][cols/32] (device) */
int brrr_q8mat_export(const brrr_q8mat *m, int8_t *d_q, float *d_s, void *stream);
void brrr_q8mat_free(brrr_q8mat *m);
/* y[r] = row r . Q8 activation.  Replaces dot_q8_i8 / Q8Mat::dot (src/bin/engine_gpt2.rs:165-191, 495-500). */
int brrr_q8_matvec(const brrr_q8mat *w, const int8_t *d_xq, const float *d_xs, float *d_y, void *stream);
/* The same product for 1..BRRR_TILE_MAX token rows in one pass over the weights: d_y[t * ldy + r] = row r . activation t
 * (d_xq [ntok][cols], d_xs [ntok][cols / 32]), every value bit-identical to brrr_q8_matvec on row t alone.  tensor_cores = 0:
 * integer units (dp4a; what the prompt tiles and batched decode run), 1: tcgen05 kind::i8 products with the int8 weights copied
 * straight into operand layout.  Replaces the q/k/v and o-proj loops of the tile path (src/bin/engine_gpt2.rs:1034-1118). */
int brrr_q8_matmul_rows(const brrr_q8mat *w, const int8_t *d_xq, const float *d_xs, int ntok, float *d_y, int ldy, int tensor_cores, void *stream);

/* GGUF MXFP4 rows (17-byte blocks, device) -> engine layout.  Replaces repack_mx
 * (src/bin/engine_gpt2.rs:439-461). rows % 16 == 0, blocks % 2 == 0. */
int brrr_mxmat_from_gguf(const uint8_t *d_raw, int rows, int blocks, brrr_mxmat **out, void *stream);
void brrr_mxmat_free(brrr_mxmat *m);
/* y[i] = row (row0 + i) . Q8 activation for i < nrows.  d_blockdots (nullable) receives the exact
 * int32 block accumulators as [nrows][blocks][4 lanes].  Replaces dot4_mx_i8
 * (src/bin/engine_gpt2.rs:193-228). */
int brrr_mx_matvec(const brrr_mxmat *w, int row0, int nrows, const int8_t *d_xq, const float *d_xs, float *d_y, int32_t *d_blockdots, void *stream);

/* The same product for a tile of up to BRRR_TILE_MAX tokens in one pass over the weights, on the tcgen05
 * tensor cores (int8 MMA into tensor memory, float chains in the epilogue): d_y[t * ldy + i] = row
 * (row0 + i) . activation t, each value bit-identical to brrr_mx_matvec on token t alone.
 * d_xq [ntok][blocks * 32] int8, d_xs [ntok][blocks].  Replaces the expert products of the tile
 * path (forward_tile_worker, src/bin/engine_gpt2.rs:1011-1250, TILE = 16). */
int brrr_mx_matmul_tile(const brrr_mxmat *w, int row0, int nrows, const int8_t *d_xq, const float *d_xs, int ntok, float *d_y, int ldy,
                        void *stream);

/* Router GEMV + top-k + softmax over the selected k.  d_b nullable.  d_logits [ne], d_top [k],
 * d_wts [k].  Replaces src/bin/engine_gpt2.rs:848-867. */
int brrr_router_topk(const float *d_w, const float *d_b, const float *d_xn, int ne, int d, int topk,
                     float *d_logits, int32_t *d_top, float *d_wts, void *stream);

/* The same router, for callers that cannot allocate device memory: a host that has given all of
 * its free HBM to its own pools, or a request path that must stay clear of cudaMalloc / cudaFree
 * because they take the driver's allocation lock and cudaFree synchronises the device.  Nothing
 * is allocated: the re-tiled matrix and the CTA arrival counter live in a fixed array inside the
 * library image (about 2.1 MB, held by every GPU that loads the library until the process
 * exits).  Limits: ne <= 128 and d <= 4096, otherwise BRRR_ERR_RANGE.  The first call on each
 * device looks up the array's device address; make that call before any stream capture.  All
 * calls share the one array, so two calls whose work overlaps on the GPU (different streams)
 * race; calls on one stream are safe.  It has no counterpart in the reference. */
int brrr_router_topk_noalloc(const float *d_w, const float *d_b, const float *d_xn, int ne, int d, int topk,
                             float *d_logits, int32_t *d_top, float *d_wts, void *stream);

/* Clamped SwiGLU on gu[topk][2d] (gate | up) then the per-32 quantiser.  Replaces
 * src/bin/engine_gpt2.rs:886-907. */
int brrr_swiglu_quant(const float *d_gu, int topk, int d, int8_t *d_hq, float *d_hs, void *stream);

/* Decode attention for all heads at position pos.  d_qkv holds this token's projected q | k | v
 * (bias added, not rotated); the kernel rotates q and k, appends k/v to the cache
 * [n_head_kv][BRRR_MAXSEQ][64] and attends over start..pos, then quantises the output.  d_rope is the
 * [BRRR_MAXSEQ][32][2] cos/sin table.  Replaces rope_yarn + the cache write + the attention stage
 * (src/bin/engine_gpt2.rs:575-587, 783-837). head_dim is 64. */
int brrr_attn_decode(const float *d_qkv, float *d_kc, float *d_vc, const float *d_rope, const float *d_sinks,
                     int n_head, int n_head_kv, int pos, int start, float *d_ao, int8_t *d_aq, float *d_as, void *stream);

/* YaRN cos/sin table [BRRR_MAXSEQ][head_dim/2][2] built on the host (src/bin/engine_gpt2.rs:531-572). */
int brrr_rope_table(const brrr_cfg *cfg, float *out);

/* One MoE FFN step of layer `il` on a normalised token: quantise d_xn, route, gate/up, SwiGLU,
 * down + weighted combine added onto d_x.  d_top/d_wts (nullable) receive the routing.
 * Replaces src/bin/engine_gpt2.rs:847-923. */
int brrr_moe_ffn_step(brrr_model *m, int il, const float *d_xn, float *d_x, int32_t *d_top, float *d_wts);

/* The same step through the expert kernels the speculative decode step runs: gate/up and down on
 * the tensor cores in their native 4-bit format (tcgen05.mma kind::mxf4.block_scale on the raw e2m1
 * codes, the Q8 activation split into three exact digit planes), results bit-identical to
 * brrr_moe_ffn_step.  BRRR_ERR_STATE when the model holds no tile-unit copy of the experts
 * (expert-parallel models, shapes with n_embd % 64 != 0, BRRR_NOMXT=1, or not enough memory).
 * Replaces src/bin/engine_gpt2.rs:847-923. */
int brrr_moe_ffn_step_tc(brrr_model *m, int il, const float *d_xn, float *d_x, int32_t *d_top, float *d_wts);
/* 1 when the decode step of this model runs its expert matvecs on the tensor cores. */
int brrr_model_uses_tensor_experts(const brrr_model *m);

/* The same MoE FFN for a tile of 1..BRRR_TILE_MAX normalised tokens (d_xn [ntok][n_embd], d_x [ntok][n_embd]
 * residuals, d_top / d_wts nullable [ntok][n_expert_used]): per-token router, then gate / up /
 * down as grouped tensor-core matmuls (tcgen05) that read each selected expert once for all the
 * tokens routed to it.  Bit-identical to brrr_moe_ffn_step applied token by token.  Replaces the MoE
 * part of forward_tile_worker (src/bin/engine_gpt2.rs:1120-1250). */
int brrr_moe_ffn_tile(brrr_model *m, int il, const float *d_xn, float *d_x, int ntok, int32_t *d_top, float *d_wts);

/* Fill a device buffer with a synthetic tensor in its GGUF format (type 0 = f32, 30 = bf16,
 * 39 = MXFP4, 12 = Q4_K, 14 = Q6_K; nelems counts values). Same generator brrr_model_open_synth uses. */
int brrr_synth_tensor(uint64_t seed, uint32_t layer, uint32_t kind, uint32_t type, uint64_t nelems, void *d_out, void *stream);

/* exp as the engine defines it (fixed IEEE sequence); d_y[i] = exp(d_x[i]). */
int brrr_expf(const float *d_x, int n, float *d_y, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* BRRR_H */
