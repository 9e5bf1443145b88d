"""numpy port of the counter-based synthetic tensor generator (csrc/brrr_synth.h) and a writer
of GGUF blobs holding a synthetic model whose bytes equal what brrr_model_open_synth generates
on the device for the same seed.

The data directory around a blob (config.txt, manifest.txt, tokens.bin) is the job of the
reference's own preparation scripts (scripts/setup_model.sh, gguf_index.py, dump_tokenizer.py);
this module writes none of it except tokens.bin for the toy vocabulary it defines itself.
"""
import struct

import numpy as np

PHI = np.uint64(0x9E3779B97F4A7C15)
L_GLOBAL = 0xFFFF
T = dict(ATTN_NORM=0, FFN_NORM=1, WQ=2, WK=3, WV=4, WO=5, BQ=6, BK=7, BV=8, BO=9, SINKS=10, ROUTER_W=11,
         ROUTER_B=12, GATE=13, UP=14, DOWN=15, GATE_B=16, UP_B=17, DOWN_B=18, Q_NORM=19, K_NORM=20, TOK_EMBD=32, OUT_NORM=33,
         OUTPUT=34, PROMPT=40, INPUT=41)

_old = np.seterr(over="ignore")


def mix64(z):
    z = np.asarray(z, dtype=np.uint64)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def tensor_key(seed, layer, kind):
    a = mix64(np.uint64(seed) + PHI)
    b = np.uint64((layer << 8) | kind) * PHI
    return mix64(a ^ b)


def draw(key, idx):
    idx = np.asarray(idx, dtype=np.uint64)
    return mix64(key + (idx + np.uint64(1)) * PHI)


def bytesum64(x):
    m1 = np.uint64(0x00FF00FF00FF00FF)
    m2 = np.uint64(0x0000FFFF0000FFFF)
    x = (x & m1) + ((x >> np.uint64(8)) & m1)
    x = (x & m2) + ((x >> np.uint64(16)) & m2)
    return ((x + (x >> np.uint64(32))) & np.uint64(0xFFFF)).astype(np.int32)


def normal(key, n):
    idx = np.arange(n, dtype=np.uint64)
    s = bytesum64(draw(key, idx * np.uint64(2))) + bytesum64(draw(key, idx * np.uint64(2) + np.uint64(1))) - 2040
    return s.astype(np.float32) * np.float32(0.0033829376)


def synth_f32(seed, layer, kind, n):
    mean = np.float32(1.0 if kind in (T["ATTN_NORM"], T["FFN_NORM"], T["OUT_NORM"], T["Q_NORM"], T["K_NORM"]) else 0.0)
    sigma = np.float32(1.0 if kind == T["SINKS"] else 0.02)
    z = normal(tensor_key(seed, layer, kind), n)
    return (z * sigma).astype(np.float32) + mean


def f32_to_bf16(v):
    b = np.asarray(v, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((b + np.uint64(0x7FFF) + ((b >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)) & np.uint64(0xFFFF)).astype(np.uint16)


def synth_bf16(seed, layer, kind, n):
    z = normal(tensor_key(seed, layer, kind), n)
    return f32_to_bf16((z * np.float32(0.02)).astype(np.float32))


def synth_mxfp4(seed, layer, kind, nblocks):
    key = tensor_key(seed, layer, kind)
    b = np.arange(nblocks, dtype=np.uint64)
    d0, d1, d2 = draw(key, b * np.uint64(3)), draw(key, b * np.uint64(3) + np.uint64(1)), draw(key, b * np.uint64(3) + np.uint64(2))
    out = np.empty((nblocks, 17), np.uint8)
    out[:, 0] = (np.uint64(117) + d2 % np.uint64(7)).astype(np.uint8)
    out[:, 1:9] = d0.view(np.uint8).reshape(nblocks, 8)      # little-endian bytes
    out[:, 9:17] = d1.view(np.uint8).reshape(nblocks, 8)
    return out.reshape(-1)


def synth_q4k_blocks(seed, layer, kind, nblocks):
    """numpy port of brrr_synth_q4k_block: uint8 [nblocks, 144]."""
    key = tensor_key(seed, layer, kind)
    b = np.arange(nblocks, dtype=np.uint64) * np.uint64(20)
    h = draw(key, b)
    k = (h & np.uint64(7)).astype(np.uint32)
    sub = ((h >> np.uint64(10)) & np.uint64(15)) == 0
    ms = np.uint32(64) + np.uint32(2) * ((h >> np.uint64(3)) & np.uint64(31)).astype(np.uint32)
    d = np.where(sub, ms, np.uint32(2 << 10) | (np.uint32(8) * k)).astype(np.uint16)
    dmin = np.where(sub, (ms * np.uint32(15)) >> np.uint32(1), np.uint32(4 << 10) | (np.uint32(896) + np.uint32(15) * k)).astype(np.uint16)
    out = np.empty((nblocks, 144), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nblocks, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(nblocks, 2)
    out[:, 4:8] = h.view(np.uint8).reshape(nblocks, 8)[:, 4:8]
    for j in range(17):
        out[:, 8 + 8 * j:16 + 8 * j] = draw(key, b + np.uint64(1 + j)).view(np.uint8).reshape(nblocks, 8)
    return out


def synth_q6k_blocks(seed, layer, kind, nblocks):
    """numpy port of brrr_synth_q6k_block: uint8 [nblocks, 210]."""
    key = tensor_key(seed, layer, kind)
    b = np.arange(nblocks, dtype=np.uint64) * np.uint64(27)
    out = np.empty((nblocks, 210), np.uint8)
    for j in range(26):
        out[:, 8 * j:8 * j + 8] = draw(key, b + np.uint64(j)).view(np.uint8).reshape(nblocks, 8)
    h = draw(key, b + np.uint64(26))
    d = (np.uint64(128) + (h & np.uint64(0x1ff))).astype(np.uint16)
    out[:, 208:210] = d.view(np.uint8).reshape(nblocks, 2)
    return out


def synth_prompt(seed, n, bound):
    key = tensor_key(seed, L_GLOBAL, T["PROMPT"])
    return (draw(key, np.arange(n, dtype=np.uint64)) % np.uint64(bound)).astype(np.uint32)


def synth_input(seed, n):
    """N(0,1)-like activation vector for stage tests."""
    return normal(tensor_key(seed, L_GLOBAL, T["INPUT"]), n)


# ---------------------------------------------------------------- data directory
_KIND_NAMES = {
    "ATTN_NORM": "attn_norm.weight", "FFN_NORM": "ffn_norm.weight", "WQ": "attn_q.weight", "WK": "attn_k.weight",
    "WV": "attn_v.weight", "WO": "attn_out.weight", "BQ": "attn_q.bias", "BK": "attn_k.bias", "BV": "attn_v.bias",
    "BO": "attn_out.bias", "SINKS": "attn_sinks", "ROUTER_W": "ffn_gate_inp.weight", "ROUTER_B": "ffn_gate_inp.bias",
    "GATE": "ffn_gate_exps.weight", "UP": "ffn_up_exps.weight", "DOWN": "ffn_down_exps.weight",
    "GATE_B": "ffn_gate_exps.bias", "UP_B": "ffn_up_exps.bias", "DOWN_B": "ffn_down_exps.bias",
}
GGML_F32, GGML_BF16, GGML_MXFP4 = 0, 30, 39


def model_tensors(cfg, seed):
    """Yield (name, ggml_type, ggml_dims, raw bytes) for every tensor of a synthetic gpt-oss model.
    ggml dims are innermost-first, as GGUF stores them."""
    d, nh, nkv, hd, ne, nl, nv = cfg.n_embd, cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.n_expert, cfg.n_layer, cfg.n_vocab
    for il in range(nl):
        def f32(kind, n, dims):
            return (f"blk.{il}.{_KIND_NAMES[kind]}", GGML_F32, dims, synth_f32(seed, il, T[kind], n).tobytes())

        def bf16(kind, rows, cols):
            return (f"blk.{il}.{_KIND_NAMES[kind]}", GGML_BF16, [cols, rows], synth_bf16(seed, il, T[kind], rows * cols).tobytes())

        def mx(kind):
            return (f"blk.{il}.{_KIND_NAMES[kind]}", GGML_MXFP4, [d, d, ne], synth_mxfp4(seed, il, T[kind], ne * d * (d // 32)).tobytes())

        yield f32("ATTN_NORM", d, [d]); yield f32("FFN_NORM", d, [d])
        yield bf16("WQ", nh * hd, d); yield bf16("WK", nkv * hd, d); yield bf16("WV", nkv * hd, d); yield bf16("WO", d, nh * hd)
        yield f32("BQ", nh * hd, [nh * hd]); yield f32("BK", nkv * hd, [nkv * hd]); yield f32("BV", nkv * hd, [nkv * hd]); yield f32("BO", d, [d])
        yield f32("SINKS", nh, [nh])
        yield f32("ROUTER_W", ne * d, [d, ne]); yield f32("ROUTER_B", ne, [ne])
        yield mx("GATE"); yield mx("UP"); yield mx("DOWN")
        yield f32("GATE_B", ne * d, [d, ne]); yield f32("UP_B", ne * d, [d, ne]); yield f32("DOWN_B", ne * d, [d, ne])
    yield ("token_embd.weight", GGML_BF16, [d, nv], synth_bf16(seed, L_GLOBAL, T["TOK_EMBD"], nv * d).tobytes())
    yield ("output_norm.weight", GGML_F32, [d], synth_f32(seed, L_GLOBAL, T["OUT_NORM"], d).tobytes())
    yield ("output.weight", GGML_BF16, [d, nv], synth_bf16(seed, L_GLOBAL, T["OUTPUT"], nv * d).tobytes())


GGML_Q4_K, GGML_Q6_K = 12, 14


def qwen_model_tensors(cfg, seed, ktypes=None):
    """(name, ggml type, dims, raw bytes) of a synthetic qwen3moe model, in the tensor names the
    reference's loader looks up (src/bin/engine_qwen2.rs:528-541).  Down experts and the output head
    are Q6_K, every other matrix Q4_K; `ktypes` maps tensor names to another K-quant type (files
    in the wild mix the two per tensor, e.g. attn_v stored as Q6_K)."""
    ktypes = ktypes or {}
    d, nh, nkv, hd, ne, ff, nv = cfg.n_embd, cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.n_expert, cfg.n_ff_exp, cfg.n_vocab

    def k(name, layer, kind, rows, cols, dims):
        ty = ktypes.get(name, GGML_Q6_K if kind in ("DOWN", "OUTPUT") else GGML_Q4_K)
        if ty == GGML_Q6_K:
            return (name, GGML_Q6_K, dims, synth_q6k_blocks(seed, layer, T[kind], rows * cols // 256).tobytes())
        return (name, GGML_Q4_K, dims, synth_q4k_blocks(seed, layer, T[kind], rows * cols // 256).tobytes())

    for il in range(cfg.n_layer):
        p = f"blk.{il}."
        yield (p + "attn_norm.weight", GGML_F32, [d], synth_f32(seed, il, T["ATTN_NORM"], d).tobytes())
        yield (p + "ffn_norm.weight", GGML_F32, [d], synth_f32(seed, il, T["FFN_NORM"], d).tobytes())
        yield (p + "attn_q_norm.weight", GGML_F32, [hd], synth_f32(seed, il, T["Q_NORM"], hd).tobytes())
        yield (p + "attn_k_norm.weight", GGML_F32, [hd], synth_f32(seed, il, T["K_NORM"], hd).tobytes())
        yield k(p + "attn_q.weight", il, "WQ", nh * hd, d, [d, nh * hd])
        yield k(p + "attn_k.weight", il, "WK", nkv * hd, d, [d, nkv * hd])
        yield k(p + "attn_v.weight", il, "WV", nkv * hd, d, [d, nkv * hd])
        yield k(p + "attn_output.weight", il, "WO", d, nh * hd, [nh * hd, d])
        yield (p + "ffn_gate_inp.weight", GGML_F32, [d, ne], synth_f32(seed, il, T["ROUTER_W"], ne * d).tobytes())
        yield k(p + "ffn_gate_exps.weight", il, "GATE", ne * ff, d, [d, ff, ne])
        yield k(p + "ffn_up_exps.weight", il, "UP", ne * ff, d, [d, ff, ne])
        yield k(p + "ffn_down_exps.weight", il, "DOWN", ne * d, ff, [ff, d, ne])
    yield k("token_embd.weight", L_GLOBAL, "TOK_EMBD", nv, d, [d, nv])
    yield ("output_norm.weight", GGML_F32, [d], synth_f32(seed, L_GLOBAL, T["OUT_NORM"], d).tobytes())
    yield k("output.weight", L_GLOBAL, "OUTPUT", nv, d, [d, nv])


def _gguf_str(s):
    b = s.encode() if isinstance(s, str) else s
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, cfg, seed, tokens=None, arch="gpt-oss", ktypes=None):
    """Write a GGUF v3 file by hand (little-endian, alignment 32): header, metadata key/values
    (the hyper-parameters setup_model.sh looks up, and the token list), tensor infos, data."""
    kv = []

    def kv_u32(k, v): kv.append(_gguf_str(k) + struct.pack("<II", 4, v))
    def kv_f32(k, v): kv.append(_gguf_str(k) + struct.pack("<If", 6, v))
    def kv_str(k, v): kv.append(_gguf_str(k) + struct.pack("<I", 8) + _gguf_str(v))

    kv_str("general.architecture", arch)
    kv_u32("general.alignment", 32)
    kv_u32(f"{arch}.embedding_length", cfg.n_embd)
    kv_u32(f"{arch}.block_count", cfg.n_layer)
    kv_u32(f"{arch}.attention.head_count", cfg.n_head)
    kv_u32(f"{arch}.attention.head_count_kv", cfg.n_head_kv)
    kv_u32(f"{arch}.attention.key_length", cfg.head_dim)
    kv_u32(f"{arch}.expert_count", cfg.n_expert)
    kv_u32(f"{arch}.expert_used_count", cfg.n_expert_used)
    kv_u32(f"{arch}.expert_feed_forward_length", cfg.n_ff_exp)
    if hasattr(cfg, "sliding_window"):
        kv_u32(f"{arch}.attention.sliding_window", cfg.sliding_window)
    kv_f32(f"{arch}.rope.freq_base", cfg.rope_freq_base)
    kv_f32(f"{arch}.attention.layer_norm_rms_epsilon", cfg.rms_eps)
    kv_u32(f"{arch}.vocab_size", cfg.n_vocab)
    kv_u32(f"{arch}.context_length", 4096)
    if tokens is None:
        tokens = default_tokens(cfg.n_vocab, arch)
    arr = struct.pack("<IQ", 8, len(tokens)) + b"".join(_gguf_str(t) for t in tokens)
    kv.append(_gguf_str("tokenizer.ggml.tokens") + struct.pack("<I", 9) + arr)

    tensors = list(qwen_model_tensors(cfg, seed, ktypes) if arch == "qwen3moe" else model_tensors(cfg, seed))
    infos, off = [], 0
    for name, ty, dims, raw in tensors:
        infos.append(_gguf_str(name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims) + struct.pack("<IQ", ty, off))
        off = (off + len(raw) + 31) // 32 * 32
    head = b"GGUF" + struct.pack("<I", 3) + struct.pack("<QQ", len(tensors), len(kv)) + b"".join(kv) + b"".join(infos)
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * ((len(head) + 31) // 32 * 32 - len(head)))
        for name, ty, dims, raw in tensors:
            f.write(raw)
            f.write(b"\0" * ((len(raw) + 31) // 32 * 32 - len(raw)))


def _byte_spelling():
    """GPT-2's byte-level spelling used by GGUF token lists: printable Latin-1 bytes stand for
    themselves, the other 68 byte values are written as U+0100, U+0101, ... in ascending byte order."""
    keep = set(range(0x21, 0x7F)) | set(range(0xA1, 0xAD)) | set(range(0xAE, 0x100))
    table, extra = [], 0
    for b in range(256):
        if b in keep:
            table.append(chr(b))
        else:
            table.append(chr(0x100 + extra))
            extra += 1
    return table


_SPECIALS = {"gpt-oss": (b"<|start|>", b"<|end|>", b"<|message|>", b"<|return|>"),
             "qwen3moe": (b"<|endoftext|>", b"<|im_start|>", b"<|im_end|>", b"<|fim_pad|>")}


def raw_tokens(n_vocab, arch="gpt-oss"):
    """Toy vocabulary as the raw byte strings tokens.bin holds: the 256 single bytes, then short
    words "w0", "w1", ...; the last four entries are special tokens of the architecture's chat
    format (spelled with '<|', which the engine's lookup skips)."""
    toks = [bytes([b]) for b in range(256)]
    i = 0
    while len(toks) < n_vocab - 4:
        toks.append(f"w{i}".encode())
        i += 1
    for s in _SPECIALS[arch]:
        if len(toks) < n_vocab:
            toks.append(s)
    return toks[:n_vocab]


def default_tokens(n_vocab, arch="gpt-oss"):
    """The toy vocabulary in its GGUF spelling (UTF-8 of the byte-level characters; special tokens
    literal)."""
    sp = _byte_spelling()
    return [t if t.startswith(b"<|") else "".join(sp[b] for b in t).encode("utf-8") for t in raw_tokens(n_vocab, arch)]


def write_tokens_bin(path, toks):
    """tokens.bin as the engine reads it (src/bin/engine_gpt2.rs:1260-1266): u32 count, then per
    token a u16 length and the raw bytes."""
    with open(path, "wb") as f:
        f.write(struct.pack("<I", len(toks)))
        for t in toks:
            f.write(struct.pack("<H", len(t)) + t)


# ---- K-quant test tensors (qwen3moe path) ------------------------------------------------------

def _f16_bits(v):
    return np.asarray(v, dtype=np.float16).view(np.uint16)


def synth_q4k(seed, rows, cols):
    """Random but well-formed Q4_K rows in the GGUF byte layout (144 B per 256 values: f16 d, f16 dmin,
    12 B of packed 6-bit scales/mins, 128 B of nibbles).  Returns uint8 [rows, cols/256*144]."""
    rng = np.random.default_rng(seed)
    nsb = cols // 256
    out = np.empty((rows, nsb, 144), np.uint8)
    d = rng.uniform(2e-4, 2e-3, size=(rows, nsb)).astype(np.float32)
    dmin = rng.uniform(2e-4, 2e-3, size=(rows, nsb)).astype(np.float32)
    out[:, :, 0:2] = _f16_bits(d)[..., None].view(np.uint8).reshape(rows, nsb, 2)
    out[:, :, 2:4] = _f16_bits(dmin)[..., None].view(np.uint8).reshape(rows, nsb, 2)
    out[:, :, 4:144] = rng.integers(0, 256, size=(rows, nsb, 140), dtype=np.uint8)
    return out.reshape(rows, nsb * 144)


def synth_q6k(seed, rows, cols):
    """Random but well-formed Q6_K rows (210 B per 256 values: 128 B low nibbles, 64 B high 2-bit
    fields, 16 int8 scales, f16 d).  Returns uint8 [rows, cols/256*210]."""
    rng = np.random.default_rng(seed)
    nsb = cols // 256
    out = np.empty((rows, nsb, 210), np.uint8)
    out[:, :, 0:192] = rng.integers(0, 256, size=(rows, nsb, 192), dtype=np.uint8)
    out[:, :, 192:208] = rng.integers(-128, 128, size=(rows, nsb, 16), dtype=np.int8).view(np.uint8)
    d = rng.uniform(1e-5, 1e-4, size=(rows, nsb)).astype(np.float32)
    out[:, :, 208:210] = _f16_bits(d)[..., None].view(np.uint8).reshape(rows, nsb, 2)
    return out.reshape(rows, nsb * 210)


def synth_activation(seed, n, scale=1.0):
    """Seeded normal activations with a few outliers, float32 [n]."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(n).astype(np.float32) * np.float32(scale)
    x[rng.integers(0, n, size=max(1, n // 97))] *= np.float32(7.5)
    return x
