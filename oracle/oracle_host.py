"""TEST INFRASTRUCTURE — pure-Python restatement of the reference's host text layer (small cases
only): tokenizer set-up and greedy longest-match encode (src/bin/engine_gpt2.rs:1261-1274),
sample_logits (82-126) with the oracle's exp, the harmony chat prompt (1401-1414) and the serve
line parser (1454-1482).  Only tests import this module."""
import struct

import numpy as np

from . import oracle as O

SYSTEM = ("You are ChatGPT, a large language model trained by OpenAI.\nKnowledge cutoff: 2024-06\nCurrent date: 2026-07-03\n\n"
          "Reasoning: low\n\n# Valid channels: analysis, commentary, final. Channel must be included for every message.")


def load_tokens(path):
    tb = open(path, "rb").read()
    (n,) = struct.unpack_from("<I", tb, 0)
    toks, p = [], 4
    for _ in range(n):
        (l,) = struct.unpack_from("<H", tb, p)
        toks.append(tb[p + 2:p + 2 + l])
        p += 2 + l
    return toks


def make_lookup(toks):
    lookup = {}
    for i, t in enumerate(toks):
        if t and not t.startswith(b"<|"):
            lookup.setdefault(t, i)
    return lookup


def encode(lookup, text, max_piece=32):
    b = text if isinstance(text, bytes) else text.encode()
    ids, i = [], 0
    while i < len(b):
        l = min(len(b) - i, max_piece)
        while True:
            assert l > 0, f"unencodable byte {b[i]}"
            if b[i:i + l] in lookup:
                ids.append(lookup[b[i:i + l]]); i += l
                break
            l -= 1
    return ids


def chat_prompt(lookup, user_text):
    ids = [200006] + encode(lookup, "system") + [200008] + encode(lookup, SYSTEM) + [200007]
    ids += [200006] + encode(lookup, "user") + [200008] + encode(lookup, user_text) + [200007]
    ids += [200006] + encode(lookup, "assistant")
    return ids


def rng_seed(seed):
    M = (1 << 64) - 1
    z = (seed + 0x9E3779B97F4A7C15) & M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
    return (z ^ (z >> 31)) | 1


def rng_next(state):
    M = (1 << 64) - 1
    x = state
    x ^= (x << 13) & M
    x ^= x >> 7
    x ^= (x << 17) & M
    return x


def sample_logits(logits, temp_milli, top_k, state):
    """Returns (token, new rng state)."""
    logits = np.asarray(logits, np.float32)
    if temp_milli == 0:
        return int(np.argmax(logits)), state           # argmax returns the first maximum
    temp = np.float32(temp_milli) / np.float32(1000.0)
    k = min(max(top_k, 1), 64)
    top = []
    for i, l in enumerate(logits):
        if len(top) < k or l > top[-1][0]:
            pos = 0
            while pos < len(top) and top[pos][0] > l:
                pos += 1
            top.insert(pos, (l, i))
            if len(top) > k:
                top.pop()
    mx = top[0][0]
    probs = [O.expf(np.float32((l - mx) / temp)).item() for l, _ in top]
    s = np.float32(0.0)
    for p in probs:
        s = np.float32(s + np.float32(p))
    probs = [np.float32(np.float32(p) / s) for p in probs]
    state = rng_next(state)
    r = np.float32(np.float32(state >> 11) / np.float32(1 << 53))
    acc = np.float32(0.0)
    for p, (_, idx) in zip(probs, top):
        acc = np.float32(acc + p)
        if r <= acc:
            return idx, state
    return top[-1][1], state


def serve_parse(line):
    """(is_tsv, temp, seed, ngen, prompt)"""
    pline = line.strip()
    parts = pline.split("\t", 3)
    if len(parts) == 4:
        try:
            temp, seed, ngen = float(parts[0]), int(parts[1]), int(parts[2])
            if seed < 0 or ngen < 0:
                raise ValueError
        except ValueError:
            return False, 0.0, 0, 0, pline
        out, it = [], iter(parts[3])
        for ch in it:
            if ch == "\\":
                o = next(it, None)
                out.append({"n": "\n", "t": "\t", "\\": "\\"}.get(o, "\\" + o) if o is not None else "\\")
            else:
                out.append(ch)
        return True, max(temp, 0.0), seed, min(max(ngen, 1), 4096), "".join(out)
    return False, 0.0, 0, 0, pline


# ---- qwen3moe host layer (src/bin/engine_qwen2.rs:493-507, 622-683) ---------------------------------

def special_ids(toks):
    """Literal spelling -> id of the tokens that start with '<|' (the reference's `spm` map; the last one wins)."""
    return {t: i for i, t in enumerate(toks) if t.startswith(b"<|")}


def qwen_chat_prompt(toks, user_text):
    """ChatML prompt ids; text pieces use the 48-byte encode window (engine_qwen2.rs:500-505, 627-631)."""
    lookup, spm = make_lookup(toks), special_ids(toks)
    im_start, im_end = spm[b"<|im_start|>"], spm[b"<|im_end|>"]
    ids = [im_start] + encode(lookup, "system\nYou are a helpful assistant.", 48) + [im_end]
    ids += [im_start] + encode(lookup, "\nuser\n" + user_text, 48) + [im_end]
    ids += [im_start] + encode(lookup, "\nassistant\n", 48)
    return ids


def qwen_serve_parse(line):
    """(is_tsv, ngen or None, prompt) of one request line, None for an empty one (engine_qwen2.rs:659-673):
    temp and seed fields are not even parsed; "\\n" and "\\t" in the prompt become spaces."""
    ptext = line.strip()
    if not ptext:
        return None
    parts = ptext.split("\t", 3)
    if len(parts) == 4:
        f = parts[2]
        digits = f[1:] if f.startswith("+") else f
        if digits.isascii() and digits.isdigit():
            return True, min(int(digits), 4096), parts[3].replace("\\n", " ").replace("\\t", " ")
    return False, None, ptext


def qwen_generate(run, toks, ids, ngen):
    """Greedy generation as the reference's generate closure: token-by-token prefill, stop on <|im_end|>
    or an id beyond the vocabulary file; returns the produced ids."""
    im_end, ntok = special_ids(toks)[b"<|im_end|>"], len(toks)
    nxt = 0
    for i, t in enumerate(ids):
        nxt = run(t, i, True)
    pos, out = len(ids), []
    for _ in range(ngen):
        if nxt == im_end or nxt >= ntok:
            break
        out.append(nxt)
        nxt = run(nxt, pos, True)
        pos += 1
    return out
