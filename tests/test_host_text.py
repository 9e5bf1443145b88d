"""Host text layer (tokenizer, sampler, chat prompt, serve line parser) of libbrrr.so against the
pure-Python restatement of the reference (oracle/oracle_host.py).  Host code only: runs without a GPU."""
import ctypes as C
import os

import numpy as np
import pytest

from cpubrrr_b200 import synth as S


@pytest.fixture(scope="module")
def L(brrr):
    return brrr.lib()


@pytest.fixture(scope="module")
def tokdir(tmp_path_factory):
    """tokens.bin of a toy vocabulary: 256 bytes, short words, duplicates, long pieces, specials."""
    d = tmp_path_factory.mktemp("tok")
    toks = S.raw_tokens(700)             # raw bytes, as tokens.bin holds them
    toks[300] = toks[65]                 # duplicate of a byte token: the lower id must win
    toks[301] = b"hello"
    toks[302] = b"hello world"
    toks[303] = b"x" * 40                # longer than the 32-byte window of the gpt-oss engine
    toks[304] = b""
    toks[305] = b"<|custom|>"
    import struct
    with open(d / "tokens.bin", "wb") as f:
        f.write(struct.pack("<I", len(toks)))
        for t in toks:
            f.write(struct.pack("<H", len(t))); f.write(t)
    return str(d)


def _open(L, tokdir):
    h = C.c_void_p()
    assert L.brrr_tokenizer_open(tokdir.encode(), C.byref(h)) == 0
    return h


def _encode(L, h, text, max_piece=32):
    b = text.encode() if isinstance(text, str) else text
    n = C.c_size_t()
    st = L.brrr_tokenizer_encode(h, b, len(b), max_piece, None, 0, C.byref(n))
    if st != 0:
        return st
    out = np.zeros(max(n.value, 1), np.uint32)
    assert L.brrr_tokenizer_encode(h, b, len(b), max_piece, out.ctypes.data, n.value, C.byref(n)) == 0
    return [int(v) for v in out[:n.value]]


def test_tokenizer_matches_reference_rules(L, orc, tokdir):
    from oracle import oracle_host as H
    h = _open(L, tokdir)
    toks = H.load_tokens(os.path.join(tokdir, "tokens.bin"))
    lookup = H.make_lookup(toks)
    assert L.brrr_tokenizer_size(h) == len(toks) == 700
    for text in ["hello world!", "hellohello worldhello w", "A" * 5 + "x" * 45, "w12 w3w44", "tab\tnew\nline", ""]:
        assert _encode(L, h, text) == H.encode(lookup, text)
        assert _encode(L, h, text, 48) == H.encode(lookup, text, 48)
    assert _encode(L, h, "A") == [65] and toks[300] == toks[65]      # duplicate byte string: the first id wins
    assert _encode(L, h, "x" * 40, 48) == [303] and len(_encode(L, h, "x" * 40, 32)) > 1
    sid = C.c_uint32()
    assert L.brrr_tokenizer_special(h, b"<|custom|>", C.byref(sid)) == 0 and sid.value == 305
    assert L.brrr_tokenizer_special(h, b"<|nope|>", C.byref(sid)) == 5
    assert _encode(L, h, "<|custom|>") == H.encode(lookup, "<|custom|>")    # specials are never matched as text
    p, n = C.c_char_p(), C.c_uint32()
    assert L.brrr_tokenizer_token(h, 302, C.byref(p), C.byref(n)) == 0 and C.string_at(p, n.value) == b"hello world"
    assert L.brrr_tokenizer_token(h, 700, C.byref(p), C.byref(n)) == 5
    L.brrr_tokenizer_close(h)
    bad = C.c_void_p()
    assert L.brrr_tokenizer_open(b"/nonexistent-dir", C.byref(bad)) == 2


def test_unencodable_byte_is_an_error(L, tmp_path):
    import struct
    with open(tmp_path / "tokens.bin", "wb") as f:
        f.write(struct.pack("<I", 2))
        for t in (b"a", b"b"):
            f.write(struct.pack("<H", len(t))); f.write(t)
    h = _open(L, str(tmp_path))
    assert _encode(L, h, "abba") == [0, 1, 1, 0]
    assert _encode(L, h, "abc") == 5
    L.brrr_tokenizer_close(h)


def test_sampler_matches_reference(L, orc):
    from oracle import oracle_host as H
    rng = np.random.default_rng(3)
    logits = (rng.standard_normal(5000) * 3).astype(np.float32)
    logits[100] = logits[4000] = logits.max() + 1          # tie at the top
    lp = logits.ctypes.data_as(C.c_void_p)
    assert L.brrr_sample_logits(lp, logits.size, 0, 40, None) == 100 == H.sample_logits(logits, 0, 40, 1)[0]
    for seed in (0, 1, 12345):
        st_o = H.rng_seed(seed)
        assert L.brrr_rng_seed(seed) == st_o and st_o & 1
        st = C.c_uint64(st_o)
        for temp_milli, k in ((700, 40), (1500, 64), (100, 1), (2000, 500), (900, 0)):
            for _ in range(6):
                want, st_o = H.sample_logits(logits, temp_milli, k, st_o)
                got = L.brrr_sample_logits(lp, logits.size, temp_milli, k, C.byref(st))
                assert got == want and st.value == st_o
    few = np.array([0.5, 0.25, 0.5], np.float32)            # fewer logits than k; equal values: the later index is listed first
    st = C.c_uint64(H.rng_seed(9)); st_o = H.rng_seed(9)
    for _ in range(20):
        want, st_o = H.sample_logits(few, 1000, 40, st_o)
        assert L.brrr_sample_logits(few.ctypes.data_as(C.c_void_p), 3, 1000, 40, C.byref(st)) == want


def test_serve_line_parser(L, orc):
    from oracle import oracle_host as H
    buf = C.create_string_buffer(4096)
    cases = ["Why is the sky blue?", "0.7\t42\t128\tTell me\\na story\\twith tabs \\\\ and \\q", "  padded prompt  \n",
             "abc\t1\t2\tnot a number first", "0.5\t-3\t10\tnegative seed", "-1.5\t7\t0\tclamped", "1\t2\t99999\tbig", "a\tb\tc"]
    for line in cases:
        temp, seed, ngen = C.c_float(), C.c_uint64(), C.c_uint32()
        form = L.brrr_serve_parse(line.encode(), C.byref(temp), C.byref(seed), C.byref(ngen), buf, 4096)
        tsv, t_o, s_o, n_o, p_o = H.serve_parse(line)
        assert form == int(tsv), line
        assert buf.value.decode() == p_o, line
        if tsv:
            assert abs(temp.value - t_o) < 1e-6 and seed.value == s_o and ngen.value == n_o


def test_chat_prompt_ids(L, orc, tokdir):
    from oracle import oracle_host as H
    h = _open(L, tokdir)
    lookup = H.make_lookup(H.load_tokens(os.path.join(tokdir, "tokens.bin")))
    n = C.c_size_t()
    text = "hello world, w5?"
    assert L.brrr_chat_prompt(h, text.encode(), None, 0, C.byref(n)) == 0
    out = np.zeros(n.value, np.uint32)
    assert L.brrr_chat_prompt(h, text.encode(), out.ctypes.data, n.value, C.byref(n)) == 0
    assert [int(v) for v in out] == H.chat_prompt(lookup, text)
    assert L.brrr_chat_prompt(h, text.encode(), out.ctypes.data, 3, C.byref(n)) == 5
    L.brrr_tokenizer_close(h)


# ---- qwen3moe host layer ----------------------------------------------------------------------------

@pytest.fixture(scope="module")
def qtokdir(tmp_path_factory):
    """tokens.bin of the qwen toy vocabulary (ChatML special tokens at the end) with a few long pieces."""
    d = tmp_path_factory.mktemp("qtok")
    toks = S.raw_tokens(700, "qwen3moe")
    toks[300] = b"You are a helpful assistant."
    toks[301] = b"\nuser\n"
    toks[302] = b"y" * 45                # inside the 48-byte window of this engine, beyond the 32 of the other
    toks[303] = b"z" * 50                # beyond it
    S.write_tokens_bin(str(d / "tokens.bin"), toks)
    return str(d)


def test_qwen_chat_prompt_matches_reference_restatement(L, qtokdir):
    from oracle import oracle_host as H
    toks = H.load_tokens(os.path.join(qtokdir, "tokens.bin"))
    h = _open(L, qtokdir)
    for text in ["Write a haiku about CPUs.", "y" * 45 + " and " + "z" * 50, "", "tabs\tand\nnewlines w12 w13"]:
        n = C.c_size_t()
        assert L.brrr_qwen_chat_prompt(h, text.encode(), None, 0, C.byref(n)) == 0
        ids = np.zeros(n.value, np.uint32)
        assert L.brrr_qwen_chat_prompt(h, text.encode(), ids.ctypes.data, n.value, C.byref(n)) == 0
        want = H.qwen_chat_prompt(toks, text)
        assert ids.tolist() == want
        assert ids[0] == len(toks) - 3 and want.count(len(toks) - 2) == 2          # im_start first, two im_end
    assert 302 in H.qwen_chat_prompt(toks, "y" * 45)                                  # the 45-byte piece is found in one step
    L.brrr_tokenizer_close(h)


def test_qwen_chat_prompt_needs_the_chatml_tokens(L, tokdir):
    h = _open(L, tokdir)                 # the gpt-oss toy vocabulary has no <|im_start|>
    n = C.c_size_t()
    assert L.brrr_qwen_chat_prompt(h, b"hi", None, 0, C.byref(n)) == 2
    L.brrr_tokenizer_close(h)


def test_qwen_serve_parse(L):
    from oracle import oracle_host as H
    lines = ["  hello there  \n", "\n", "   ", "0.7\t5\t12\tline one\\nline two\\tend\n", "x\ty\t7\tnot validated\n", "0\t1\tseven\ta b\n",
             "0\t1\t+9\tplus\n", "a\tb\tc\n", "0\t1\t99999\tbig\n", "0\t1\t3\ttabs\tin\tprompt\\\\n\n"]
    for line in lines:
        ngen = C.c_uint32(0)
        buf = C.create_string_buffer(256)
        form = L.brrr_qwen_serve_parse(line.encode(), C.byref(ngen), buf, 256)
        want = H.qwen_serve_parse(line)
        if want is None:
            assert form == -1
            continue
        assert form == int(want[0]) and buf.value.decode() == want[2], line
        if want[0]:
            assert ngen.value == want[1]
