"""generate() and the command-line front end on the GPU against the oracle: greedy bursts cut at a
stop token, sampled decoding through host logits, and the serve protocol of the engine binary."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from cpubrrr_b200 import synth as S

pytestmark = pytest.mark.gpu


class Stats(C.Structure):
    _fields_ = [("prefill_tokens", C.c_uint32), ("decode_tokens", C.c_uint32), ("prefill_seconds", C.c_double), ("decode_seconds", C.c_double)]


def ocfg_of(orc, c):
    return orc.make_cfg(d=c.n_embd, nh=c.n_head, nkv=c.n_head_kv, hd=c.head_dim, nl=c.n_layer, ne=c.n_expert,
                        topk=c.n_expert_used, nvocab=c.n_vocab, swa=c.sliding_window, rope_base=c.rope_freq_base, rms_eps=c.rms_eps)


def oracle_generate(orc, om, ids, ngen, temp_milli=0, top_k=40, state=0, stop=(200002, 199999)):
    from oracle import oracle_host as H
    nxt = 0
    for i, t in enumerate(ids):
        nxt = om.run(int(t), i, i == len(ids) - 1)
    if temp_milli:
        nxt, state = H.sample_logits(om.logits(), temp_milli, top_k, state)
    out, pos = [], len(ids)
    for _ in range(ngen):
        if nxt in stop or pos + 1 >= 4096:
            break
        out.append(nxt)
        g = om.run(nxt, pos, True)
        nxt = g
        if temp_milli:
            nxt, state = H.sample_logits(om.logits(), temp_milli, top_k, state)
        pos += 1
    return out


def run_generate(brrr, eng, ids, ngen, temp_milli=0, top_k=40, state=0):
    L = brrr.lib()
    ids = np.ascontiguousarray(ids, np.uint32)
    out = np.zeros(ngen + 1, np.uint32)
    st = Stats()
    rng = C.c_uint64(state)
    assert L.brrr_generate(eng._h, None, ids.ctypes.data, ids.size, ngen, temp_milli, top_k, C.byref(rng) if temp_milli else None,
                           None, None, out.ctypes.data, out.size, C.byref(st)) == 0
    assert st.prefill_tokens == ids.size
    return [int(t) for t in out[:st.decode_tokens]]


def test_generate_greedy_bursts_equal_oracle(brrr, orc):
    cfg = brrr.make_cfg(128, 2, 4, 2, 8, 4, 512, sliding_window=16)
    eng = brrr.Engine.synth(cfg, 23)
    om = orc.Model.synth(ocfg_of(orc, cfg), 23)
    prompt = S.synth_prompt(23, 12, 512)
    for ngen in (1, 31, 32, 33, 100):          # around the 32-token burst size
        assert run_generate(brrr, eng, prompt, ngen) == oracle_generate(orc, om, prompt, ngen)
    eng.close()


def test_generate_stops_at_the_context_limit(brrr, orc):
    """A prompt that ends 6 positions before the 4096-token context: both sides stop by the
    position rule (pos + 1 >= MAXSEQ), after the same tokens."""
    cfg = brrr.make_cfg(64, 1, 2, 1, 4, 2, 256, sliding_window=16)
    eng = brrr.Engine.synth(cfg, 29)
    om = orc.Model.synth(ocfg_of(orc, cfg), 29)
    prompt = S.synth_prompt(29, 4090, 256)
    want = oracle_generate(orc, om, prompt, 50)
    assert 0 < len(want) < 50
    assert run_generate(brrr, eng, prompt, 50) == want
    eng.close()


def test_generate_sampled_equals_oracle(brrr, orc):
    from oracle import oracle_host as H
    cfg = brrr.make_cfg(128, 2, 4, 2, 8, 4, 512, sliding_window=16)
    eng = brrr.Engine.synth(cfg, 31)
    om = orc.Model.synth(ocfg_of(orc, cfg), 31)
    prompt = S.synth_prompt(31, 7, 512)
    for temp_milli, k, seed in ((800, 40, 5), (1500, 8, 6)):
        st = H.rng_seed(seed)
        want = oracle_generate(orc, om, prompt, 24, temp_milli, k, st)
        assert run_generate(brrr, eng, prompt, 24, temp_milli, k, st) == want
        assert len(set(want)) > 4
    eng.close()


def test_engine_binary_serve_protocol(brrr, orc, tmp_path):
    """brrr_engine <data-dir> <blob> --serve on a synthetic gpt-oss data directory whose vocabulary
    contains the harmony special ids: [READY], streamed bytes, [STATS] and [DONE] lines; the token
    count and text equal what the oracle generates for the same prompt ids."""
    from oracle import oracle_host as H
    import refdata
    cfg, d, blob = refdata.case_data_dir(str(tmp_path / "m"), "gptoss_serve", 37)
    exe = os.path.join(os.path.dirname(brrr.__file__), "brrr_engine")
    req = "What is 2+2?\n0\t1\t5\tw3 w4\\nw5\n"
    r = subprocess.run([exe, d, blob, "--serve"], input=req.encode(), capture_output=True, timeout=300)
    assert r.returncode == 0, r.stderr.decode()
    assert b"[READY]" in r.stderr
    out = r.stdout.decode("utf-8", "replace")
    assert out.count("[DONE]") == 2 and out.count("[STATS]") == 2
    toks = H.load_tokens(os.path.join(d, "tokens.bin"))
    lookup = H.make_lookup(toks)
    om = orc.Model.open(d, blob)
    first, second = out.split("[DONE]\n")[:2]
    for text, ngen, chunk in (("What is 2+2?", 256, first), ("w3 w4\nw5", 5, second)):
        ids = H.chat_prompt(lookup, text)
        want = oracle_generate(orc, om, ids, ngen)
        body, stats = chunk.rsplit("\n[STATS] ", 1)
        assert f"prefill_tok={len(ids)} " in stats and f"decode_tok={len(want)} " in stats
        assert body.encode("utf-8", "replace") == b"".join(toks[t] for t in want).decode("utf-8", "replace").encode("utf-8", "replace")


# ---- qwen3moe: ChatML generate, the engine binary, and the reference's own HTTP front end -----------

def test_qwen_generate_and_binary_serve_protocol(brrr, orc, tmp_path):
    """brrr_qwen_generate and `brrr_engine_qwen <data-dir> <blob> --serve` on a synthetic qwen3moe data
    directory whose vocabulary holds the ChatML special tokens: prompt ids, produced ids, streamed text and
    the [STATS] / [DONE] lines equal what the oracle generates (src/bin/engine_qwen2.rs:622-683: greedy
    only, stop on <|im_end|>, prefill_tok=0 in the stats line, escapes of a TSV prompt become spaces)."""
    import refdata
    from oracle import oracle_host as H
    cfg, d, blob = refdata.case_data_dir(str(tmp_path / "q"), "qwen_d256", 41)
    toks = H.load_tokens(os.path.join(d, "tokens.bin"))
    om = orc.QwenModel.open(d, blob)
    L = brrr.lib()
    tok = C.c_void_p()
    assert L.brrr_tokenizer_open(d.encode(), C.byref(tok)) == 0
    eng = brrr.QwenEngine.open(d, blob)
    for text, ngen in (("w1 w2 w3", 40), ("Write a haiku about CPUs.", 33)):
        n = C.c_size_t()
        assert L.brrr_qwen_chat_prompt(tok, text.encode(), None, 0, C.byref(n)) == 0
        ids = np.zeros(n.value, np.uint32)
        assert L.brrr_qwen_chat_prompt(tok, text.encode(), ids.ctypes.data, n.value, C.byref(n)) == 0
        assert ids.tolist() == H.qwen_chat_prompt(toks, text)
        want = H.qwen_generate(om.run, toks, ids.tolist(), ngen)
        out = np.zeros(ngen + 1, np.uint32)
        st = Stats()
        assert L.brrr_qwen_generate(eng._h, tok, ids.ctypes.data, ids.size, ngen, None, None, out.ctypes.data, out.size, C.byref(st)) == 0
        assert [int(t) for t in out[:st.decode_tokens]] == want and st.prefill_tokens == ids.size
    eng.close()
    L.brrr_tokenizer_close(tok)
    exe = os.path.join(os.path.dirname(brrr.__file__), "brrr_engine_qwen")
    req = "w1 w2 w3\n0.8\t7\t5\tw3 w4\\nw5\n"
    r = subprocess.run([exe, d, blob, "--serve", "24"], input=req.encode(), capture_output=True, timeout=300)
    assert r.returncode == 0, r.stderr.decode()
    assert b"[READY]" in r.stderr
    out = r.stdout.decode("utf-8", "replace")
    assert out.count("[DONE]") == 2 and out.count("[STATS]") == 2
    first, second = out.split("[DONE]\n")[:2]
    for text, ngen, chunk in (("w1 w2 w3", 24, first), ("w3 w4 w5", 5, second)):
        want = H.qwen_generate(om.run, toks, H.qwen_chat_prompt(toks, text), ngen)
        body, stats = chunk.rsplit("\n[STATS] ", 1)
        assert "prefill_tok=0 " in stats and f"decode_tok={len(want)} " in stats
        assert body.encode("utf-8", "replace") == b"".join(toks[t] for t in want).decode("utf-8", "replace").encode("utf-8", "replace")
    om.close()


def test_reference_openai_server_drives_the_engine_binaries(brrr, orc, tmp_path):
    """The reference's own HTTP front end (scripts/openai_server.py, class Engine, lines 34-90) spawns an
    engine binary with `<data-dir> <blob> --serve` and talks to it over the pipe.  Here it is imported
    unmodified from the reference checkout (skipped where there is none), pointed at brrr_engine and
    brrr_engine_qwen, and its request() must return the text and the [STATS] fields the oracle predicts."""
    import importlib.util
    import refdata
    from oracle import oracle_host as H
    src = os.path.join(refdata.REF, "scripts", "openai_server.py")
    if not os.path.exists(src):
        pytest.skip("reference checkout not present")
    spec = importlib.util.spec_from_file_location("ref_openai_server", src)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)                       # defines Engine; starts nothing (no engines found under its ROOT)
    bindir = os.path.dirname(brrr.__file__)
    for case, seed, exe, qwen in (("gptoss_serve", 37, "brrr_engine", False), ("qwen_d256", 41, "brrr_engine_qwen", True)):
        cfg, d, blob = refdata.case_data_dir(str(tmp_path / case), case, seed)
        toks = H.load_tokens(os.path.join(d, "tokens.bin"))
        om = (orc.QwenModel if qwen else orc.Model).open(d, blob)
        eng = mod.Engine({"id": "test/" + case, "bin": os.path.join(bindir, exe), "data": d})
        with eng.lock:
            eng.ensure()
            got = []
            stats = eng.request("w3 w4\nw5", 6, 0.0, got.append)
        eng.proc.stdin.close()
        eng.proc.wait(timeout=60)
        if qwen:
            want = H.qwen_generate(om.run, toks, H.qwen_chat_prompt(toks, "w3 w4 w5"), 6)
        else:
            want = oracle_generate(orc, om, H.chat_prompt(H.make_lookup(toks), "w3 w4\nw5"), 6)
        assert "".join(got) == b"".join(toks[t] for t in want).decode("utf-8", "replace")
        assert int(stats["decode_tok"]) == len(want) and stats["tok_s"] >= 0
        om.close()
