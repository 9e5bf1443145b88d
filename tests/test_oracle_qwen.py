"""CPU tests of the oracle's qwen3moe kernels (Q8_K quantiser, Q4_K / Q6_K x Q8_K dots).

Pins: (1) results of the reference's own scalar C dots (metal/engine_metal.m:589-643), committed as
tests/golden/kq_ref_dots.json and, when the reference checkout is present, re-run live;
(2) the gguf package's Q4_K / Q6_K dequantiser, dequantise-then-dot in float64 within the
reference's verifier threshold (rel < 1e-3, src/bin/q8k_verify.rs)."""
import ctypes as C
import json
import os
import zlib

import numpy as np
import pytest

from cpubrrr_b200 import synth as S

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "kq_ref_dots.json")))


def _weights(c):
    return S.synth_q4k(c["seed"], c["rows"], c["cols"]) if c["kind"] == "q4k" else S.synth_q6k(c["seed"], c["rows"], c["cols"])


def _oracle_y(orc, c, want_dbg=False):
    x = S.synth_activation(c["seed"] + 7, c["cols"])
    xq, ys, bs = orc.quant_q8k(x)
    w = _weights(c)
    if c["kind"] == "q4k":
        return x, xq, ys, bs, w, orc.q4k_matvec(w, c["rows"], c["cols"], xq, ys, bs, want_dbg)
    return x, xq, ys, bs, w, orc.q6k_matvec(w, c["rows"], c["cols"], xq, ys, want_dbg)


def _metal_order_q4k(w, ys, dbg):
    """The reference has two float associations for the Q4_K superblock update: the CPU engine's
    ys*d*acc - ys*dmin*mint (src/bin/engine_qwen2.rs:110, what the oracle computes) and the C check
    code's ys*(d*acc - dmin*mint) (metal/engine_metal.m:618).  Rebuilding the second one from the
    oracle's integer accumulators must give the C code's bits exactly; that pins the half
    conversion, the 6-bit scale unpacking and every integer of the oracle."""
    rows, nsb = dbg.shape[:2]
    blk = w.reshape(rows, nsb, 144)
    d = blk[:, :, 0:2].copy().view(np.float16).astype(np.float32)[:, :, 0]
    dmin = blk[:, :, 2:4].copy().view(np.float16).astype(np.float32)[:, :, 0]
    out = []
    for r in range(rows):
        sumf = np.float32(0)
        for sb in range(nsb):
            t = np.float32(d[r, sb] * np.float32(dbg[r, sb, 0])) - np.float32(dmin[r, sb] * np.float32(dbg[r, sb, 1]))
            sumf = np.float32(sumf + np.float32(ys[sb] * np.float32(t)))
        out.append(int(sumf.view(np.uint32)))
    return out


@pytest.mark.parametrize("i", range(len(GOLD["cases"])))
def test_dots_match_reference_c_golden(orc, i):
    c = GOLD["cases"][i]
    _, xq, ys, _, w, (y, dbg) = _oracle_y(orc, c, True)
    assert zlib.crc32(xq.tobytes()) == c["xq_crc"]
    assert [int(v) for v in ys.view(np.uint32)] == c["ys_bits"]
    if c["kind"] == "q6k":
        assert [int(v) for v in y.view(np.uint32)] == c["y_bits"]
        return
    assert _metal_order_q4k(w, ys, dbg) == c["y_bits"]
    gold = np.array(c["y_bits"], np.uint32).view(np.float32)
    assert np.max(np.abs(y - gold)) <= 4e-6 * np.max(np.abs(gold))


def test_half_matches_reference_c_golden(orc):
    for h, b in GOLD["half"]:
        assert int(orc.half_to_f32(h).view(np.uint32)) == b


def test_half_all_values_match_numpy(orc):
    hs = np.arange(65536, dtype=np.uint16)
    want = hs.view(np.float16).astype(np.float32).view(np.uint32)
    got = np.array([orc.half_to_f32(int(h)).view(np.uint32) for h in hs[::7]], dtype=np.uint32)
    nan = np.isnan(hs[::7].view(np.float16))
    assert np.array_equal(got[~nan], want[::7][~nan])


def test_live_reference_c_when_present(orc):
    R = orc.ref_kq()
    if R is None:
        pytest.skip("reference checkout not present and no prebuilt oracle/_ref")
    P = lambda a: a.ctypes.data_as(C.c_void_p)
    for c in (dict(kind="q4k", seed=9, rows=40, cols=1024), dict(kind="q6k", seed=10, rows=40, cols=1024)):
        _, xq, ys, bs, w, (y, dbg) = _oracle_y(orc, c, True)
        alt = _metal_order_q4k(w, ys, dbg) if c["kind"] == "q4k" else None
        for r in range(c["rows"]):
            row = np.ascontiguousarray(w[r])
            if c["kind"] == "q4k":
                v = R.refkq_q4k_dot(P(row), P(xq), P(ys), P(bs), C.c_int(c["cols"]))
                assert np.float32(v).view(np.uint32) == alt[r]
            else:
                v = R.refkq_q6k_dot(P(row), P(xq), P(ys), C.c_int(c["cols"]))
                assert np.float32(v).view(np.uint32) == y[r].view(np.uint32)


def test_q8k_quantiser_against_numpy(orc):
    x = S.synth_activation(5, 2048, 3.0)
    x[256:512] = 0.0                       # an all-zero superblock: scale floor 1e-12/127
    q, s, bs = orc.quant_q8k(x)
    xb = x.reshape(-1, 256)
    amax = np.maximum(np.abs(xb).max(1), np.float32(1e-12)).astype(np.float32)
    sc = (amax / np.float32(127.0)).astype(np.float32)
    assert np.array_equal(s.view(np.uint32), sc.view(np.uint32))
    v = (xb / sc[:, None]).astype(np.float32)
    r = np.clip(np.sign(v) * np.floor(np.abs(v) + np.float32(0.5)), -127, 127).astype(np.int8)
    assert np.array_equal(q.reshape(-1, 256), r)
    assert np.array_equal(bs, q.reshape(-1, 32).astype(np.int32).sum(1))
    assert np.all(q[256:512] == 0) and np.abs(q).max() == 127


@pytest.mark.parametrize("kind", ["q4k", "q6k"])
def test_dots_against_gguf_dequantiser(orc, kind):
    from gguf import quants, GGMLQuantizationType as QT
    c = dict(kind=kind, seed=31, rows=32, cols=2048)
    x, xq, ys, bs, w, (y, dbg) = _oracle_y(orc, c, True)
    wd = quants.dequantize(w, QT.Q4_K if kind == "q4k" else QT.Q6_K).astype(np.float64)
    assert wd.shape == (c["rows"], c["cols"])
    # exact statement of what the integer kernel computes: dequantised weights x dequantised activations
    xd = (xq.reshape(-1, 256).astype(np.float64) * ys[:, None].astype(np.float64)).ravel()
    exact = wd @ xd
    scale = np.abs(wd) @ np.abs(xd)
    assert np.max(np.abs(y - exact) / scale) < 2e-6
    # and the reference verifier's own bar against the unquantised activations
    full = wd @ x.astype(np.float64)
    assert np.linalg.norm(y - full) / np.linalg.norm(full) < 2e-2
    assert np.max(np.abs(y - exact)) / np.max(np.abs(exact)) < 1e-3
    assert dbg.dtype == np.int32


# ---- the oracle's qwen3moe forward pass ---------------------------------------------------------
QGOLD = json.load(open(os.path.join(HERE, "golden", "qwen_tiny_tokens.json")))


def _greedy(m, prompt, n):
    tok = 0
    for i, t in enumerate(prompt):
        tok = m.run(t, i, i == len(prompt) - 1)
    out, pos = [], len(prompt)
    for _ in range(n):
        out.append(tok)
        tok = m.run(tok, pos, True)
        pos += 1
    return out


def test_qwen_golden_tokens(orc):
    g = QGOLD
    m = orc.QwenModel.synth(orc.make_qcfg(**g["cfg"]), g["seed"])
    assert _greedy(m, g["prompt"], len(g["tokens"])) == g["tokens"]
    assert [int(b) for b in m.logits()[:8].view(np.uint32)] == g["last_logit_bits"]


def test_qwen_data_dir_equals_synth(orc, tmp_path):
    """The file-loading path (GGUF blob + config.txt + manifest.txt in the reference's formats)
    gives the same model as the in-memory generator: same tensors, same tokens."""
    import refdata
    c = QGOLD["cfg"]
    cfg, d, blob = refdata.case_data_dir(str(tmp_path / "qw"), "qwen_gold", QGOLD["seed"])
    text = open(os.path.join(d, "config.txt")).read()
    assert "n_ff_exp 256" in text and "head_dim 128" in text
    m = orc.QwenModel.open(d, blob)
    assert m.cfg.ff == c["ff"] and m.cfg.nvocab == c["nvocab"]
    assert _greedy(m, QGOLD["prompt"], 24) == QGOLD["tokens"][:24]


def test_qwen_mixed_types_data_dir(orc, tmp_path):
    """Per-tensor K-quant types come from the manifest (engine_qwen2.rs:202-212): a directory whose
    attn_v (layer 0) is Q6_K and whose down experts (layer 1) are Q4_K loads and runs; its tensors
    carry the stored types."""
    import refdata
    cfg, d, blob = refdata.case_data_dir(str(tmp_path / "qm"), "qwen_mixed", 12)
    m = orc.QwenModel.open(d, blob)
    p = S.synth_prompt(12, 7, cfg.n_vocab)
    toks = _greedy(m, [int(t) for t in p], 12)
    assert len(toks) == 12 and np.isfinite(m.logits()).all()
    plain = orc.QwenModel.synth(orc.make_qcfg(cfg.n_embd, cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.n_layer, cfg.n_expert,
                                              cfg.n_expert_used, cfg.n_ff_exp, cfg.n_vocab), 12)
    _greedy(plain, [int(t) for t in p], 12)
    assert not np.array_equal(plain.hidden(), m.hidden())


def test_qwen_norm_and_router_pieces(orc):
    """12-slice RMS norm against a float64 computation; router order on exact ties."""
    L = orc.lib()
    d = 2048
    x = S.synth_activation(3, d, 2.0)
    w = S.synth_f32(1, 0, S.T["ATTN_NORM"], d)
    out = np.empty(d, np.float32)
    L.orcq_rmsnorm(x.ctypes.data_as(C.c_void_p), w.ctypes.data_as(C.c_void_p), C.c_float(1e-6), d, out.ctypes.data_as(C.c_void_p))
    ref = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-6) * w
    assert np.max(np.abs(out - ref)) < 1e-5 * np.max(np.abs(ref))
    ne, k = 16, 4
    W = np.zeros((ne, 256), np.float32)
    W[3, 0] = W[9, 0] = 1.0
    W[5, 0] = 2.0
    xn = np.zeros(256, np.float32); xn[0] = 1.0
    lg = np.empty(ne, np.float32); top = np.empty(k, np.int32); wts = np.empty(k, np.float32)
    L.orcq_router_topk(W.ctypes.data_as(C.c_void_p), xn.ctypes.data_as(C.c_void_p), ne, 256, k, lg.ctypes.data_as(C.c_void_p),
                       top.ctypes.data_as(C.c_void_p), wts.ctypes.data_as(C.c_void_p))
    assert list(top) == [5, 3, 9, 0]           # value first, then the lower index among equals (stable sort)
    assert abs(float(wts.sum()) - 1.0) < 1e-6 and wts[0] > wts[1] == wts[2] > wts[3]
