"""Batched decode over independent sequences (brrr_batch_*): every row's token and logits must equal what
the one-sequence engine produces for that sequence alone, bit for bit - whatever the other rows of the
pass are.  The reference decodes one sequence; its tile path groups token rows by routed expert
(src/bin/engine_gpt2.rs:1160-1172), which is what a batch of sequences generalises."""
import numpy as np
import pytest

from conftest import bits
from cpubrrr_b200 import synth as S

pytestmark = pytest.mark.gpu


def serial_run(eng, prompt, ngen, want_logits_at=None):
    """Tokens the one-sequence engine generates greedily after `prompt` (token-serial schedule), and the
    logits of the step that produced generated token `want_logits_at`."""
    tok = 0
    for i, t in enumerate(prompt):
        tok = eng.run(int(t), i, i == len(prompt) - 1)
    out, lg = [tok], eng.logits().copy() if want_logits_at == 0 else None
    for k in range(1, ngen):
        tok = eng.run(tok, len(prompt) + k - 1, True)
        out.append(tok)
        if want_logits_at == k:
            lg = eng.logits().copy()
    return out, lg


def test_batch_rows_equal_each_sequence_alone(brrr):
    cfg = brrr.make_cfg(256, 3, 8, 2, 8, 4, 1024, sliding_window=8)
    eng = brrr.Engine.synth(cfg, 21)
    eng.set_tile_prefill(False)
    lens = [3, 17, 70, 1, 33]
    prompts = [[int(t) for t in S.synth_prompt(50 + i, n, 1000)] for i, n in enumerate(lens)]
    ngen = 10
    want = [serial_run(eng, p, ngen, want_logits_at=2) for p in prompts]
    eng.batch_open(len(prompts))
    for s, p in enumerate(prompts):
        if len(p) > 1:
            eng.batch_prefill(s, p[:-1])
    seqs = list(range(len(prompts)))
    toks = [p[-1] for p in prompts]
    pos = [len(p) - 1 for p in prompts]
    got = [[] for _ in prompts]
    for k in range(ngen):
        if k == 2:
            out, lg = eng.batch_step(toks, pos, seqs, logits=True)
            for s in seqs:
                assert np.array_equal(bits(lg[s]), bits(want[s][1])), f"logits of sequence {s}"
        else:
            out = eng.batch_step(toks, pos, seqs)
        for s in seqs:
            got[s].append(int(out[s]))
        toks = [int(t) for t in out]
        pos = [q + 1 for q in pos]
    for s in seqs:
        assert got[s] == want[s][0], f"sequence {s}"
    assert len({tuple(g) for g in got}) > 1
    eng.close()


def test_batch_ragged_and_mixed_rows(brrr):
    """Sequences leave the batch at different times; one pass mixes the prompt rows of a late sequence
    (ascending positions of one sequence) with single decode rows of the others; 64 rows in one pass."""
    cfg = brrr.make_cfg(128, 2, 4, 2, 8, 4, 512, sliding_window=16)
    eng = brrr.Engine.synth(cfg, 22)
    eng.set_tile_prefill(False)
    pa = [int(t) for t in S.synth_prompt(1, 9, 500)]
    pb = [int(t) for t in S.synth_prompt(2, 5, 500)]
    pc = [int(t) for t in S.synth_prompt(3, 20, 500)]
    wa, _ = serial_run(eng, pa, 8)
    wb, _ = serial_run(eng, pb, 3)
    wc, _ = serial_run(eng, pc, 4)
    eng.batch_open(64)
    eng.batch_prefill(7, pa[:-1])
    eng.batch_prefill(0, pb[:-1])
    out = eng.batch_step([pa[-1], pb[-1]], [8, 4], [7, 0])
    ga, gb = [int(out[0])], [int(out[1])]
    # next pass: a and b decode one row each, c arrives with its whole prompt as 20 rows of sequence 63
    out = eng.batch_step([ga[-1], gb[-1]] + pc, [9, 5] + list(range(20)), [7, 0] + [63] * 20)
    ga.append(int(out[0])); gb.append(int(out[1])); gc = [int(out[-1])]
    out = eng.batch_step([ga[-1], gb[-1], gc[-1]], [10, 6, 20], [7, 0, 63])
    ga.append(int(out[0])); gb.append(int(out[1])); gc.append(int(out[2]))
    assert gb == wb                                   # b leaves
    for k in range(2):
        out = eng.batch_step([ga[-1], gc[-1]], [11 + k, 21 + k], [7, 63])
        ga.append(int(out[0])); gc.append(int(out[1]))
    assert gc == wc
    for k in range(3):
        out = eng.batch_step([ga[-1]], [13 + k], [7])
        ga.append(int(out[0]))
    assert ga == wa
    # 64 rows in one pass: 64 sequences with the same first token give 64 equal answers, equal to the serial engine's
    first = eng.run(pa[0], 0, True)
    out = eng.batch_step([pa[0]] * 64, [0] * 64, list(range(64)))
    assert [int(t) for t in out] == [first] * 64
    eng.close()


def test_batch_bad_args(brrr):
    cfg = brrr.make_cfg(64, 1, 2, 1, 4, 2, 256)
    eng = brrr.Engine.synth(cfg, 23)
    L = brrr.lib()
    # statuses: 1 = BRRR_ERR_ARG, 5 = BRRR_ERR_RANGE, 6 = BRRR_ERR_STATE
    one = np.zeros(600, np.uint32)
    out = np.zeros(600, np.uint32)
    p = one.ctypes.data
    assert L.brrr_batch_step(eng._h, 1, p, p, p, out.ctypes.data) == 6      # before brrr_batch_open
    assert L.brrr_batch_open(eng._h, 0) == 1 and L.brrr_batch_open(eng._h, 257) == 1
    assert L.brrr_batch_open(eng._h, 2) == 0
    assert L.brrr_batch_open(eng._h, 2) == 6
    assert L.brrr_batch_step(eng._h, 513, p, p, p, out.ctypes.data) == 1
    assert L.brrr_batch_step(eng._h, 0, p, p, p, out.ctypes.data) == 1
    bad = np.array([2], np.uint32)
    assert L.brrr_batch_step(eng._h, 1, p, p, bad.ctypes.data, out.ctypes.data) == 5     # sequence 2 of 2
    bad = np.array([256], np.uint32)
    assert L.brrr_batch_step(eng._h, 1, bad.ctypes.data, p, p, out.ctypes.data) == 5     # token outside the vocabulary
    bad = np.array([4096], np.uint32)
    assert L.brrr_batch_step(eng._h, 1, p, bad.ctypes.data, p, out.ctypes.data) == 5
    assert L.brrr_batch_prefill(eng._h, 2, p, 4, 0) == 5
    assert L.brrr_batch_step(eng._h, 1, p, p, p, out.ctypes.data) == 0
    eng.close()
