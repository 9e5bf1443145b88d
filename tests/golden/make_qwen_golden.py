"""Generates tests/golden/qwen_tiny_tokens.json from the CPU oracle's qwen3moe model.

    python tests/golden/make_qwen_golden.py

Prompt, 96 greedy tokens and the first logits (bit patterns) of a tiny seeded qwen3moe-architecture
model.  The reference stores no golden vectors for its forward pass and cannot run here (Rust +
NEON); the oracle's kernels are pinned separately against the reference's own C dots
(kq_ref_dots.json).  This fixture pins the oracle's forward pass against drift and gives the CUDA
tests a size-independent anchor.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from cpubrrr_b200 import synth as S  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    cfg = dict(d=256, nh=4, nkv=2, hd=128, nl=3, ne=16, topk=4, ff=256, nvocab=1024)
    seed = 7
    m = O.QwenModel.synth(O.make_qcfg(**cfg), seed)
    prompt = [int(t) for t in S.synth_prompt(seed, 9, cfg["nvocab"])]
    tok = 0
    for i, t in enumerate(prompt):
        tok = m.run(t, i, i == len(prompt) - 1)
    out, pos = [], len(prompt)
    for _ in range(96):
        out.append(tok)
        tok = m.run(tok, pos, True)
        pos += 1
    g = dict(cfg=cfg, seed=seed, prompt=prompt, tokens=out, last_logit_bits=[int(b) for b in m.logits()[:8].view(np.uint32)])
    json.dump(g, open(os.path.join(HERE, "qwen_tiny_tokens.json"), "w"))
    print("distinct tokens:", len(set(out)))


if __name__ == "__main__":
    main()
