"""Generates the committed fixtures under tests/golden/ from the CPU oracle.

    python tests/golden/make_golden.py

gptoss_tiny_tokens.json: prompt, 160 greedy tokens and the first logits (as bit patterns) of a
tiny seeded gpt-oss-architecture model with a sliding window of 16, so the run crosses the window.
The reference stores no golden vectors for this path and cannot be run here (Rust + NEON); these
fixtures pin the oracle against drift and give the CUDA tests a size-independent anchor.
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
    cfg = dict(d=128, nh=8, nkv=2, nl=3, ne=8, topk=4, nvocab=1024, swa=16)
    seed = 20
    m = O.Model.synth(O.make_cfg(hd=64, **cfg), seed)
    prompt = [int(t) for t in S.synth_prompt(seed, 9, cfg["nvocab"])]
    tok = 0
    for i, t in enumerate(prompt):
        tok = m.run(t, i, i == len(prompt) - 1)
    out, pos = [], len(prompt)
    for _ in range(160):
        out.append(tok)
        tok = m.run(tok, pos, True)
        pos += 1
    g = dict(cfg=cfg, seed=seed, prompt=prompt, tokens=out, last_logit_bits=[int(b) for b in m.logits()[:8].view(np.uint32)])
    json.dump(g, open(os.path.join(HERE, "gptoss_tiny_tokens.json"), "w"))
    print("distinct tokens:", len(set(out)))


if __name__ == "__main__":
    main()
