"""Generates tests/golden/kq_ref_dots.json by RUNNING THE REFERENCE'S OWN C CODE: the scalar
Q4_K / Q6_K x Q8_K dots that metal/engine_metal.m:589-643 of the reference defines as plain C
(ref_q4k_dot, ref_q6k_dot, half2f), compiled from the reference checkout into oracle/_ref/ by
oracle/Makefile (target `ref`).  Inputs are seeded (cpubrrr_b200.synth), so the fixture stores
seeds, shapes and the result bit patterns only.

    python tests/golden/make_kq_golden.py     # needs the reference checkout

The activations are quantised with the oracle's Q8_K quantiser; the fixture stores a CRC of the
quantised bytes too, so a drift of the quantiser is seen as such.
"""
import ctypes as C
import json
import os
import sys
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from cpubrrr_b200 import synth as S  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [dict(kind="q4k", seed=101, rows=24, cols=256), dict(kind="q4k", seed=102, rows=16, cols=2048),
         dict(kind="q6k", seed=201, rows=24, cols=256), dict(kind="q6k", seed=202, rows=16, cols=2048),
         dict(kind="q4k", seed=103, rows=8, cols=768), dict(kind="q6k", seed=203, rows=8, cols=768)]


def P(a):
    return a.ctypes.data_as(C.c_void_p)


def run_case(R, c):
    x = S.synth_activation(c["seed"] + 7, c["cols"])
    xq, ys, bs = O.quant_q8k(x)
    w = S.synth_q4k(c["seed"], c["rows"], c["cols"]) if c["kind"] == "q4k" else S.synth_q6k(c["seed"], c["rows"], c["cols"])
    y = np.empty(c["rows"], np.float32)
    for r in range(c["rows"]):
        row = np.ascontiguousarray(w[r])
        if c["kind"] == "q4k":
            y[r] = R.refkq_q4k_dot(P(row), P(xq), P(ys), P(bs), C.c_int(c["cols"]))
        else:
            y[r] = R.refkq_q6k_dot(P(row), P(xq), P(ys), C.c_int(c["cols"]))
    return dict(c, xq_crc=zlib.crc32(xq.tobytes()), ys_bits=[int(v) for v in ys.view(np.uint32)],
                y_bits=[int(v) for v in y.view(np.uint32)])


def main():
    R = O.ref_kq()
    if R is None:
        raise SystemExit("reference checkout not present: cannot build oracle/_ref/libref_kq.so")
    halves = [0, 1, 0x3FF, 0x400, 0x3C00, 0x7BFF, 0x8001, 0xBC00, 0xFBFF, 0x0200, 0x03FE, 0x7C00]
    g = dict(cases=[run_case(R, c) for c in CASES],
             half=[[h, int(np.float32(R.refkq_half2f(h)).view(np.uint32))] for h in halves])
    json.dump(g, open(os.path.join(HERE, "kq_ref_dots.json"), "w"))
    print("wrote", len(g["cases"]), "cases")


if __name__ == "__main__":
    main()
