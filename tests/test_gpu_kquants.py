"""Parity of the qwen3moe K-quant kernels (Q8_K quantiser, Q4_K / Q6_K matvec) against the CPU
oracle through the C ABI.  Bar: int8 quants, int32 sums and superblock accumulators bit-exact;
float outputs bit-exact (0 ulp), asserted on the bit patterns.  The committed results of the
reference's own C dots (tests/golden/kq_ref_dots.json) are checked directly as well."""
import ctypes as C
import json
import os

import numpy as np
import pytest

from conftest import bits, to_dev
from cpubrrr_b200 import synth as S

pytestmark = pytest.mark.gpu
GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kq_ref_dots.json")))


def P(t):
    return C.c_void_p(t.data_ptr())


def ok(status):
    assert status == 0, status


@pytest.fixture(scope="module")
def L(brrr):
    return brrr.lib()


def gpu_quant(L, dev, x):
    import torch
    n = x.size
    dx = to_dev(x, dev)
    dq = torch.empty(n, dtype=torch.int8, device=dev)
    ds = torch.empty(n // 256, dtype=torch.float32, device=dev)
    db = torch.empty(n // 32, dtype=torch.int32, device=dev)
    ok(L.brrr_quant_q8k(P(dx), n, P(dq), P(ds), P(db), None))
    torch.cuda.synchronize()
    return dq, ds, db


@pytest.mark.parametrize("n", [256, 768, 2048, 4096 * 8])
def test_quant_q8k(L, orc, dev, n):
    x = S.synth_activation(n, n, 2.0)
    if n >= 768:
        x[256:512] = 0.0
        x[513] = 1e-25
    dq, ds, db = gpu_quant(L, dev, x)
    q, s, bs = orc.quant_q8k(x)
    assert np.array_equal(dq.cpu().numpy(), q)
    assert np.array_equal(bits(ds.cpu().numpy()), bits(s))
    assert np.array_equal(db.cpu().numpy(), bs)


def gpu_matvec(L, dev, kind, w, rows, cols, dq, ds, db):
    import torch
    dw = to_dev(w.reshape(-1), dev)
    dy = torch.empty(rows, dtype=torch.float32, device=dev)
    nsb = cols // 256
    if kind == "q4k":
        dd = torch.empty(rows * nsb * 2, dtype=torch.int32, device=dev)
        ok(L.brrr_q4k_matvec(P(dw), rows, cols, P(dq), P(ds), P(db), P(dy), P(dd), None))
        shape = (rows, nsb, 2)
    else:
        dd = torch.empty(rows * nsb, dtype=torch.int32, device=dev)
        ok(L.brrr_q6k_matvec(P(dw), rows, cols, P(dq), P(ds), P(dy), P(dd), None))
        shape = (rows, nsb)
    torch.cuda.synchronize()
    return dy.cpu().numpy(), dd.cpu().numpy().reshape(shape)


@pytest.mark.parametrize("kind", ["q4k", "q6k"])
@pytest.mark.parametrize("rows,cols", [(1, 256), (13, 768), (768, 2048), (2048, 768), (4096, 4096)])
def test_kquant_matvec(L, orc, dev, kind, rows, cols):
    x = S.synth_activation(rows + cols, cols)
    w = S.synth_q4k(rows, rows, cols) if kind == "q4k" else S.synth_q6k(rows, rows, cols)
    dq, ds, db = gpu_quant(L, dev, x)
    xq, ys, bs = orc.quant_q8k(x)
    y, dbg = gpu_matvec(L, dev, kind, w, rows, cols, dq, ds, db)
    if kind == "q4k":
        yo, do = orc.q4k_matvec(w, rows, cols, xq, ys, bs, True)
    else:
        yo, do = orc.q6k_matvec(w, rows, cols, xq, ys, True)
    assert np.array_equal(dbg, do)
    assert np.array_equal(bits(y), bits(yo))


@pytest.mark.parametrize("i", range(len(GOLD["cases"])))
def test_kquant_matvec_reference_golden(L, dev, i):
    """Against what the reference's own C dots returned for the same seeded inputs.  Q6_K: same bits.
    Q4_K: the reference's CPU engine and its C check code associate the superblock update
    differently (ys*d*acc - ys*dmin*mint against ys*(d*acc - dmin*mint)); the kernel follows the
    engine, so it meets the C code within a few ulp of the row's scale, and its integers rebuilt
    in the C code's order give the C code's bits."""
    c = GOLD["cases"][i]
    x = S.synth_activation(c["seed"] + 7, c["cols"])
    w = S.synth_q4k(c["seed"], c["rows"], c["cols"]) if c["kind"] == "q4k" else S.synth_q6k(c["seed"], c["rows"], c["cols"])
    dq, ds, db = gpu_quant(L, dev, x)
    assert [int(v) for v in bits(ds.cpu().numpy())] == c["ys_bits"]
    y, dbg = gpu_matvec(L, dev, c["kind"], w, c["rows"], c["cols"], dq, ds, db)
    if c["kind"] == "q6k":
        assert [int(v) for v in bits(y)] == c["y_bits"]
        return
    from test_oracle_qwen import _metal_order_q4k
    assert _metal_order_q4k(w, ds.cpu().numpy(), dbg) == c["y_bits"]
    gold = np.array(c["y_bits"], np.uint32).view(np.float32)
    assert np.max(np.abs(y - gold)) <= 4e-6 * np.max(np.abs(gold))


def test_kquant_bad_args(L, dev):
    import torch
    t = torch.zeros(1024, dtype=torch.uint8, device=dev)
    assert L.brrr_quant_q8k(P(t), 100, P(t), P(t), P(t), None) == 1
    assert L.brrr_q4k_matvec(P(t), 1, 100, P(t), P(t), P(t), P(t), None, None) == 1
    assert L.brrr_q6k_matvec(None, 1, 256, P(t), P(t), P(t), None, None) == 1
