"""Stage-level parity of the CUDA kernels against the CPU oracle, through the C ABI.

Bar: integer results (int8 quants, int32 block dots, expert indices) bit-exact; float results
bit-exact too, because every kernel reproduces the oracle's operation order (tolerance 0 ulp,
asserted on the bit patterns)."""
import ctypes as C

import numpy as np
import pytest

from conftest import bits, to_dev
from cpubrrr_b200 import synth as S

pytestmark = pytest.mark.gpu


def P(t):
    return C.c_void_p(t.data_ptr())


def ok(status):
    assert status == 0, status


@pytest.fixture(scope="module")
def L(brrr):
    return brrr.lib()


def test_expf_bits(L, orc, dev):
    import torch
    x = np.concatenate([np.linspace(-104.5, 89.0, 20001), np.linspace(-3, 3, 10001), [0.0, -0.0, 88.72283, -87.4, -103.0]]).astype(np.float32)
    dx = to_dev(x, dev); dy = torch.empty_like(dx)
    ok(L.brrr_expf(P(dx), x.size, P(dy), None))
    assert np.array_equal(bits(dy.cpu().numpy()), bits(orc.expf(x)))


@pytest.mark.parametrize("n", [32, 2880, 4096])
def test_quant_q8(L, orc, dev, n):
    import torch
    x = S.synth_input(n, n) * np.float32(2.5)
    x[:32] = 0.0
    if n > 64:
        x[40] = 1e-20; x[41] = -3.0e4
    dx = to_dev(x, dev)
    dq = torch.empty(n, dtype=torch.int8, device=dev); ds = torch.empty(n // 32, dtype=torch.float32, device=dev)
    ok(L.brrr_quant_q8(P(dx), n, P(dq), P(ds), None))
    q, s = orc.quant_q8(x)
    assert np.array_equal(dq.cpu().numpy(), q) and np.array_equal(bits(ds.cpu().numpy()), bits(s))


@pytest.mark.parametrize("n", [64, 2880, 2048])
def test_rmsnorm_quant(L, orc, dev, n):
    import torch
    x = S.synth_input(n + 1, n) * np.float32(7.0)
    w = S.synth_f32(1, 0, S.T["ATTN_NORM"], n)
    dx, dw = to_dev(x, dev), to_dev(w, dev)
    dxn = torch.empty(n, dtype=torch.float32, device=dev)
    dq = torch.empty(n, dtype=torch.int8, device=dev); ds = torch.empty(n // 32, dtype=torch.float32, device=dev)
    ok(L.brrr_rmsnorm_quant(P(dx), P(dw), C.c_float(1e-5), n, P(dxn), P(dq), P(ds), None))
    xn = orc.rmsnorm(x, w, 1e-5)
    q, s = orc.quant_q8(xn)
    assert np.array_equal(bits(dxn.cpu().numpy()), bits(xn))
    assert np.array_equal(dq.cpu().numpy(), q) and np.array_equal(bits(ds.cpu().numpy()), bits(s))


@pytest.mark.parametrize("rows,cols", [(64, 64), (96, 2880), (36, 4096), (1028, 128)])
def test_q8_pack_and_matvec(L, orc, dev, rows, cols):
    import torch
    wb = S.synth_bf16(rows, 0, S.T["WQ"], rows * cols)
    dw = to_dev(wb, dev)
    h = C.c_void_p()
    ok(L.brrr_q8mat_from_bf16(P(dw), rows, cols, C.byref(h), None))
    dq = torch.empty((rows, cols), dtype=torch.int8, device=dev)
    ds = torch.empty((rows, cols // 32), dtype=torch.float32, device=dev)
    ok(L.brrr_q8mat_export(h, P(dq), P(ds), None))
    q, s = orc.q8_from_bf16(wb, rows, cols)
    assert np.array_equal(dq.cpu().numpy(), q) and np.array_equal(bits(ds.cpu().numpy()), bits(s))
    x = S.synth_input(cols, cols)
    xq, xs = orc.quant_q8(x)
    dy = torch.empty(rows, dtype=torch.float32, device=dev)
    dxq, dxs = to_dev(xq, dev), to_dev(xs, dev)      # keep the inputs alive across the call
    ok(L.brrr_q8_matvec(h, P(dxq), P(dxs), P(dy), None))
    torch.cuda.synchronize()
    assert np.array_equal(bits(dy.cpu().numpy()), bits(orc.q8_matvec(q, s, xq, xs)))
    L.brrr_q8mat_free(h)


@pytest.mark.parametrize("rows,cols,ntok", [(64, 64, 1), (96, 2880, 5), (36, 4096, 16), (1028, 128, 9), (5120, 2880, 64), (2880, 4096, 33)])
def test_q8_matmul_rows_equal_oracle_on_both_engines(L, orc, dev, rows, cols, ntok):
    """Q8 matrix x token rows (the q/k/v and o-proj products of a tile) on the integer units and on the tcgen05
    kind::i8 tensor-core kernel: every output equals the oracle's one-row dot bit for bit; nothing is written
    beyond the matrix rows (ldy > rows), ragged row tiles and chunks included."""
    import torch
    wb = S.synth_bf16(rows + ntok, 1, S.T["WQ"], rows * cols)
    h = C.c_void_p()
    dw = to_dev(wb, dev)
    ok(L.brrr_q8mat_from_bf16(P(dw), rows, cols, C.byref(h), None))
    q, s = orc.q8_from_bf16(wb, rows, cols)
    xq = np.empty((ntok, cols), np.int8); xs = np.empty((ntok, cols // 32), np.float32)
    want = np.empty((ntok, rows), np.float32)
    for t in range(ntok):
        x = S.synth_input(200 + t, cols) * np.float32(0.25 + t)
        if t == 2:
            x[:96] = 0.0
        xq[t], xs[t] = orc.quant_q8(x)
        want[t] = orc.q8_matvec(q, s, xq[t], xs[t])
    dxq, dxs = to_dev(xq, dev), to_dev(xs, dev)
    ldy = rows + 5
    for tensor_cores in (0, 1):
        dy = torch.full((ntok, ldy), 3.0, dtype=torch.float32, device=dev)
        ok(L.brrr_q8_matmul_rows(h, P(dxq), P(dxs), ntok, P(dy), ldy, tensor_cores, None))
        torch.cuda.synchronize()
        got = dy.cpu().numpy()
        assert np.array_equal(bits(got[:, :rows]), bits(want)), f"engine {tensor_cores}"
        assert np.all(got[:, rows:] == 3.0)
    L.brrr_q8mat_free(h)


@pytest.mark.parametrize("rows,blocks", [(16, 2), (64, 90), (208, 4), (2880, 90), (48, 26)])
def test_mx_pack_and_matvec_int_exact(L, orc, dev, rows, blocks):
    """int32 lane accumulators of every (row, block) equal the oracle's; f32 row results too."""
    import torch
    raw = S.synth_mxfp4(rows + blocks, 1, S.T["UP"], rows * blocks)
    # widen the exponent range beyond the synthetic 117..123, including both subnormal scales
    r = raw.reshape(rows * blocks, 17)
    r[::7, 0] = np.arange(len(r[::7])) % 200     # 2^(e-128) up to 2^71: no overflow to inf
    h = C.c_void_p()
    draw = to_dev(raw, dev)
    ok(L.brrr_mxmat_from_gguf(P(draw), rows, blocks, C.byref(h), None))
    x = S.synth_input(blocks, blocks * 32) * np.float32(1e-3 if blocks == 4 else 1.0)
    xq, xs = orc.quant_q8(x)
    nib, exps = orc.repack_mx(raw, rows, blocks)
    y, dbg = orc.mx_matvec(nib, exps, rows, blocks, xq, xs, want_dbg=True)
    dy = torch.empty(rows, dtype=torch.float32, device=dev)
    dd = torch.empty((rows, blocks, 4), dtype=torch.int32, device=dev)
    dxq, dxs = to_dev(xq, dev), to_dev(xs, dev)
    ok(L.brrr_mx_matvec(h, 0, rows, P(dxq), P(dxs), P(dy), P(dd), None))
    want = dbg.transpose(0, 2, 1, 3).reshape(rows, blocks, 4)   # [quad][blk][row][lane] -> [row][blk][lane]
    assert np.array_equal(dd.cpu().numpy(), want)
    assert np.array_equal(bits(dy.cpu().numpy()), bits(y))
    # production variant (no debug output), and a row window
    dy2 = torch.empty(rows, dtype=torch.float32, device=dev)
    ok(L.brrr_mx_matvec(h, 0, rows, P(dxq), P(dxs), P(dy2), None, None))
    assert np.array_equal(bits(dy2.cpu().numpy()), bits(y))
    if rows >= 16:
        dy3 = torch.empty(8, dtype=torch.float32, device=dev)
        ok(L.brrr_mx_matvec(h, 8, 8, P(dxq), P(dxs), P(dy3), None, None))
        assert np.array_equal(bits(dy3.cpu().numpy()), bits(y[8:16]))
    L.brrr_mxmat_free(h)


def test_mx_all_nibble_codes(L, orc, dev):
    """Every 4-bit code against every sign of activation, one code pair per byte."""
    import torch
    rows, blocks = 16, 16
    raw = np.zeros((rows * blocks, 17), np.uint8)
    raw[:, 0] = 128
    codes = np.arange(256, dtype=np.uint8)
    raw[:, 1:] = np.resize(codes, (rows * blocks, 16))
    raw = raw.reshape(-1)
    x = np.resize(np.array([127, -127, 1, -1, 64, -3, 0, 5], np.float32), blocks * 32)
    xq, xs = orc.quant_q8(x)
    h = C.c_void_p()
    draw = to_dev(raw, dev)
    ok(L.brrr_mxmat_from_gguf(P(draw), rows, blocks, C.byref(h), None))
    dy = torch.empty(rows, dtype=torch.float32, device=dev)
    dd = torch.empty((rows, blocks, 4), dtype=torch.int32, device=dev)
    dxq, dxs = to_dev(xq, dev), to_dev(xs, dev)
    ok(L.brrr_mx_matvec(h, 0, rows, P(dxq), P(dxs), P(dy), P(dd), None))
    nib, exps = orc.repack_mx(raw, rows, blocks)
    y, dbg = orc.mx_matvec(nib, exps, rows, blocks, xq, xs, want_dbg=True)
    assert np.array_equal(dd.cpu().numpy(), dbg.transpose(0, 2, 1, 3).reshape(rows, blocks, 4))
    assert np.array_equal(bits(dy.cpu().numpy()), bits(y))
    L.brrr_mxmat_free(h)


@pytest.mark.parametrize("ne,d,topk,bias", [(32, 2880, 4, True), (8, 128, 4, True), (128, 2048, 8, False), (40, 320, 2, True)])
def test_router_topk(L, orc, dev, ne, d, topk, bias):
    import torch
    w = S.synth_f32(ne, 0, S.T["ROUTER_W"], ne * d).reshape(ne, d)
    b = S.synth_f32(ne, 0, S.T["ROUTER_B"], ne) if bias else None
    if bias:
        w[3] = w[7]; b[3] = b[7]          # exact tie between two experts
    xn = S.synth_input(d, d)
    dl = torch.empty(ne, dtype=torch.float32, device=dev)
    dt = torch.empty(topk, dtype=torch.int32, device=dev)
    dwt = torch.empty(topk, dtype=torch.float32, device=dev)
    db = to_dev(b, dev) if bias else None
    dw, dxn = to_dev(w, dev), to_dev(xn, dev)
    for _ in range(2):   # second call checks the self-resetting arrival counter
        ok(L.brrr_router_topk(P(dw), P(db) if bias else None, P(dxn), ne, d, topk, P(dl), P(dt), P(dwt), None))
        torch.cuda.synchronize()
    logits, top, wts = orc.router_topk(w, b, xn, topk)
    assert np.array_equal(bits(dl.cpu().numpy()), bits(logits))
    assert np.array_equal(dt.cpu().numpy(), top)
    assert np.array_equal(bits(dwt.cpu().numpy()), bits(wts))


def test_swiglu_quant(L, orc, dev):
    import torch
    topk, d = 4, 2880
    gu = S.synth_input(77, topk * 2 * d) * np.float32(4.0)
    gu[:8] = [7.0, 7.5, -7.0, -30.0, 0.0, 100.0, -100.0, 6.999]
    dq = torch.empty((topk, d), dtype=torch.int8, device=dev)
    ds = torch.empty((topk, d // 32), dtype=torch.float32, device=dev)
    dgu = to_dev(gu, dev)
    ok(L.brrr_swiglu_quant(P(dgu), topk, d, P(dq), P(ds), None))
    hq, hs, _ = orc.swiglu_quant(gu, topk, d)
    assert np.array_equal(dq.cpu().numpy(), hq) and np.array_equal(bits(ds.cpu().numpy()), bits(hs))


@pytest.mark.parametrize("pos,start", [(0, 0), (5, 0), (128, 0), (129, 0), (200, 0), (200, 73), (300, 173), (1500, 0), (4095, 0), (4095, 3968)])
def test_attention_decode(L, orc, brrr, dev, pos, start):
    """RoPE + cache append + sink softmax + Q8 of the output, all heads, vs the oracle per head."""
    import torch
    nh, nkv, hd = 16, 4, 64
    cfg = brrr.make_cfg(nh * hd, 1, nh, nkv, 8, 4, 512)
    tab = np.empty((4096, 32, 2), np.float32)
    ok(L.brrr_rope_table(C.byref(cfg), tab.ctypes.data))
    ocfg = orc.make_cfg(d=nh * hd, nh=nh, nkv=nkv, hd=hd, nl=1, ne=8, topk=4, nvocab=512)
    assert np.array_equal(bits(tab), bits(orc.rope_table(ocfg)))
    rng = np.random.default_rng(pos)
    kc = np.zeros((4096, nkv, hd), np.float32); vc = np.zeros((4096, nkv, hd), np.float32)   # oracle layout [pos][kv head][64]
    kc[:pos] = rng.standard_normal((pos, nkv, hd)); vc[:pos] = rng.standard_normal((pos, nkv, hd))
    qkv = rng.standard_normal((nh + 2 * nkv) * hd).astype(np.float32)
    sinks = rng.standard_normal(nh).astype(np.float32)
    dkc, dvc = to_dev(kc.transpose(1, 0, 2), dev), to_dev(vc.transpose(1, 0, 2), dev)   # engine layout [kv head][pos][64]
    dao = torch.empty(nh * hd, dtype=torch.float32, device=dev)
    daq = torch.empty(nh * hd, dtype=torch.int8, device=dev)
    das = torch.empty(nh * hd // 32, dtype=torch.float32, device=dev)
    dqkv, dtab, dsinks = to_dev(qkv, dev), to_dev(tab, dev), to_dev(sinks, dev)
    ok(L.brrr_attn_decode(P(dqkv), P(dkc), P(dvc), P(dtab), P(dsinks), nh, nkv, pos, start, P(dao), P(daq), P(das), None))
    # oracle: rotate q and k, append, attend
    q = qkv[:nh * hd].reshape(nh, hd).copy(); k = qkv[nh * hd:(nh + nkv) * hd].reshape(nkv, hd).copy()
    v = qkv[(nh + nkv) * hd:].reshape(nkv, hd)
    Lo = orc.lib()
    for hh in range(nh):
        Lo.orc_rope_apply(q[hh].ctypes.data_as(C.c_void_p), tab.ctypes.data_as(C.c_void_p), C.c_int(pos), C.c_int(hd))
    for hh in range(nkv):
        Lo.orc_rope_apply(k[hh].ctypes.data_as(C.c_void_p), tab.ctypes.data_as(C.c_void_p), C.c_int(pos), C.c_int(hd))
    kc[pos] = k; vc[pos] = v
    ao = np.concatenate([orc.attn_head(q[hh], kc, vc, nkv, hd, hh // (nh // nkv), start, pos, float(sinks[hh])) for hh in range(nh)])
    aq, asb = orc.quant_q8(ao)
    assert np.array_equal(bits(dkc.cpu().numpy()[:, pos]), bits(k)) and np.array_equal(bits(dvc.cpu().numpy()[:, pos]), bits(v))
    assert np.array_equal(bits(dao.cpu().numpy()), bits(ao))
    assert np.array_equal(daq.cpu().numpy(), aq) and np.array_equal(bits(das.cpu().numpy()), bits(asb))


@pytest.mark.parametrize("kind,type_,n", [("BQ", 0, 4096), ("ATTN_NORM", 0, 2880), ("SINKS", 0, 64), ("WQ", 30, 64 * 2880), ("GATE", 39, 32 * 2880)])
def test_synth_device_equals_numpy(L, dev, kind, type_, n):
    import torch
    nbytes = {0: n * 4, 30: n * 2, 39: n // 32 * 17}[type_]
    out = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    ok(L.brrr_synth_tensor(5, 3, S.T[kind], type_, n, P(out), None))
    got = out.cpu().numpy()
    if type_ == 0:
        want = S.synth_f32(5, 3, S.T[kind], n).view(np.uint8)
    elif type_ == 30:
        want = S.synth_bf16(5, 3, S.T[kind], n).view(np.uint8)
    else:
        want = S.synth_mxfp4(5, 3, S.T[kind], n // 32)
    assert np.array_equal(got, want)


def _fold_case(dev, d, topk, ne, seed):
    import torch
    rng = np.random.default_rng(seed)
    dpad = (d + 127) // 128 * 128
    x = rng.standard_normal(d).astype(np.float32) * np.float32(3.0)
    part = rng.standard_normal((topk, dpad)).astype(np.float32)
    bias = (rng.standard_normal((ne, d)) * 0.02).astype(np.float32)
    top = rng.permutation(ne)[:topk].astype(np.int32)
    wts = rng.random(topk).astype(np.float32)
    wts /= wts.sum(dtype=np.float32)
    w = (1.0 + 0.02 * rng.standard_normal(d)).astype(np.float32)
    want = x.copy()
    for k in range(topk):                       # multiply, then add, slot by slot (float32 at every step)
        want = want + wts[k] * (part[k, :d] + bias[top[k]])
    dv = dict(x=to_dev(x, dev), part=to_dev(part, dev), bias=to_dev(bias, dev), top=to_dev(top, dev), wts=to_dev(wts, dev), w=to_dev(w, dev),
              q=torch.empty(d, dtype=torch.int8, device=dev), s=torch.empty(d // 32, dtype=torch.float32, device=dev))
    return dv, want.astype(np.float32), w


@pytest.mark.parametrize("d,topk,ne", [(2880, 4, 32), (128, 4, 8), (2048, 8, 128), (4096, 2, 4)])
def test_fold_norm_stage(L, orc, dev, d, topk, ne):
    """The decode step's last kernel of a layer (fold with the exact routing, next RMS norm, Q8 image)
    against a float32 numpy fold followed by the oracle's norm and quantiser; also without the norm."""
    dv, want, w = _fold_case(dev, d, topk, ne, 5)
    ok(L.brrr_fold_norm(P(dv["top"]), P(dv["wts"]), topk, d, P(dv["part"]), P(dv["bias"]), P(dv["x"]), P(dv["w"]), C.c_float(1e-5),
                        P(dv["q"]), P(dv["s"]), 0, None))
    assert np.array_equal(bits(dv["x"].cpu().numpy()), bits(want))
    q, s = orc.quant_q8(orc.rmsnorm(want, w, 1e-5))
    assert np.array_equal(dv["q"].cpu().numpy(), q) and np.array_equal(bits(dv["s"].cpu().numpy()), bits(s))
    dv2, want2, _ = _fold_case(dev, d, topk, ne, 6)
    ok(L.brrr_fold_norm(P(dv2["top"]), P(dv2["wts"]), topk, d, P(dv2["part"]), P(dv2["bias"]), P(dv2["x"]), None, C.c_float(0.0), None, None, 0, None))
    assert np.array_equal(bits(dv2["x"].cpu().numpy()), bits(want2))


def test_fold_wait_runs_out_and_reports(L, dev):
    """The fold of the decode step waits for the router's routing words with a limit.  Here nothing
    publishes them: the kernel gives up after about a second, records the failure in its state word and
    returns; the call reports BRRR_ERR_STATE, and the context keeps working (the next call passes)."""
    import time
    dv, want, _ = _fold_case(dev, 256, 4, 8, 7)
    t0 = time.time()
    st = L.brrr_fold_norm(P(dv["top"]), P(dv["wts"]), 4, 256, P(dv["part"]), P(dv["bias"]), P(dv["x"]), P(dv["w"]), C.c_float(1e-5),
                          P(dv["q"]), P(dv["s"]), 1, None)
    assert st == 6, st          # BRRR_ERR_STATE
    assert time.time() - t0 < 30
    dv, want, _ = _fold_case(dev, 256, 4, 8, 8)
    ok(L.brrr_fold_norm(P(dv["top"]), P(dv["wts"]), 4, 256, P(dv["part"]), P(dv["bias"]), P(dv["x"]), P(dv["w"]), C.c_float(1e-5),
                        P(dv["q"]), P(dv["s"]), 0, None))
    assert np.array_equal(bits(dv["x"].cpu().numpy()), bits(want))


def test_attention_block_against_reference_script_fixture(L, orc, brrr, dev):
    """The CUDA attention block (brrr_rmsnorm_quant -> brrr_q8_matvec q/k/v + bias -> brrr_attn_decode
    with a plain NeoX table -> brrr_q8_matvec o-proj + bias) on the input and cache of
    scripts/attn_reference.py of the reference (fixture tests/golden/attn_ref, made by running that
    script): bit-identical to the oracle's block, and within the same bounds of the script's float64
    output (cosine > 0.9998, relative L2 < 2e-2; the reference's own bar for an int8 path is
    cosine > 0.999, src/bin/ffn_quant.rs:119-129)."""
    import torch
    import test_oracle as TO
    fx = TO._attn_ref_fixture()
    want, o = TO.attn_block_oracle(orc, 78, fx)
    nh, nkv, hd, d, T = 64, 8, 64, 2880, 8
    seed = 78
    f32 = lambda kind, n: S.synth_f32(seed, 0, S.T[kind], n)
    mats = []
    for kind, rows, cols in (("WQ", nh * hd, d), ("WK", nkv * hd, d), ("WV", nkv * hd, d), ("WO", d, nh * hd)):
        dw = to_dev(S.synth_bf16(seed, 0, S.T[kind], rows * cols), dev)
        h = C.c_void_p()
        ok(L.brrr_q8mat_from_bf16(P(dw), rows, cols, C.byref(h), None))
        torch.cuda.synchronize()
        mats.append(h)
    dx, dw = to_dev(fx["h"], dev), to_dev(f32("ATTN_NORM", d), dev)
    dq = torch.empty(d, dtype=torch.int8, device=dev); ds = torch.empty(d // 32, dtype=torch.float32, device=dev)
    ok(L.brrr_rmsnorm_quant(P(dx), P(dw), C.c_float(1e-5), d, None, P(dq), P(ds), None))
    assert np.array_equal(dq.cpu().numpy(), o["xq"]) and np.array_equal(bits(ds.cpu().numpy()), bits(o["xs"]))
    dqkv = torch.empty((nh + 2 * nkv) * hd, dtype=torch.float32, device=dev)
    off = 0
    for h, kind, rows in zip(mats[:3], ("BQ", "BK", "BV"), (nh * hd, nkv * hd, nkv * hd)):
        dy = torch.empty(rows, dtype=torch.float32, device=dev)
        ok(L.brrr_q8_matvec(h, P(dq), P(ds), P(dy), None))
        torch.cuda.synchronize()
        dqkv[off:off + rows] = dy + to_dev(f32(kind, rows), dev)
        off += rows
    kc = np.zeros((nkv, 4096, hd), np.float32); vc = np.zeros((nkv, 4096, hd), np.float32)       # engine layout [kv head][pos][64]
    kc[:, :T] = fx["kcache"].reshape(T, nkv, hd).transpose(1, 0, 2); vc[:, :T] = fx["vcache"].reshape(T, nkv, hd).transpose(1, 0, 2)
    dkc, dvc, dtab, dsinks = to_dev(kc, dev), to_dev(vc, dev), to_dev(o["tab"], dev), to_dev(o["sinks"], dev)
    dao = torch.empty(nh * hd, dtype=torch.float32, device=dev)
    daq = torch.empty(nh * hd, dtype=torch.int8, device=dev); das = torch.empty(nh * hd // 32, dtype=torch.float32, device=dev)
    ok(L.brrr_attn_decode(P(dqkv), P(dkc), P(dvc), P(dtab), P(dsinks), nh, nkv, T, 0, P(dao), P(daq), P(das), None))
    torch.cuda.synchronize()
    assert np.array_equal(bits(dao.cpu().numpy()), bits(o["ao"]))
    assert np.array_equal(daq.cpu().numpy(), o["aq"])
    dy = torch.empty(d, dtype=torch.float32, device=dev)
    ok(L.brrr_q8_matvec(mats[3], P(daq), P(das), P(dy), None))
    torch.cuda.synchronize()
    y = (dy + to_dev(f32("BO", d), dev)).cpu().numpy()
    assert np.array_equal(bits(y), bits(want))
    cos, rel = TO.attn_ref_agreement(y, fx["attn_yref"])
    assert cos > 0.9998 and rel < 2e-2, (cos, rel)
    for h in mats:
        L.brrr_q8mat_free(h)
