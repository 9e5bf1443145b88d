"""Token-tile MXFP4 matmul on the tcgen05 tensor cores (brrr_mx_matmul_tile) against the CPU oracle:
every output must equal the per-token expert matvec bit for bit (0 ulp), for any number of tokens
in the tile (1..512: four entries per CTA up to 16 tokens, eight up to 64, sixteen beyond), ragged row counts and row
windows."""
import ctypes as C

import numpy as np
import pytest

from conftest import bits, to_dev
from cpubrrr_b200 import synth as S

pytestmark = pytest.mark.gpu


def P(t):
    return C.c_void_p(t.data_ptr())


@pytest.fixture(scope="module")
def L(brrr):
    return brrr.lib()


def _case(L, orc, dev, rows, blocks, ntok, row0=0, nrows=None, wide_exponents=False):
    import torch
    nrows = rows - row0 if nrows is None else nrows
    raw = S.synth_mxfp4(rows + blocks + ntok, 2, S.T["GATE"], rows * blocks)
    if wide_exponents:
        r = raw.reshape(rows * blocks, 17)
        r[::5, 0] = np.arange(len(r[::5])) % 200
    h = C.c_void_p()
    draw = to_dev(raw, dev)
    assert L.brrr_mxmat_from_gguf(P(draw), rows, blocks, C.byref(h), None) == 0
    nib, exps = orc.repack_mx(raw, rows, blocks)
    xq = np.empty((ntok, blocks * 32), np.int8); xs = np.empty((ntok, blocks), np.float32)
    want = np.empty((ntok, rows), np.float32)
    for t in range(ntok):
        x = S.synth_input(100 + t, blocks * 32) * np.float32(0.5 + t)
        if t == 1:
            x[:64] = 0.0                      # all-zero blocks
        xq[t], xs[t] = orc.quant_q8(x)
        want[t] = orc.mx_matvec(nib, exps, rows, blocks, xq[t], xs[t])
    dxq, dxs = to_dev(xq, dev), to_dev(xs, dev)
    ldy = nrows + 3
    dy = torch.full((ntok, ldy), 7.0, dtype=torch.float32, device=dev)
    assert L.brrr_mx_matmul_tile(h, row0, nrows, P(dxq), P(dxs), ntok, P(dy), ldy, None) == 0
    torch.cuda.synchronize()
    got = dy.cpu().numpy()
    assert np.array_equal(bits(got[:, :nrows]), bits(want[:, row0:row0 + nrows]))
    assert np.all(got[:, nrows:] == 7.0)                      # nothing written beyond the row window
    L.brrr_mxmat_free(h)


@pytest.mark.parametrize("rows,blocks,ntok", [(128, 2, 16), (128, 4, 1), (256, 90, 16), (16, 2, 3), (208, 6, 5), (2880, 90, 16), (5760, 90, 7),
                                               (256, 6, 17), (2880, 90, 64), (208, 10, 41), (256, 6, 200), (128, 4, 512)])
def test_tile_equals_per_token_matvec(L, orc, dev, rows, blocks, ntok):
    _case(L, orc, dev, rows, blocks, ntok)


def test_tile_row_window_and_wide_exponents(L, orc, dev):
    _case(L, orc, dev, 320, 8, 4, row0=40, nrows=150, wide_exponents=True)
    _case(L, orc, dev, 160, 4, 16, row0=16, nrows=144)


def test_tile_bad_args(L, dev):
    import torch
    t = torch.zeros(4096, dtype=torch.uint8, device=dev)
    raw = to_dev(S.synth_mxfp4(1, 0, S.T["UP"], 16 * 2), dev)
    h = C.c_void_p()
    assert L.brrr_mxmat_from_gguf(P(raw), 16, 2, C.byref(h), None) == 0
    assert L.brrr_mx_matmul_tile(h, 0, 16, P(t), P(t), 513, P(t), 16, None) == 1
    assert L.brrr_mx_matmul_tile(h, 0, 16, P(t), P(t), 0, P(t), 16, None) == 1
    assert L.brrr_mx_matmul_tile(h, 8, 16, P(t), P(t), 1, P(t), 16, None) == 1
    assert L.brrr_mx_matmul_tile(h, 0, 16, P(t), P(t), 1, P(t), 8, None) == 1
    L.brrr_mxmat_free(h)


@pytest.mark.parametrize("ntok", [1, 5, 16, 17, 40, 64, 130, 512])
def test_moe_ffn_tile_equals_token_by_token(brrr, dev, ntok):
    """The grouped tensor-core MoE step on a tile of tokens against the per-token step (itself
    bit-identical to the oracle): routing, weights and residual outputs, at the gpt-oss-20b layer
    shape (d 2880, 32 experts top-4)."""
    import torch
    cfg = brrr.make_cfg(2880, 1, 64, 8, 32, 4, 1024)
    eng = brrr.Engine.synth(cfg, 1)
    L = brrr.lib()
    rng = np.random.default_rng(ntok)
    xn = rng.standard_normal((ntok, 2880)).astype(np.float32)
    x0 = rng.standard_normal((ntok, 2880)).astype(np.float32)
    dxn = to_dev(xn, dev)
    # token by token
    want_x = to_dev(x0, dev).clone(); want_top = torch.zeros((ntok, 4), dtype=torch.int32, device=dev)
    want_w = torch.zeros((ntok, 4), dtype=torch.float32, device=dev)
    for t in range(ntok):
        eng.moe_ffn_step(0, C.c_void_p(dxn[t].data_ptr()), C.c_void_p(want_x[t].data_ptr()), C.c_void_p(want_top[t].data_ptr()),
                         C.c_void_p(want_w[t].data_ptr()))
    # the tile
    got_x = to_dev(x0, dev).clone(); got_top = torch.zeros_like(want_top); got_w = torch.zeros_like(want_w)
    assert L.brrr_moe_ffn_tile(eng._h, 0, P(dxn), P(got_x), ntok, P(got_top), P(got_w)) == 0
    torch.cuda.synchronize()
    assert np.array_equal(got_top.cpu().numpy(), want_top.cpu().numpy())
    assert np.array_equal(bits(got_w.cpu().numpy()), bits(want_w.cpu().numpy()))
    assert np.array_equal(bits(got_x.cpu().numpy()), bits(want_x.cpu().numpy()))
    assert len(np.unique(want_top.cpu().numpy())) > min(4, ntok)          # the tokens do not all share one expert set
    eng.close()
