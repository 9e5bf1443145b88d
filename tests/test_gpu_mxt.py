"""Expert matvecs on the tensor cores in native fp4 (tcgen05.mma kind::mxf4.block_scale, kernels_mxt.cu):
the MoE FFN step through them equals the oracle bit for bit, at the gpt-oss-20b layer shape and at
ragged small shapes (partial last tile of down, partial last ring stage, one block pair), and the
decode step that uses them emits the same tokens and logits as the integer-unit kernels."""
import ctypes as C

import numpy as np
import pytest

from conftest import bits, to_dev
from cpubrrr_b200 import synth as S
from test_gpu_model import greedy, ocfg_of

pytestmark = pytest.mark.gpu


def _ffn_oracle(orc, om, ocfg, xn):
    Lo = orc.lib()
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    d, k = ocfg.d, ocfg.topk
    y = np.zeros(d, np.float32)
    top = np.zeros(k, np.int32); wts = np.zeros(k, np.float32)
    Lo.orc_moe_ffn_step(C.byref(ocfg), vp(xn), Lo.orc_layer_f32(om.h, 0, S.T["ROUTER_W"]), Lo.orc_layer_f32(om.h, 0, S.T["ROUTER_B"]),
                        Lo.orc_layer_mx(om.h, 0, 0), Lo.orc_layer_mx(om.h, 0, 1), Lo.orc_layer_mx(om.h, 0, 2),
                        Lo.orc_layer_f32(om.h, 0, S.T["GATE_B"]), Lo.orc_layer_f32(om.h, 0, S.T["UP_B"]), Lo.orc_layer_f32(om.h, 0, S.T["DOWN_B"]),
                        vp(y), vp(top), vp(wts))
    return y, top, wts


@pytest.mark.parametrize("shape", [
    dict(n_embd=2880, n_layer=1, n_head=64, n_head_kv=8, n_expert=32, n_expert_used=4, n_vocab=256),     # gpt-oss-20b layer
    dict(n_embd=64, n_layer=1, n_head=2, n_head_kv=1, n_expert=4, n_expert_used=2, n_vocab=256),         # one block pair, half a down tile
    dict(n_embd=320, n_layer=1, n_head=10, n_head_kv=2, n_expert=8, n_expert_used=8, n_vocab=256),       # 5 pairs: ragged stage, ragged down tile
    dict(n_embd=1024, n_layer=1, n_head=16, n_head_kv=4, n_expert=6, n_expert_used=1, n_vocab=256),      # top-1, 16 pairs: ring wraps
])
def test_moe_ffn_step_tensor_cores_bit_exact(brrr, orc, dev, shape):
    import torch
    cfg = brrr.make_cfg(**shape)
    d, k = cfg.n_embd, cfg.n_expert_used
    eng = brrr.Engine.synth(cfg, 5)
    assert eng.uses_tensor_experts
    ocfg = ocfg_of(orc, cfg)
    om = orc.Model.synth(ocfg, 5)
    for trial in range(3):
        x = S.synth_input(10 + trial, d)
        xn = orc.rmsnorm(x, np.ones(d, np.float32), 1e-5) * np.float32(1.0 + 3.0 * trial)
        want_y, want_top, want_w = _ffn_oracle(orc, om, ocfg, xn)
        dy = torch.zeros(d, dtype=torch.float32, device=dev)
        dt = torch.zeros(k, dtype=torch.int32, device=dev); dw = torch.zeros(k, dtype=torch.float32, device=dev)
        dxn = to_dev(xn, dev)
        torch.cuda.synchronize()
        P = lambda t: C.c_void_p(t.data_ptr())
        eng.moe_ffn_step_tc(0, P(dxn), P(dy), P(dt), P(dw))
        assert np.array_equal(dt.cpu().numpy(), want_top)
        assert np.array_equal(bits(dw.cpu().numpy()), bits(want_w))
        assert np.array_equal(bits(dy.cpu().numpy()), bits(want_y))
        # and the integer-unit kernels give the same bits
        dy2 = torch.zeros(d, dtype=torch.float32, device=dev)
        eng.moe_ffn_step(0, P(dxn), P(dy2), P(dt), P(dw))
        assert np.array_equal(bits(dy2.cpu().numpy()), bits(want_y))
    # the fold adds onto what the residual already holds, and the arrival counters are back at zero
    dy = to_dev(x, dev)
    eng.moe_ffn_step_tc(0, P(dxn), P(dy), None, None)
    eng.moe_ffn_step_tc(0, P(dxn), P(dy), None, None)
    ref = to_dev(x, dev)
    eng.moe_ffn_step(0, P(dxn), P(ref), None, None)
    eng.moe_ffn_step(0, P(dxn), P(ref), None, None)
    assert np.array_equal(bits(dy.cpu().numpy()), bits(ref.cpu().numpy()))
    eng.close()


def test_worst_case_magnitudes_stay_exact(brrr, orc, dev):
    """Activation bytes at +-127 in every position (digits 3, -3, -1 / -3, 3, 1) against all weight codes:
    the largest partial sums the digit planes can produce."""
    import torch
    cfg = brrr.make_cfg(n_embd=256, n_layer=1, n_head=4, n_head_kv=2, n_expert=4, n_expert_used=4, n_vocab=256)
    eng = brrr.Engine.synth(cfg, 9)
    ocfg = ocfg_of(orc, cfg)
    om = orc.Model.synth(ocfg, 9)
    rng = np.random.default_rng(3)
    P = lambda t: C.c_void_p(t.data_ptr())
    for trial in range(4):
        sign = rng.integers(0, 2, 256) * 2 - 1
        xn = (sign * (1.0 + 0.001 * (trial == 3) * rng.random(256))).astype(np.float32)     # every |x| equal: every byte +-127
        want_y, want_top, _ = _ffn_oracle(orc, om, ocfg, xn)
        dy = torch.zeros(256, dtype=torch.float32, device=dev)
        eng.moe_ffn_step_tc(0, P(to_dev(xn, dev)), P(dy), None, None)
        assert np.array_equal(bits(dy.cpu().numpy()), bits(want_y))
    eng.close()


def test_decode_same_with_and_without_tensor_experts(brrr, orc, monkeypatch):
    cfg = brrr.make_cfg(n_embd=256, n_layer=3, n_head=8, n_head_kv=4, n_expert=16, n_expert_used=4, n_vocab=1024)
    prompt = S.synth_prompt(4, 9, cfg.n_vocab)
    eng = brrr.Engine.synth(cfg, 4)
    assert eng.uses_tensor_experts
    got = greedy(eng.run, prompt, 64)
    lg = eng.logits()
    eng.close()
    monkeypatch.setenv("BRRR_NOMXT", "1")
    old = brrr.Engine.synth(cfg, 4)
    assert not old.uses_tensor_experts
    assert greedy(old.run, prompt, 64) == got
    assert np.array_equal(bits(old.logits()), bits(lg))
    old.close()
    om = orc.Model.synth(ocfg_of(orc, cfg), 4)
    assert greedy(om.run, prompt, 64) == got
    assert np.array_equal(bits(om.logits()), bits(lg))
