"""brrr_router_topk_noalloc: the router entry point for callers that cannot allocate device
memory (all HBM already in the host's own pools, or a request path that must avoid the driver's
allocation lock).  Its scratch is a fixed array inside the library, shared by every call, so the
test runs two calls back to back with different shapes and checks each against the ordinary
brrr_router_topk bit for bit (the tolerance the other router tests use: zero)."""
import ctypes as C

import numpy as np
import pytest

from conftest import bits, to_dev
from cpubrrr_b200 import synth as S

pytestmark = pytest.mark.gpu


def P(t):
    return C.c_void_p(t.data_ptr())


def run(L, fn, w, b, xn, topk, dev):
    import torch
    ne, d = w.shape
    dw, dxn = to_dev(w, dev), to_dev(xn, dev)
    db = to_dev(b, dev) if b is not None else None
    dl = torch.zeros(ne, dtype=torch.float32, device=dev)
    dt = torch.zeros(topk, dtype=torch.int32, device=dev)
    dwt = torch.zeros(topk, dtype=torch.float32, device=dev)
    st = fn(P(dw), P(db) if b is not None else None, P(dxn), ne, d, topk, P(dl), P(dt), P(dwt), None)
    assert st == 0, st
    torch.cuda.synchronize()
    return dl.cpu().numpy(), dt.cpu().numpy(), dwt.cpu().numpy()


def test_router_noalloc_matches_router_two_calls_in_a_row(brrr, dev):
    L = brrr.lib()
    cases = [(128, 2880, 8, True), (32, 2880, 4, True), (8, 128, 4, False), (128, 4096, 4, True)]
    for ne, d, topk, bias in cases:           # consecutive calls: bigger shape first, so stale scratch would show
        w = S.synth_f32(ne + d, 0, S.T["ROUTER_W"], ne * d).reshape(ne, d)
        b = S.synth_f32(ne + d, 0, S.T["ROUTER_B"], ne) if bias else None
        xn = S.synth_input(ne + d, d)
        got = run(L, L.brrr_router_topk_noalloc, w, b, xn, topk, dev)
        want = run(L, L.brrr_router_topk, w, b, xn, topk, dev)
        assert np.array_equal(bits(got[0]), bits(want[0]))
        assert np.array_equal(got[1], want[1])
        assert np.array_equal(bits(got[2]), bits(want[2]))


def test_router_noalloc_rejects_sizes_beyond_its_scratch(brrr, dev):
    import torch
    L = brrr.lib()
    t = torch.zeros(16, dtype=torch.float32, device=dev)
    ti = torch.zeros(16, dtype=torch.int32, device=dev)
    assert L.brrr_router_topk_noalloc(P(t), None, P(t), 160, 2880, 4, P(t), P(ti), P(t), None) == 5      # BRRR_ERR_RANGE
    assert L.brrr_router_topk_noalloc(P(t), None, P(t), 32, 4160, 4, P(t), P(ti), P(t), None) == 5
    assert L.brrr_router_topk_noalloc(P(t), None, P(t), 32, 100, 4, P(t), P(ti), P(t), None) == 1        # BRRR_ERR_ARG
