"""Child process of the GPU tests that need the test-hook build of the library (libbrrr_hooks.so,
-DBRRR_TEST_HOOKS): the parent sets BRRR_LIBRARY to it, so this process loads it instead of the
default build, which contains no hook.  No GPU fault is provoked: a missed speculation is a
flagged step, a silent router is a bounded wait that runs out and is reported.

    python tests/hooks_worker.py sabotage | mute
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def greedy(run, prompt, n):
    tok = 0
    for i, t in enumerate(prompt):
        tok = run(int(t), i, i == len(prompt) - 1)
    out, pos = [], len(prompt)
    for _ in range(n):
        out.append(tok)
        tok = run(tok, pos, True)
        pos += 1
    return out


def main(mode):
    assert os.environ.get("BRRR_LIBRARY", "").endswith("libbrrr_hooks.so")
    import cpubrrr_b200 as B
    from cpubrrr_b200 import synth as S
    from oracle import oracle as O
    bits = lambda a: np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    cfg = B.make_cfg(128, 2, 4, 2, 8, 4, 512, sliding_window=8)
    om = O.Model.synth(O.make_cfg(d=128, nh=4, nkv=2, hd=64, nl=2, ne=8, topk=4, nvocab=512, swa=8), 17)
    prompt = S.synth_prompt(17, 9, 500)
    want = greedy(om.run, prompt, 40)
    if mode == "sabotage":
        # the estimate is spoiled on every third position: those steps are flagged and run again
        os.environ["BRRR_SPEC_SABOTAGE"] = "1"
        eng = B.Engine.synth(cfg, 17)
        del os.environ["BRRR_SPEC_SABOTAGE"]
        assert greedy(eng.run, prompt, 40) == want                  # host-driven steps
        assert np.array_equal(bits(eng.logits()), bits(om.logits()))
        first = eng.prefill(prompt)
        toks = eng.decode(first, len(prompt), 40)                   # device-chained run with redos inside
        assert [first] + [int(t) for t in toks[:-1]] == want
        assert eng.spec_redos() > 10 and eng.wait_fallbacks() == 0
        clean = B.Engine.synth(cfg, 17)                             # without the hook the estimate practically never misses
        assert greedy(clean.run, prompt, 40) == want and clean.spec_redos() == 0
        eng.close(); clean.close()
    elif mode == "mute":
        # the exact router never publishes: the fold's bounded wait (about a second) runs out in the
        # first speculative step; the host re-runs that step with the plain graph, stops speculating
        # on this model, and every result is still the oracle's
        os.environ["BRRR_ROUTER_MUTE"] = "1"
        eng = B.Engine.synth(cfg, 17)
        del os.environ["BRRR_ROUTER_MUTE"]
        assert greedy(eng.run, prompt, 40) == want
        assert np.array_equal(bits(eng.logits()), bits(om.logits()))
        assert eng.wait_fallbacks() == 1
        first = eng.prefill(prompt)
        toks = eng.decode(first, len(prompt), 40)
        assert [first] + [int(t) for t in toks[:-1]] == want and eng.wait_fallbacks() == 1
        eng.close()
        # the same through the device-chained loop first (the recovery inside brrr_decode_wait)
        os.environ["BRRR_ROUTER_MUTE"] = "1"
        eng = B.Engine.synth(cfg, 17)
        del os.environ["BRRR_ROUTER_MUTE"]
        tok = 0
        for i, t in enumerate(prompt):
            tok = om.run(int(t), i, True)       # (oracle state only)
        first = eng.prefill(prompt)
        assert first == want[0]
        toks = eng.decode(first, len(prompt), 12)
        assert [first] + [int(t) for t in toks[:-1]] == want[:12]
        assert eng.wait_fallbacks() == 1
        eng.close()
    else:
        raise SystemExit("mode?")
    print("hooks_worker ok:", mode)


if __name__ == "__main__":
    main(sys.argv[1])
