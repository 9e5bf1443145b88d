"""Expert parallelism.  CPU: the sharding rule and the handle exchange under a 2-rank gloo group.
GPU: the expert-parallel kernels with a single rank (self-exchange) against the oracle in the
ordinary GPU suite, and 2 ranks on 2 GPUs (skipped where fewer are visible)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import bits
from cpubrrr_b200 import synth as S

HERE = os.path.dirname(os.path.abspath(__file__))


def test_expert_range_rule():
    from cpubrrr_b200.ep import expert_range
    assert [expert_range(128, r, 8) for r in range(8)] == [(16 * r, 16) for r in range(8)]
    assert expert_range(32, 1, 2) == (16, 16) and expert_range(32, 0, 1) == (0, 32)
    for bad in ((32, 0, 3), (32, 2, 2), (32, 0, 16), (32, -1, 2)):
        with pytest.raises(ValueError):
            expert_range(*bad)


def _gloo_rank(rank, world, port, q):
    import torch.distributed as dist
    from cpubrrr_b200.ep import gather_handles
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    handle = bytes([(rank * 64 + i) % 251 for i in range(64)])
    q.put((rank, gather_handles(handle, rank, world, dist)))
    dist.barrier()
    dist.destroy_process_group()


def test_handle_exchange_two_ranks_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    ps = [ctx.Process(target=_gloo_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in ps:
        p.join(60)
        assert p.exitcode == 0
    want = b"".join(bytes([(r * 64 + i) % 251 for i in range(64)]) for r in range(2))
    assert got[0] == got[1] == want and len(want) == 128


def _ocfg(orc, c):
    return orc.make_cfg(d=c.n_embd, nh=c.n_head, nkv=c.n_head_kv, hd=c.head_dim, nl=c.n_layer, ne=c.n_expert,
                        topk=c.n_expert_used, nvocab=c.n_vocab, swa=c.sliding_window, rope_base=c.rope_freq_base, rms_eps=c.rms_eps)


def _oracle_run(orc, cfg, seed, nsteps):
    om = orc.Model.synth(_ocfg(orc, cfg), seed)
    prompt = S.synth_prompt(seed, 9, cfg.n_vocab)
    tok = 0
    for i, t in enumerate(prompt):
        tok = om.run(int(t), i, i == len(prompt) - 1)
    first, out, pos = tok, [], len(prompt)
    for _ in range(nsteps):
        tok = om.run(tok, pos, True); pos += 1
        out.append(tok)
    return first, out, om


@pytest.mark.gpu
def test_ep_single_rank_equals_oracle(brrr, orc):
    """world = 1: the expert-parallel step (slices published to and read from the rank's own
    exchange region, step hand-shake with itself) is bit-identical to the oracle."""
    from cpubrrr_b200 import ep
    cfg = brrr.make_cfg(128, 3, 4, 2, 8, 4, 512, sliding_window=16)
    eng = ep.open_synth_ep(cfg, 51, 0, 1)
    first, want, om = _oracle_run(orc, cfg, 51, 40)
    prompt = S.synth_prompt(51, 9, cfg.n_vocab)
    assert eng.prefill(prompt) == first
    assert [int(t) for t in eng.decode(first, len(prompt), 40)] == want
    assert np.array_equal(bits(eng.hidden()), bits(om.hidden()))
    assert np.array_equal(bits(eng.logits()), bits(om.logits()))
    eng.close()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_ep_multi_rank_equals_oracle(brrr, orc, tmp_path, world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    shape = dict(n_embd=128, n_layer=3, n_head=4, n_head_kv=2, n_expert=8, n_expert_used=4, n_vocab=512, sliding_window=16)
    cfg = brrr.make_cfg(**shape)
    seed, nsteps = 53, 48
    first, want, om = _oracle_run(orc, cfg, seed, nsteps)
    port = 29600 + os.getpid() % 2000
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), os.path.join(HERE, "ep_worker.py"), str(tmp_path), json.dumps(shape), str(seed), str(nsteps)],
                       capture_output=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr.decode()[-3000:]
    for rank in range(world):
        res = json.load(open(tmp_path / f"rank{rank}.json"))
        assert res["first"] == first and res["tokens"] == want, f"rank {rank}"
        assert res["hidden_bits"] == [int(b) for b in bits(om.hidden())], f"rank {rank}"
        assert res["logit_bits"] == [int(b) for b in bits(om.logits())[:64]], f"rank {rank}"


@pytest.mark.gpu
def test_ep_stalled_peer_is_reported_not_hung(brrr, orc, tmp_path):
    """Two ranks attach; after the prompt the second one stops issuing steps (alive, memory mapped).
    The first rank's next step waits (bounded, about ten seconds) for the row sums of the experts the
    stalled rank owns, gives up, and the call returns BRRR_ERR_STATE; its CUDA context still works.
    No kernel faults or hangs; NVLS is off and the exchange uses plain peer stores."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    shape = dict(n_embd=128, n_layer=3, n_head=4, n_head_kv=2, n_expert=8, n_expert_used=4, n_vocab=512, sliding_window=16)
    port = 29600 + (os.getpid() + 7) % 2000
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), os.path.join(HERE, "ep_worker.py"), str(tmp_path), json.dumps(shape), "53", "0", "stall"],
                       capture_output=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr.decode()[-3000:]
    res = json.load(open(tmp_path / "rank0.json"))
    assert res["error"] is not None and "not valid in the current state" in res["error"], res
    assert 5.0 < res["seconds"] < 60.0, res
    assert res["small_ok"]
