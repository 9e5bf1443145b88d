#!/usr/bin/env python
"""Benchmark of the per-token MoE decode path on the gpt-oss-20b architecture.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the reference's headline measurement): gpt-oss-20b architecture, seeded synthetic
weights (MXFP4 experts, bf16 attention/embedding/unembedding quantised to Q8 at load), a 73-token
random-id prompt, then K greedy decode steps from position 73 (K = 128 reproduces pos 73 -> 201).
One "step" is one decoded token.  Every step streams ~2.66 GB of weights, far more than the
126 MB L2, so no explicit L2 flush is needed between steps.

`value` is tokens/s with the token id chained on the device (inputs resident in HBM), timed with
CUDA events on the engine's stream; `e2e` drives every step through Engine.run(tok, pos) with a
host token in and a host token out.  With --gpus N > 1 (launched by torchrun) every rank decodes
its own sequence on its own GPU (independent replicas, no data-path collective); the time is the
maximum over ranks.

--impl reference times the CPU restatement of the reference's algorithm (oracle/, kind "port":
the reference itself is Rust + aarch64 NEON and cannot be built here) on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_LEN = 73
SEED = 2
WORKLOAD = "gpt-oss-20b decode, 73-token prompt, batch 1, greedy"
METRIC = "batch-1 decode tok/s (gpt-oss-20b shape, MXFP4)"
ARCH = "24 layers, d 2880, 64/8 heads x 64, 32 experts top-4, vocab 201088"
DTYPE = "int8xfp4->int32,f32"
TOK_BOUND = 199999


def use_qwen_workload():
    """--workload qwen3-30b-a3b: the reference's second engine (qwen3moe, K-quants) instead of the
    headline gpt-oss workload: 64-token prompt, then K decode steps."""
    global PROMPT_LEN, SEED, WORKLOAD, METRIC, ARCH, DTYPE, TOK_BOUND
    PROMPT_LEN, SEED = 64, 3
    WORKLOAD = "Qwen3-30B-A3B (qwen3moe) decode, 64-token prompt, batch 1, greedy"
    METRIC = "batch-1 decode tok/s (Qwen3-30B-A3B shape, Q4_K/Q6_K)"
    ARCH = "48 layers, d 2048, 32/4 heads x 128, 128 experts top-8 x 768, vocab 151936"
    DTYPE = "int8 x (4|6)-bit->int32,f32"
    TOK_BOUND = 151936


def use_120b_workload():
    """--workload gptoss120b: 36 layers, 128 experts top-4; meant for --parallel ep over 1/2/4/8 GPUs."""
    global WORKLOAD, METRIC, ARCH
    WORKLOAD = "gpt-oss-120b decode, 73-token prompt, batch 1, greedy"
    METRIC = "batch-1 decode tok/s (gpt-oss-120b shape, MXFP4)"
    ARCH = "36 layers, d 2880, 64/8 heads x 64, 128 experts top-4, vocab 201088"


def oracle_model(qwen):
    from oracle import oracle as O
    O.build()
    if qwen:
        return O, O.QwenModel.synth(O.make_qcfg(2048, 32, 4, 128, 48, 128, 8, 768, 151936), SEED)
    return O, O.Model.synth(O.make_cfg(d=2880, nh=64, nkv=8, hd=64, nl=24, ne=32, topk=4, nvocab=201088), SEED)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.idx)],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return None
        time.sleep(0.25)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        rows = [l.strip().split(", ") for l in open(self.f.name) if l.strip()]
        os.unlink(self.f.name)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); smax.append(float(r[2]))
            except ValueError:
                continue
            for n, v in zip(names, r[5:9]):
                if v.strip().lower() == "active":
                    reasons.add(n)
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons), "samples": len(sm)}


def algorithmic_bytes(qwen, big, pos):
    """Bytes one decode step must read once in the reference's run-time formats (weights + f32 KV
    window + embedding row), the same accounting as brrr_model_bytes_per_step /
    brrr_qwen_bytes_per_step; used where no engine is open (the CPU arm)."""
    if qwen:
        d, nh, nkv, hd, nl, ne, k, ff, nv = 2048, 32, 4, 128, 48, 128, 8, 768, 151936
        q4, q6 = lambda r, c: r * (c // 256) * 144, lambda r, c: r * (c // 256) * 210
        per = q4(nh * hd, d) + 2 * q4(nkv * hd, d) + q4(d, nh * hd) + k * (2 * q4(ff, d) + q6(d, ff)) + ne * d * 4 + 2 * d * 4 + 2 * hd * 4
        return nl * (per + (pos + 1) * nkv * hd * 8) + q6(nv, d) + d * 4 + q4(1, d)
    d, nh, nkv, hd, nl, ne, k, nv, swa = 2880, 64, 8, 64, (36 if big else 24), (128 if big else 32), 4, 201088, 128
    nb = d // 32
    q8 = lambda r, c: r * c + r * (c // 32) * 4
    per = k * 3 * d * nb * 17 + q8((nh + 2 * nkv) * hd, d) + q8(d, nh * hd) + ne * d * 4 + ne * 4
    per += ((nh + 2 * nkv) * hd + d) * 4 + k * 3 * d * 4 + 2 * d * 4 + nh * 4
    tot = per * nl
    for il in range(nl):
        start = max(0, pos + 1 - swa) if (il + 1) % 2 else 0
        tot += (pos - start + 1) * nkv * hd * 8
    return tot + q8(nv, d) + d * 4 + d * 2


def config_dict(K, world, ep_mode, reduced_note=None):
    """The `config` object of the JSON line; both arms print the same one for the same arguments."""
    par = (f"expert-parallel x{world}" if ep_mode else f"replicas x{world}") if (world > 1 or ep_mode) else "single GPU"
    return {"workload": WORKLOAD if not reduced_note else reduced_note, "arch": ARCH, "positions": [PROMPT_LEN, PROMPT_LEN + K],
            "parallelism": par, "l2": "inputs larger than L2 (a step streams 2-4 GB of weights; L2 holds 126 MB)"}


def oracle_decode(m, prompt, nsteps, warm=0, want_gaps=False):
    """Prompt, `warm` untimed greedy steps from the prompt's end, then - from the prompt's end again,
    as the GPU arm does (recomputing a position overwrites its KV entries with the same values) -
    nsteps timed greedy steps on the oracle.  Returns (first token after the prompt, tokens of the
    timed steps, seconds, smallest top-1/top-2 logit gap of the timed steps or None)."""
    import numpy as np
    tok = 0
    for i, t in enumerate(prompt):
        tok = m.run(int(t), i, i == len(prompt) - 1)
    first = tok
    pos = len(prompt)
    for _ in range(warm):
        tok = m.run(tok, pos, True); pos += 1
    tok, pos, got, gap = first, len(prompt), [], None
    t0 = time.perf_counter()
    for _ in range(nsteps):
        tok = m.run(tok, pos, True); pos += 1
        got.append(tok)
        if want_gaps:
            a = np.partition(m.logits(), -2)[-2:]
            g = float(a[1] - a[0])
            gap = g if gap is None else min(gap, g)
    return first, got, time.perf_counter() - t0, gap


def run_reference(args, rank, world):
    """CPU arm: the oracle (a port of the reference's algorithm) on all host threads, same workload,
    step count and warm-up as the GPU arm.  Under a multi-rank launcher rank 0 alone runs it."""
    if rank != 0:
        return
    qwen, big = args.workload == "qwen3-30b-a3b", args.workload == "gptoss120b"
    if big:
        print(json.dumps({"impl": "reference", "unavailable": "the CPU port would need 61 GB of expert weights in host memory"}), flush=True)
        return
    cores = os.cpu_count() or 1
    O, m = oracle_model(qwen)
    threads = O.set_threads(cores)          # launchers export OMP_NUM_THREADS=1: ask for every core explicitly
    prompt = O.synth_prompt(SEED, PROMPT_LEN, TOK_BOUND)
    K = max(1, min(args.steps, 256))        # bounded: ~0.1 s per step
    warm = max(args.warmup, 3)
    first, toks, dt, _ = oracle_decode(m, prompt, K, warm)
    v = K / dt
    # one thread, two steps: the scalar figure beside the threaded one
    O.set_threads(1)
    t0 = time.perf_counter()
    tok, pos = toks[-1], PROMPT_LEN + K
    for _ in range(2):
        tok = m.run(tok, pos, True); pos += 1
    v1 = 2 / (time.perf_counter() - t0)
    O.set_threads(cores)
    by = sum(algorithmic_bytes(qwen, big, PROMPT_LEN + i) for i in range(K)) / K
    sample = f"{K} decode steps from position {PROMPT_LEN} after the {PROMPT_LEN}-token prompt (full model)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tok/s", "n_gpus": args.gpus, "steps": K, "warmup": warm,
        "ms_per_step": 1000.0 * dt / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": DTYPE,
        "data": "synthetic", "config": config_dict(K, world, False),
        "cpu_baseline": {"value": v, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample,
                         "value_1thread": v1, "gbs": by * v / 1e9, "gbs_1thread": by * v1 / 1e9},
        "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def cpu_baseline_and_parity(eng_tokens, first_tok, nsteps, qwen=False):
    """Rank 0, N = 1: time the oracle on a bounded sample of the same workload (all host threads) and
    use it as the checker of the GPU's decoded tokens."""
    O, m = oracle_model(qwen)
    cores = O.set_threads(os.cpu_count() or 1)
    prompt = O.synth_prompt(SEED, PROMPT_LEN, TOK_BOUND)
    first, got, dt, gap = oracle_decode(m, prompt, nsteps, 0, want_gaps=True)
    ok = first == first_tok and got == [int(t) for t in eng_tokens[:nsteps]]
    by = sum(algorithmic_bytes(qwen, False, PROMPT_LEN + i) for i in range(nsteps)) / nsteps
    m.close()
    return {"value": nsteps / dt, "unit": "tok/s", "cores": cores, "kind": "port", "gbs": by * nsteps / dt / 1e9,
            "sample": f"{nsteps} decode steps from position {PROMPT_LEN} after the {PROMPT_LEN}-token prompt (full model; includes reading back the logits of every step for the gap statistic)"}, \
           {"tokens_checked": nsteps + 1, "identical": bool(ok), "min_top1_top2_logit_gap": gap}


def ncu_traffic_table():
    """dram__bytes_read.sum + dram__bytes_write.sum per launch and kernel class, from the table in
    profiles/ncu_dram_traffic_per_launch.md (rows `| class | bytes | capture |`)."""
    import re
    out = {}
    p = os.path.join(ROOT, "profiles", "ncu_dram_traffic_per_launch.md")
    if os.path.exists(p):
        for line in open(p):
            m = re.match(r"\|\s*([a-z0-9_]+)\s*\|\s*([0-9.]+(?:e[0-9]+)?)\s*\|", line)
            if m:
                out[m.group(1)] = float(m.group(2))
    return out


def run_moe_tile(args):
    """--workload moe-tile: the MoE FFN stage of the gpt-oss-20b layers on token tiles (batched
    decode / prefill building block): per-token kernels against the grouped tcgen05 matmuls at tile
    sizes 1, 4 and 16.  One step = one pass of a tile through the MoE FFN of all 24 layers."""
    import ctypes as C
    import torch
    import cpubrrr_b200 as B
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    eng = B.Engine.synth(B.gptoss_20b_cfg() if args.layers == 24 else B.make_cfg(2880, args.layers, 64, 8, 32, 4, 32768), SEED)
    L = B.lib()
    nl, d = eng.cfg.n_layer, eng.cfg.n_embd
    P = lambda t: C.c_void_p(t.data_ptr())
    g = torch.Generator(device=dev); g.manual_seed(SEED)
    rows = []
    for ntok in (1, 4, 16):
        xn = torch.randn((ntok, d), device=dev, generator=g)
        x = torch.zeros((ntok, d), device=dev)

        def tile_pass():
            for il in range(nl):
                B._lib.check(L.brrr_moe_ffn_tile(eng._h, il, P(xn), P(x), ntok, None, None), "brrr_moe_ffn_tile")

        def token_pass():
            for il in range(nl):
                for t in range(ntok):
                    eng.moe_ffn_step(il, P(xn[t]), P(x[t]))

        res = {}
        for name, fn in (("tile_tcgen05", tile_pass), ("per_token", token_pass)):
            for _ in range(max(args.warmup // 4, 1)):
                fn()
            torch.cuda.synchronize()
            reps = max(args.steps // 16, 3)
            t0 = time.perf_counter()
            for _ in range(reps):
                fn()
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t0) / reps
            res[name] = {"ms_per_pass": 1000 * dt, "token_layers_per_s": ntok * nl / dt}
        rows.append({"tile_tokens": ntok, **res, "speedup": res["per_token"]["ms_per_pass"] / res["tile_tcgen05"]["ms_per_pass"]})
    best = rows[-1]["tile_tcgen05"]
    print(json.dumps({"metric": "MoE FFN stage token-layers/s (gpt-oss-20b layers, token tiles on tcgen05)", "value": best["token_layers_per_s"],
                      "unit": "token-layers/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": best["ms_per_pass"],
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xfp4->int32 (tcgen05 kind::i8),f32",
                      "data": "synthetic", "config": {"workload": "gpt-oss-20b MoE FFN stage on tiles of 1/4/16 tokens, all layers, host-synchronous calls",
                                                      "l2": "inputs larger than L2 (every pass streams the selected experts of all layers)"},
                      "tiles": rows}), flush=True)
    eng.close()


def run_batched(args):
    """--workload batched: greedy decode of b = 1, 4, 16, 64, 256 independent sequences (one KV cache each, 32-token
    prompts) through Engine.batch_step, one pass per step for all rows of the batch.  One step = one pass
    = b tokens; the clock is the host's around the calls (each returns the rows' tokens to host memory).  The
    first 16 tokens of four sequences are checked against the one-sequence engine."""
    import numpy as np
    import torch
    import cpubrrr_b200 as B
    from cpubrrr_b200 import synth as S
    torch.cuda.set_device(0)
    eng = B.Engine.synth(B.gptoss_20b_cfg() if args.layers == 24 else B.make_cfg(2880, args.layers, 64, 8, 32, 4, args.vocab), SEED)
    vmax = 199999 if args.vocab > 199999 else args.vocab - 1
    plen, nb = 32, 256
    prompts = [[int(t) for t in S.synth_prompt(SEED + 100 + i, plen, vmax)] for i in range(nb)]
    # the checker: four sequences on the one-sequence engine (token-serial schedule)
    ncheck, want = 16, []
    eng.set_tile_prefill(False)
    for s in range(4):
        tok = 0
        for i, t in enumerate(prompts[s]):
            tok = eng.run(t, i, i == plen - 1)
        w = [tok]
        for k in range(1, ncheck):
            tok = eng.run(tok, plen + k - 1, True)
            w.append(tok)
        want.append(w)
    # serial decode rate of one sequence, for scale
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    eng.decode(want[0][-1], plen + ncheck - 1, 64)
    serial_tok_s = 64 / (time.perf_counter() - t0)
    eng.batch_open(nb)
    rows, same = [], True
    steps = max(args.steps, ncheck)
    for b in (1, 4, 16, 64, 256):
        for s in range(b):
            eng.batch_prefill(s, prompts[s][:-1])
        toks = [prompts[s][-1] for s in range(b)]
        pos = [plen - 1] * b
        seqs = list(range(b))
        got = [[] for _ in range(b)]
        for k in range(max(args.warmup, 3)):                     # warm-up passes (captures the graph of this row count)
            out = eng.batch_step(toks, [p + k for p in pos], seqs) if k == 0 else eng.batch_step([int(t) for t in out], [p + k for p in pos], seqs)
            for s in range(b):
                got[s].append(int(out[s]))
        w = max(args.warmup, 3)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for k in range(w, w + steps):
            out = eng.batch_step([int(t) for t in out], [p + k for p in pos], seqs)
            for s in range(b):
                got[s].append(int(out[s]))
        dt = time.perf_counter() - t0
        for s in range(min(b, 4)):
            same = same and got[s][:ncheck] == want[s]
        rows.append({"batch": b, "tok_s": b * steps / dt, "ms_per_pass": 1000 * dt / steps, "per_sequence_tok_s": steps / dt})
    best = max(rows, key=lambda r: r["tok_s"])
    print(json.dumps({"metric": "batched decode tok/s (gpt-oss-20b shape, independent sequences)", "value": best["tok_s"], "unit": "tok/s", "n_gpus": 1,
                      "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": best["ms_per_pass"], "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "int8xfp4->int32 (tcgen05 kind::i8), int8 dp4a, f32", "data": "synthetic",
                      "config": {"workload": "gpt-oss-20b batched greedy decode, 32-token prompts, b = 1/4/16/64/256 sequences (one 403 MB KV cache each), wall clock through Engine.batch_step",
                                 "l2": "inputs larger than L2 (every pass streams the dense layers, the routed experts and the vocabulary projection)"},
                      "batches": rows, "one_sequence_decode_tok_s": serial_tok_s,
                      "parity": {"sequences_checked": 4, "tokens_each": ncheck, "identical_to_one_sequence_engine": bool(same)}}), flush=True)
    eng.close()


def run_prefill(args):
    """--workload prefill: one 2048-token prompt through Engine.run_tile (tiles of 512 tokens: q/k/v and o-proj
    per 16 rows, attention for all rows in one launch, the MoE block per tile on the tcgen05 tile kernels)
    against the token-serial schedule on a 256-token sample of the same prompt (its first 256 positions, where
    attention is cheapest: the comparison favours the serial schedule).  One step = one prompt token.  The tile
    path is checked against the serial one on the sample (same next token, same hidden state bits)."""
    import numpy as np
    import torch
    import cpubrrr_b200 as B
    from cpubrrr_b200 import synth as S
    torch.cuda.set_device(0)
    eng = B.Engine.synth(B.gptoss_20b_cfg() if args.layers == 24 else B.make_cfg(2880, args.layers, 64, 8, 32, 4, args.vocab), SEED)
    n = 2048
    prompt = [int(t) for t in S.synth_prompt(SEED, n, 199999 if args.vocab > 199999 else args.vocab - 1)]
    if args.profile_range:
        # for a profiler started with --profile-from-start off: two tiles untimed, then one tile inside the range
        tr = int(os.environ.get("BRRR_TILE_ROWS", "512"))
        eng.run_tile(prompt[:2 * tr], 0, False)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        eng.run_tile(prompt[2 * tr:3 * tr], 2 * tr, False)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profile_range": "one prompt tile", "tile_rows": tr, "layers": eng.cfg.n_layer}), flush=True)
        eng.close()
        return
    sample = 256
    # serial sample (also the checker)
    tile_rows = int(os.environ.get("BRRR_TILE_ROWS", "512"))
    eng.set_tile_prefill(True)
    eng.run_tile(prompt[:2 * tile_rows], 0, False)            # warm-up of both paths (graphs of the tile sizes in use)
    eng.run_tile(prompt[:sample % tile_rows or tile_rows], 0, False)
    for i in range(8):
        eng.run(prompt[i], i, False)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    tok_s = 0
    for i in range(sample):
        tok_s = eng.run(prompt[i], i, i == sample - 1)
    torch.cuda.synchronize()
    dt_serial = time.perf_counter() - t0
    h_s = eng.hidden().copy()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    tok_t = eng.run_tile(prompt[:sample], 0, True)
    torch.cuda.synchronize()
    dt_tile_sample = time.perf_counter() - t0
    same = bool(tok_t == tok_s and np.array_equal(eng.hidden().view(np.uint32), h_s.view(np.uint32)))
    # the full prompt on tiles
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    eng.run_tile(prompt, 0, True)
    torch.cuda.synchronize()
    dt_tile = time.perf_counter() - t0
    print(json.dumps({"metric": "prefill tok/s (gpt-oss-20b shape, one 2048-token prompt)", "value": n / dt_tile, "unit": "tok/s", "n_gpus": 1,
                      "steps": n, "warmup": 16, "ms_per_step": 1000 * dt_tile / n, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "int8xfp4->int32 (tcgen05 kind::i8),f32", "data": "synthetic",
                      "config": {"workload": f"gpt-oss-20b prefill, 2048-token prompt, tiles of {tile_rows} tokens, wall clock through Engine.run_tile",
                                 "l2": "inputs larger than L2 (every tile streams the dense layers per token and the routed experts per tile)"},
                      "serial": {"tok_s": sample / dt_serial, "sample_tokens": sample}, "tiles_on_sample": {"tok_s": sample / dt_tile_sample, "sample_tokens": sample},
                      "speedup_vs_serial_on_sample": dt_serial / dt_tile_sample, "speedup_full_prompt_vs_serial_sample": (n / dt_tile) / (sample / dt_serial),
                      "parity": {"tokens_checked": sample, "identical_to_serial": same}}), flush=True)
    eng.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline / parity leg")
    ap.add_argument("--no-stages", action="store_true", help="skip the per-kernel-class timing")
    ap.add_argument("--profile-range", action="store_true",
                    help="for ncu --profile-from-start off: cudaProfilerStart/Stop around the K timed decode steps (decode workloads), or around "
                         "one prompt tile after two untimed ones (--workload prefill, which then exits)")
    ap.add_argument("--no-ep", action="store_true", help="N > 1: skip the expert-parallel gpt-oss-120b leg")
    ap.add_argument("--workload", default="gptoss20b", choices=["gptoss20b", "gptoss120b", "qwen3-30b-a3b", "moe-tile", "prefill", "batched"],
                    help="gptoss20b is the benchmark workload; gptoss120b is the expert-parallel configuration; qwen3-30b-a3b measures the reference's second engine")
    ap.add_argument("--parallel", default="replicas", choices=["replicas", "ep"],
                    help="N > 1: independent replicas (weak scaling, default) or one sequence with the experts sharded over the ranks (strong scaling)")
    ap.add_argument("--layers", type=int, default=24, help="profiling aid: fewer layers (not the benchmark workload)")
    ap.add_argument("--vocab", type=int, default=201088, help="profiling aid: smaller vocabulary (not the benchmark workload)")
    args = ap.parse_args()
    if args.workload == "batched":
        return run_batched(args)
    if args.workload == "moe-tile":
        run_moe_tile(args)
        return
    if args.workload == "prefill":
        run_prefill(args)
        return
    qwen = args.workload == "qwen3-30b-a3b"
    big = args.workload == "gptoss120b"
    if qwen:
        use_qwen_workload()
    if big:
        use_120b_workload()
        args.no_cpu = True                  # the CPU port would need the 61 GB of expert weights in host memory
    ep_mode = args.parallel == "ep" or (big and int(os.environ.get("WORLD_SIZE", "1")) > 1)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)
    K = max(1, min(args.steps, 4096 - PROMPT_LEN - 1))

    import numpy as np
    import torch
    import cpubrrr_b200 as B
    from cpubrrr_b200 import synth as S

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    cfg = B.gptoss_20b_cfg()
    reduced = args.layers != 24 or args.vocab != 201088
    if qwen:
        full = B.qwen3_30b_a3b_cfg()
        reduced = args.layers != 24                             # --layers N: small case for profiler captures only
        cfg = B.make_qwen_cfg(2048, args.layers, 32, 4, 128, 8, 768, 151936) if reduced else full
        args.no_cpu = args.no_cpu or reduced
        args.no_stages = True
        eng = B.QwenEngine.synth(cfg, SEED, device=local_rank)
        prompt = S.synth_prompt(SEED + rank, PROMPT_LEN, TOK_BOUND)
    else:
        if big:
            reduced = args.layers != 24
            cfg = B.make_cfg(2880, args.layers if reduced else 36, 64, 8, 128, 4, 201088)
        elif reduced:                                           # small case for profiler captures only
            cfg = B.make_cfg(2880, args.layers, 64, 8, 32, 4, args.vocab)
            args.no_cpu = True
        if ep_mode:
            # one sequence, experts sharded by index over the ranks; every rank computes the same tokens
            from cpubrrr_b200 import ep
            args.no_stages = True
            eng = ep.open_synth_ep(cfg, SEED, rank, world, device=local_rank, dist=dist, torch_device=torch.device("cuda", local_rank))
            prompt = S.synth_prompt(SEED, PROMPT_LEN, min(199999, args.vocab))
        else:
            eng = B.Engine.synth(cfg, SEED, device=local_rank)
            prompt = S.synth_prompt(SEED + rank, PROMPT_LEN, min(199999, args.vocab))   # every replica decodes its own sequence
    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(x):
        if dist is None:
            return x
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def measure(eng, prompt, sample_clocks):
        """Prompt, W warm-up steps, exactly K timed device-chained steps (CUDA events on the engine's
        stream; the closing event is recorded after brrr_decode_wait, so any step the host had to
        re-run because the routing estimate missed lies inside the timed region), then the same K steps
        end to end through Engine.run.  Times are the maximum over ranks."""
        first = eng.prefill(prompt)
        stream = torch.cuda.ExternalStream(eng.stream, device=torch.device("cuda", local_rank))
        eng.decode(first, PROMPT_LEN, args.warmup)
        redos0 = eng.spec_redos() if hasattr(eng, "spec_redos") else 0
        sampler = ClockSampler(local_rank) if (rank == 0 and sample_clocks) else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        if sampler:
            sampler.start()
        if args.profile_range:
            torch.cuda.synchronize()
            torch.cuda.profiler.start()          # for ncu --profile-from-start off: exactly the K timed steps
        e0.record(stream)
        eng.decode_enqueue(first, PROMPT_LEN, K)
        toks = eng.decode_wait(K)
        e1.record(stream)
        if args.profile_range:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        barrier()
        ms = reduce_max(e0.elapsed_time(e1))
        redos = (eng.spec_redos() if hasattr(eng, "spec_redos") else 0) - redos0
        # keep the GPUs busy long enough for the clock sampler on short runs; the number of extra calls
        # is derived from the reduced time, so every rank issues the same calls (expert-parallel ranks must)
        clocks = None
        if sample_clocks:
            extra = int(max(0.0, 1.0 - ms / 1000.0) / (16 * ms / K / 1000.0)) + 1
            for _ in range(extra):
                eng.decode(first, PROMPT_LEN, 16)
            clocks = sampler.stop() if sampler else None
        # end to end through the public API: host token in, host token out, every step
        tok, pos = first, PROMPT_LEN
        for _ in range(args.warmup):
            tok = eng.run(tok, pos, True); pos += 1
        tok, pos = first, PROMPT_LEN
        barrier()
        t0 = time.perf_counter()
        for _ in range(K):
            tok = eng.run(tok, pos, True); pos += 1
        torch.cuda.synchronize()
        e2e_s = reduce_max(time.perf_counter() - t0)
        return {"first": first, "toks": toks, "ms": ms, "e2e_s": e2e_s, "redos": redos, "clocks": clocks}

    def roofline_of(eng, ms, ngpu):
        by = sum(eng.bytes_per_step(PROMPT_LEN + i) for i in range(K)) / K
        ach = by / (ms / K) / 1e6
        return {"bound": "hbm", "bytes_per_step": by, "achieved": ach, "peak": peak * ngpu, "unit": "GB/s", "frac": ach / (peak * ngpu),
                "peak_kind": peak_kind, "frac_of_8TBs": ach / (8000.0 * ngpu)}

    peak, peak_kind = measured_peaks()
    r = measure(eng, prompt, True)
    ms, toks, first = r["ms"], r["toks"], r["first"]
    nseq = 1 if ep_mode else world          # expert-parallel ranks share one sequence
    out = None
    if rank == 0:
        note = f"PROFILING CASE ({args.layers} layers, vocab {args.vocab}) - not the benchmark workload" if reduced else None
        out = {
            "metric": METRIC, "value": nseq * K / (ms / 1000.0), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": args.warmup,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong" if ep_mode else "weak", "vs_baseline": None,
            "dtype": DTYPE, "data": "synthetic", "config": config_dict(K, world, ep_mode, note),
            "e2e": {"value": nseq * K / r["e2e_s"], "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4},
            "gpu_launches": K * eng.launches_per_step(True), "spec_redos": r["redos"], "clocks": r["clocks"],
            "step_roofline": roofline_of(eng, ms, world if ep_mode else 1),
        }
        if not args.no_stages:
            mid = PROMPT_LEN + K // 2
            st = [x for x in eng.stage_times(mid, reps=10) if x[3] > 0]      # classes the step does not launch report 0 launches
            tot = sum(t * n for _, t, _, n in st)
            stages = [{"kernel": nm, "launches_per_step": n, "us_per_launch": 1000 * t, "share": t * n / tot,
                       "bytes_per_launch": by, "gbs": by / t / 1e6 if t > 0 else 0.0} for nm, t, by, n in st]
            out["stages"] = stages
            traffic = ncu_traffic_table()
            # the dominant kernel of the step: the exact router is left out, it runs on a side stream
            # beside gate/up and down and is not on the step's critical path
            top = max((x for x in stages if x["kernel"] != "norm_router_topk" or qwen), key=lambda x: x["share"])
            out["roofline"] = {"bound": "hbm", "kernel": top["kernel"], "achieved": top["gbs"], "peak": peak, "unit": "GB/s",
                               "frac": top["gbs"] / peak, "traffic": traffic.get(top["kernel"]), "peak_kind": peak_kind,
                               "bytes_per_launch": top["bytes_per_launch"], "us_per_launch": top["us_per_launch"]}
        if world == 1 and not args.no_cpu:
            cpu, parity = cpu_baseline_and_parity(toks, first, min(K, 128), qwen)
            out["cpu_baseline"] = cpu
            out["parity"] = parity
    if dist is not None:
        dist.barrier()                  # nobody frees memory its peers may still write to
    eng.close()

    # ---- N > 1, default workload: the split the path has across GPUs - gpt-oss-120b with the experts
    # sharded by index over the same ranks (one sequence, strong scaling) - reported under "ep"
    if world > 1 and not ep_mode and not qwen and not big and not reduced and not args.no_ep:
        from cpubrrr_b200 import ep
        cfg120 = B.make_cfg(2880, 36, 64, 8, 128, 4, 201088)
        if cfg120.n_expert % world == 0:
            eng = ep.open_synth_ep(cfg120, SEED, rank, world, device=local_rank, dist=dist, torch_device=torch.device("cuda", local_rank))
            prompt = S.synth_prompt(SEED, PROMPT_LEN, 199999)
            r = measure(eng, prompt, False)
            same = [int(t) for t in r["toks"]]
            agree = True
            if dist is not None:
                t = torch.tensor(same, device="cuda", dtype=torch.int64)
                lo, hi = t.clone(), t.clone()
                dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                agree = bool(torch.equal(lo, hi))
            if rank == 0:
                out["ep"] = {"workload": "gpt-oss-120b decode (36 layers, 128 experts top-4), 73-token prompt, batch 1, greedy; experts sharded by index, dense layers replicated",
                             "n_gpus": world, "scaling": "strong", "value": K / (r["ms"] / 1000.0), "unit": "tok/s", "ms_per_step": r["ms"] / K,
                             "e2e": {"value": K / r["e2e_s"], "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4},
                             "gpu_launches": K * eng.launches_per_step(True), "step_roofline": roofline_of(eng, r["ms"], world),
                             "tokens_identical_across_ranks": agree}
            dist.barrier()
            eng.close()
    if rank == 0:
        print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
