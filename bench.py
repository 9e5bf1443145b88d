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


def run_reference(args, rank, world):
    """CPU arm: the oracle (a port of the reference's algorithm) on all host threads."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    O, m = oracle_model(args.workload != "gptoss20b")
    prompt = O.synth_prompt(SEED, PROMPT_LEN, TOK_BOUND)
    tok = 0
    for i, t in enumerate(prompt):
        tok = m.run(int(t), i, i == len(prompt) - 1)
    pos = PROMPT_LEN
    # bounded sample: each call is one decode token; cap the total so the run ends within minutes
    steps = min(args.steps, 64)
    warm = min(args.warmup, 3)
    for _ in range(warm):
        tok = m.run(tok, pos, True); pos += 1
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = m.run(tok, pos, True); pos += 1
    dt = time.perf_counter() - t0
    v = steps / dt
    sample = f"{steps} decode steps from position {PROMPT_LEN + warm} after a {PROMPT_LEN}-token prompt (full model)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tok/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": 1000.0 * dt / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": DTYPE,
        "data": "synthetic", "config": {"workload": WORKLOAD, "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": v, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def cpu_baseline_and_parity(eng_tokens, first_tok, nsteps, qwen=False):
    """Rank 0, N = 1: time the oracle on a bounded sample of the same workload and use it as the
    checker of the GPU's first decoded tokens."""
    O, m = oracle_model(qwen)
    prompt = O.synth_prompt(SEED, PROMPT_LEN, TOK_BOUND)
    tok = 0
    for i, t in enumerate(prompt):
        tok = m.run(int(t), i, i == len(prompt) - 1)
    ok = tok == first_tok
    pos = PROMPT_LEN
    t0 = time.perf_counter()
    got = []
    for _ in range(nsteps):
        tok = m.run(tok, pos, True); pos += 1
        got.append(tok)
    dt = time.perf_counter() - t0
    ok = ok and got == [int(t) for t in eng_tokens[:nsteps]]
    m.close()
    return {"value": nsteps / dt, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"{nsteps} decode steps from position {PROMPT_LEN} after the {PROMPT_LEN}-token prompt (full model)"}, \
           {"tokens_checked": nsteps + 1, "identical": bool(ok)}


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


def run_prefill(args):
    """--workload prefill: one 2048-token prompt through Engine.run_tile (16-token tiles: q/k/v, attention
    and o-proj per token, the MoE block per tile on the tcgen05 tile kernels) against the token-serial
    schedule on a 256-token sample of the same prompt.  One step = one prompt token.  The tile path
    is checked against the serial one on the sample (same next token, same hidden state bits)."""
    import numpy as np
    import torch
    import cpubrrr_b200 as B
    from cpubrrr_b200 import synth as S
    torch.cuda.set_device(0)
    eng = B.Engine.synth(B.gptoss_20b_cfg() if args.layers == 24 else B.make_cfg(2880, args.layers, 64, 8, 32, 4, args.vocab), SEED)
    n = 2048
    prompt = [int(t) for t in S.synth_prompt(SEED, n, 199999 if args.vocab > 199999 else args.vocab - 1)]
    sample = 256
    # serial sample (also the checker)
    eng.set_tile_prefill(True)
    eng.run_tile(prompt[:16], 0, False)                       # warm-up of both paths
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
                      "config": {"workload": "gpt-oss-20b prefill, 2048-token prompt, tiles of 16 tokens, wall clock through Engine.run_tile",
                                 "l2": "inputs larger than L2 (every tile streams the dense layers per token and the routed experts per tile)"},
                      "serial": {"tok_s": sample / dt_serial, "sample_tokens": sample}, "tiles_on_sample": {"tok_s": sample / dt_tile_sample, "sample_tokens": sample},
                      "speedup_vs_serial_on_sample": dt_serial / dt_tile_sample,
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
    ap.add_argument("--workload", default="gptoss20b", choices=["gptoss20b", "gptoss120b", "qwen3-30b-a3b", "moe-tile", "prefill"],
                    help="gptoss20b is the benchmark workload; gptoss120b is the expert-parallel configuration; qwen3-30b-a3b measures the reference's second engine")
    ap.add_argument("--parallel", default="replicas", choices=["replicas", "ep"],
                    help="N > 1: independent replicas (weak scaling, default) or one sequence with the experts sharded over the ranks (strong scaling)")
    ap.add_argument("--layers", type=int, default=24, help="profiling aid: fewer layers (not the benchmark workload)")
    ap.add_argument("--vocab", type=int, default=201088, help="profiling aid: smaller vocabulary (not the benchmark workload)")
    args = ap.parse_args()
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
    first = eng.prefill(prompt)
    stream = torch.cuda.ExternalStream(eng.stream, device=torch.device("cuda", local_rank))

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-chained decode: W warm-up steps, then exactly K timed steps
    eng.decode(first, PROMPT_LEN, args.warmup)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    if sampler:
        sampler.start()
    e0.record(stream)
    eng.decode_enqueue(first, PROMPT_LEN, K)
    e1.record(stream)
    toks = eng.decode_wait(K)
    barrier()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # keep the GPUs busy long enough for the clock sampler on short runs; the number of extra calls
    # is derived from the reduced time, so every rank issues the same calls (expert-parallel ranks must)
    extra = int(max(0.0, 1.0 - ms / 1000.0) / (16 * ms / K / 1000.0)) + 1
    for _ in range(extra):
        eng.decode(first, PROMPT_LEN, 16)
    clocks = sampler.stop() if sampler else None

    # ---- end to end through the public API: host token in, host token out, every step
    tok, pos = first, PROMPT_LEN
    for _ in range(args.warmup):
        tok = eng.run(tok, pos, True); pos += 1
    tok, pos = first, PROMPT_LEN
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        tok = eng.run(tok, pos, True); pos += 1
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    if rank != 0:
        if dist is not None:
            dist.barrier()              # nobody frees memory its peers may still write to
        eng.close()
        if dist is not None:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    mid = PROMPT_LEN + K // 2
    step_bytes = sum(eng.bytes_per_step(PROMPT_LEN + i) for i in range(K)) / K
    nseq = 1 if ep_mode else world          # expert-parallel ranks share one sequence
    value = nseq * K / (ms / 1000.0)
    out = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": args.warmup,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong" if ep_mode else "weak", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic",
        "config": {"workload": WORKLOAD if not reduced else f"PROFILING CASE ({args.layers} layers, vocab {args.vocab}) - not the benchmark workload", "arch": ARCH,
                   "positions": [PROMPT_LEN, PROMPT_LEN + K], "parallelism": (f"expert-parallel x{world}" if ep_mode else f"replicas x{world}") if (world > 1 or ep_mode) else "single GPU",
                   "l2": f"inputs larger than L2 ({eng.bytes_per_step(PROMPT_LEN) / 1e9:.2f} GB of weights streamed per step)"},
        "e2e": {"value": nseq * K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4},
        "gpu_launches": K * eng.launches_per_step(True),
        "clocks": clocks,
        "step_roofline": {"bound": "hbm", "bytes_per_step": step_bytes, "achieved": step_bytes / (ms / K) / 1e6, "peak": peak * (world if ep_mode else 1),
                          "unit": "GB/s", "frac": step_bytes / (ms / K) / 1e6 / (peak * (world if ep_mode else 1)), "peak_kind": peak_kind,
                          "frac_of_8TBs": step_bytes / (ms / K) / 1e6 / 8000.0},
    }
    if not args.no_stages:
        st = [r for r in eng.stage_times(mid, reps=10) if r[3] > 0]      # classes the step does not launch report 0 launches
        tot = sum(t * n for _, t, _, n in st)
        stages = [{"kernel": nm, "launches_per_step": n, "us_per_launch": 1000 * t, "share": t * n / tot,
                   "bytes_per_launch": by, "gbs": by / t / 1e6 if t > 0 else 0.0} for nm, t, by, n in st]
        out["stages"] = stages
        # dram__bytes_read+write per launch from the committed ncu captures (profiles/
        # gptoss20b_expert_kernels_tcgen05_ncu_full_small_case.md for gate/up and down,
        # gptoss20b_layer_kernels_ncu_full_small_case.md for the rest); the layer kernels' shapes do
        # not depend on the layer count or vocabulary of the captured case.
        ncu_traffic = {"norm_gate_up_swiglu_mxfp4": 35.42e6, "down_combine_mxfp4": 18.20e6, "norm_qkv_gemv": 16.68e6,
                       "oproj_gemv": 13.32e6, "norm_router_topk": 0.49e6, "attention": 0.06e6}
        # the dominant kernel of the step: the exact router is left out, it runs on a side stream
        # beside gate/up and down and is not on the step's critical path
        top = max((s for s in stages if s["kernel"] != "norm_router_topk" or qwen), key=lambda s: s["share"])
        out["roofline"] = {"bound": "hbm", "kernel": top["kernel"], "achieved": top["gbs"], "peak": peak, "unit": "GB/s",
                           "frac": top["gbs"] / peak, "traffic": ncu_traffic.get(top["kernel"]), "peak_kind": peak_kind,
                           "bytes_per_launch": top["bytes_per_launch"], "us_per_launch": top["us_per_launch"]}
    if world == 1 and not args.no_cpu:
        cpu, parity = cpu_baseline_and_parity(toks, first, 16, qwen)
        out["cpu_baseline"] = cpu
        out["parity"] = parity
    if dist is not None:
        dist.barrier()
    eng.close()
    print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
