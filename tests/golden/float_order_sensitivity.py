"""TEST INFRASTRUCTURE - how much does the fixed float order matter for the parity bar?

Builds the CPU oracle twice from the sources under oracle/: with its own flags (every sum in the reference's
order, fused multiply-adds only where written) and with `-fassociative-math -ffp-contract=fast` (the compiler may re-associate sums into
vector lanes and contract multiply-adds: a stand-in for kernels that keep the integer block dots exact but do
not keep the float order).  Both run the gpt-oss-20b workload of bench.py (seeded synthetic weights, 73-token
prompt, 128 greedy steps from position 73) on the CPU.  The relaxed build is teacher-forced with the strict
build's tokens, so every step compares logits of the same input; reported per run:

  * steps where the relaxed build's argmax differs from the strict token (and the first such step:
    a free-running relaxed decoder would leave the strict sequence there),
  * relative L2 distance of the logits per step (max, median),
  * the strict build's smallest top-1 / top-2 logit gap.

Each variant runs in its own process.  Usage: python tests/golden/float_order_sensitivity.py [--layers 24] [--steps 128] [--seed 1234]
Needs about 30 GB of host memory and ten minutes on 8 cores at full size; not part of the test run.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
ORC = os.path.join(ROOT, "oracle")
SRC = ["oracle_kernels.c", "oracle_gptoss.c", "oracle_qwen.c", "oracle_qwen_model.c"]
FLAGS = {
    "strict": ["-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fno-fast-math"],
    # re-association and contraction only: no reciprocal approximations, no finite-math assumptions, libm untouched
    "relaxed": ["-O3", "-march=x86-64-v3", "-ffp-contract=fast", "-fassociative-math", "-fno-signed-zeros", "-fno-trapping-math"],
}


class Cfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("d", "nh", "nkv", "hd", "nl", "ne", "topk", "nvocab", "swa")] + [
        ("rope_base", C.c_float), ("rms_eps", C.c_float)]


def build(variant, out_dir):
    so = os.path.join(out_dir, f"liboracle_{variant}.so")
    cmd = ["gcc"] + FLAGS[variant] + ["-fopenmp", "-fPIC", "-std=gnu11", "-shared", "-o", so] + [os.path.join(ORC, s) for s in SRC] + ["-lm"]
    subprocess.run(cmd, check=True, cwd=ORC)
    return so


def worker(so, layers, steps, seed, prompt_len, force_path, out_path):
    L = C.CDLL(so)
    L.orc_open_synth.restype = C.c_void_p
    L.orc_open_synth.argtypes = [C.POINTER(Cfg), C.c_uint64]
    L.orc_forward.restype = C.c_uint32
    L.orc_forward.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_int]
    L.orc_logits.restype = C.POINTER(C.c_float)
    L.orc_logits.argtypes = [C.c_void_p]
    L.orc_synth_prompt.argtypes = [C.c_uint64, C.c_int, C.c_uint32, C.c_void_p]
    L.orc_close.argtypes = [C.c_void_p]
    cfg = Cfg(2880, 64, 8, 64, layers, 32, 4, 201088, 128, 150000.0, 1e-5)
    m = L.orc_open_synth(C.byref(cfg), seed)
    assert m
    prompt = np.zeros(prompt_len, np.uint32)
    L.orc_synth_prompt(seed, prompt_len, 199999, prompt.ctypes.data)
    forced = np.load(force_path) if force_path else None
    tok = 0
    for i, t in enumerate(prompt):
        tok = L.orc_forward(m, int(t), i, int(i == prompt_len - 1))
    toks, logits, gaps = [], [], []
    pos = prompt_len
    for k in range(steps + 1):                      # the prompt's last step counts as step 0
        lg = np.ctypeslib.as_array(L.orc_logits(m), shape=(cfg.nvocab,)).copy()
        toks.append(int(np.argmax(lg)))
        top2 = np.partition(lg, -2)[-2:]
        gaps.append(float(top2[1] - top2[0]))
        logits.append(lg)
        if k == steps:
            break
        feed = int(forced[k]) if forced is not None else toks[-1]
        L.orc_forward(m, feed, pos, 1)
        pos += 1
    np.save(out_path + ".toks.npy", np.array(toks, np.uint32))
    np.save(out_path + ".logits.npy", np.stack(logits))
    json.dump({"gaps": gaps}, open(out_path + ".json", "w"))
    L.orc_close(m)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--prompt", type=int, default=73)
    ap.add_argument("--worker", nargs=4, help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.worker:
        so, force, out, _ = args.worker
        worker(so, args.layers, args.steps, args.seed, args.prompt, force if force != "-" else None, out)
        return
    with tempfile.TemporaryDirectory() as td:
        res = {}
        for variant in ("strict", "relaxed"):
            so = build(variant, td)
            out = os.path.join(td, variant)
            force = os.path.join(td, "strict.toks.npy") if variant == "relaxed" else "-"
            subprocess.run([sys.executable, os.path.abspath(__file__), "--layers", str(args.layers), "--steps", str(args.steps), "--seed", str(args.seed),
                            "--prompt", str(args.prompt), "--worker", so, force, out, "x"], check=True)
            res[variant] = (np.load(out + ".toks.npy"), np.load(out + ".logits.npy"), json.load(open(out + ".json"))["gaps"])
        ts, ls, gs = res["strict"]
        tr, lr, _ = res["relaxed"]
        rel = np.linalg.norm((lr - ls).astype(np.float64), axis=1) / np.linalg.norm(ls.astype(np.float64), axis=1)
        diff = np.nonzero(tr != ts)[0]
        print(json.dumps({
            "workload": f"gpt-oss-20b shape, {args.layers} layers, {args.prompt}-token prompt, {args.steps} steps, seed {args.seed}",
            "steps_compared": int(len(ts)),
            "argmax_differs_at_steps": [int(i) for i in diff],
            "first_divergence": int(diff[0]) if len(diff) else None,
            "logits_rel_l2_max": float(rel.max()), "logits_rel_l2_median": float(np.median(rel)),
            "strict_min_top1_top2_gap": float(min(gs)),
            "logit_abs_diff_max": float(np.abs(lr - ls).max()),
        }))


if __name__ == "__main__":
    main()
