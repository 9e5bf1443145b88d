"""TEST INFRASTRUCTURE - data directories for the file-loading tests, made by the reference's own
preparation scripts.

A data directory is what scripts/setup_model.sh of the reference leaves beside a GGUF blob:
config.txt, manifest.txt, tokens.bin (plus index.json).  When a checkout of the reference is
present (environment variable BRRR_REFERENCE_DIR, else the default location below) `make_data_dir` runs, unmodified,
  * scripts/gguf_index.py <blob>            -> index.json
  * scripts/dump_tokenizer.py <blob> <dir>  -> tokens.bin
  * the inline generator of scripts/setup_model.sh (the `python3 -c "..."` command after
    "writing manifest + config...", handed to bash as it stands with OUT set) -> manifest.txt, config.txt
on a blob written by cpubrrr_b200.synth.write_gguf, and checks the result against the committed
copy under tests/golden/datadir/<case>/ (made the same way by tests/golden/make_datadir_golden.py).
Without the checkout (the GPU box) the committed copy is used: config.txt and manifest.txt as
files, tokens.bin rewritten from the toy vocabulary's raw bytes and checked against the SHA-256 the
reference's script produced.
"""
import hashlib
import os
import re
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from cpubrrr_b200 import synth as S  # noqa: E402

REF = os.environ.get("BRRR_REFERENCE_DIR", "/root/reference")
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "datadir")


def have_reference():
    return os.path.exists(os.path.join(REF, "scripts", "setup_model.sh"))


def _inline_generator():
    """The manifest/config command of setup_model.sh, verbatim."""
    text = open(os.path.join(REF, "scripts", "setup_model.sh")).read()
    m = re.search(r'echo "writing manifest \+ config\.\.\."\n(python3 -c ".*?\n")\n', text, re.S)
    assert m, "setup_model.sh: manifest/config generator not found"
    return m.group(1)


def run_reference_setup(blob, out_dir):
    """The three steps of setup_model.sh after it has located the blob."""
    os.makedirs(out_dir, exist_ok=True)
    scripts = os.path.join(REF, "scripts")
    with open(os.path.join(out_dir, "index.json"), "w") as w:
        subprocess.run([sys.executable, os.path.join(scripts, "gguf_index.py"), blob], stdout=w, check=True)
    subprocess.run([sys.executable, os.path.join(scripts, "dump_tokenizer.py"), blob, out_dir], check=True, capture_output=True)
    env = dict(os.environ, OUT=out_dir)
    # the command says python3; make that this interpreter
    bindir = os.path.dirname(sys.executable)
    env["PATH"] = bindir + os.pathsep + env.get("PATH", "")
    subprocess.run(["bash", "-c", _inline_generator()], env=env, check=True, capture_output=True)
    with open(os.path.join(out_dir, "blob_path.txt"), "w") as w:
        w.write(blob + "\n")


def _sha(path):
    return hashlib.sha256(open(path, "rb").read()).hexdigest()


def make_data_dir(out_dir, cfg, seed, case, arch="gpt-oss", ktypes=None):
    """Write a synthetic model as GGUF into out_dir and the data directory around it; returns
    (data_dir, blob_path).  `case` names the committed copy (it depends on the shapes, the tensor
    types and the vocabulary only, not on the seed)."""
    os.makedirs(out_dir, exist_ok=True)
    blob = os.path.join(out_dir, "model.gguf")
    S.write_gguf(blob, cfg, seed, arch=arch, ktypes=ktypes)
    gold = os.path.join(GOLD, case)
    if have_reference():
        run_reference_setup(blob, out_dir)
        if os.path.isdir(gold):
            for f in ("config.txt", "manifest.txt"):
                assert open(os.path.join(out_dir, f)).read() == open(os.path.join(gold, f)).read(), f"{case}/{f} differs from the committed copy"
            assert _sha(os.path.join(out_dir, "tokens.bin")) == open(os.path.join(gold, "tokens.sha256")).read().strip()
    else:
        assert os.path.isdir(gold), f"no reference checkout and no committed data directory for case {case}"
        for f in ("config.txt", "manifest.txt"):
            shutil.copy(os.path.join(gold, f), os.path.join(out_dir, f))
        S.write_tokens_bin(os.path.join(out_dir, "tokens.bin"), S.raw_tokens(cfg.n_vocab, arch))
        assert _sha(os.path.join(out_dir, "tokens.bin")) == open(os.path.join(gold, "tokens.sha256")).read().strip()
    # the manifest must describe the blob that was just written
    rows = open(os.path.join(out_dir, "manifest.txt")).read().split("\n")
    data_start = int(rows[0].split()[1])
    name, ty, off, nel = rows[-2].split() if rows[-1] == "" else rows[-1].split()
    per = {0: (1, 4), 30: (1, 2), 39: (32, 17), 12: (256, 144), 14: (256, 210)}[int(ty)]
    end = data_start + int(off) + int(nel) // per[0] * per[1]
    assert (end + 31) // 32 * 32 == os.path.getsize(blob), "manifest does not match the blob"
    return out_dir, blob


# the cases the tests use: name -> (arch, cfg constructor arguments, K-quant type overrides)
CASES = {
    "gptoss_d128": ("gpt-oss", dict(n_embd=128, n_layer=2, n_head=4, n_head_kv=2, n_expert=8, n_expert_used=4, n_vocab=512), None),
    "gptoss_serve": ("gpt-oss", dict(n_embd=64, n_layer=1, n_head=2, n_head_kv=1, n_expert=4, n_expert_used=2, n_vocab=200064, sliding_window=16), None),
    "qwen_gold": ("qwen3moe", None, None),          # shape taken from tests/golden/qwen_tiny_tokens.json
    "qwen_d256": ("qwen3moe", dict(n_embd=256, n_layer=2, n_head=4, n_head_kv=2, n_expert=8, n_expert_used=4, n_ff_exp=256, n_vocab=600), None),
    # per-tensor K-quant types as real files mix them: attn_v of layer 0 as Q6_K, the down experts of layer 1 as Q4_K
    "qwen_mixed": ("qwen3moe", dict(n_embd=256, n_layer=2, n_head=4, n_head_kv=2, n_expert=8, n_expert_used=4, n_ff_exp=256, n_vocab=600),
                   {"blk.0.attn_v.weight": 14, "blk.1.ffn_down_exps.weight": 12}),
}


def case_cfg(case):
    import json
    import cpubrrr_b200 as B
    arch, kw, ktypes = CASES[case]
    if case == "qwen_gold":
        c = json.load(open(os.path.join(os.path.dirname(GOLD), "qwen_tiny_tokens.json")))["cfg"]
        return arch, B.make_qwen_cfg(c["d"], c["nl"], c["nh"], c["nkv"], c["ne"], c["topk"], c["ff"], c["nvocab"]), ktypes
    if arch == "qwen3moe":
        return arch, B.make_qwen_cfg(kw["n_embd"], kw["n_layer"], kw["n_head"], kw["n_head_kv"], kw["n_expert"], kw["n_expert_used"], kw["n_ff_exp"], kw["n_vocab"]), ktypes
    return arch, B.make_cfg(**kw), ktypes


def case_data_dir(out_dir, case, seed):
    arch, cfg, ktypes = case_cfg(case)
    d, blob = make_data_dir(out_dir, cfg, seed, case, arch=arch, ktypes=ktypes)
    return cfg, d, blob
