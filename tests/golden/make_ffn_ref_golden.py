"""Generates tests/golden/ffn_ref/*.npy by RUNNING THE REFERENCE'S OWN PYTHON CODE:
scripts/ffn_reference.py of the reference (a float64 numpy statement of the gpt-oss layer-0 MoE FFN:
router + top-4 softmax, SwiGLU-OAI, biases, weighted combine) on a seeded synthetic one-layer model
of the gpt-oss-20b layer shape, written as a GGUF blob by cpubrrr_b200.synth and indexed by the reference's scripts/gguf_index.py.

    python tests/golden/make_ffn_ref_golden.py      # needs the reference checkout, ~1 GB of /tmp

That script scales MXFP4 blocks by 2^(e-127) on the doubled code table, twice the value the engine
(and ggml) gives them; the reference's own log records the offset (docs/RESEARCH_LOG.md:470, "correct is
2^(e-128)").  To make the script evaluate the model the engine sees, the copy of the blob it reads has
every exponent byte of the three expert tensors lowered by one.

Fixture: the script's input x (it draws it itself), its output, its top-4 experts and weights.
The model is not stored: the tests regenerate it from the seed."""
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import cpubrrr_b200 as B  # noqa: E402
from cpubrrr_b200 import synth as S  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import refdata  # noqa: E402
REF = os.path.join(refdata.REF, "scripts", "ffn_reference.py")
SEED = 77


def lower_expert_exponents(blob, idx_path):
    import json
    idx = json.load(open(idx_path))
    tn = {t["name"]: t for t in idx["tensors"]}
    nbytes = 32 * 2880 * (2880 // 32) * 17
    with open(blob, "r+b") as f:
        for name in ("blk.0.ffn_gate_exps.weight", "blk.0.ffn_up_exps.weight", "blk.0.ffn_down_exps.weight"):
            off = idx["data_start"] + tn[name]["offset"]
            f.seek(off)
            a = np.frombuffer(f.read(nbytes), np.uint8).reshape(-1, 17).copy()
            assert a[:, 0].min() >= 1
            a[:, 0] -= 1
            f.seek(off)
            f.write(a.tobytes())


def main():
    if not os.path.exists(REF):
        raise SystemExit("reference checkout not present")
    out = os.path.join(HERE, "ffn_ref")
    os.makedirs(out, exist_ok=True)
    cfg = B.make_cfg(2880, 1, 64, 8, 32, 4, 256)
    with tempfile.TemporaryDirectory() as tmp:
        d = os.path.join(tmp, "m")
        os.makedirs(d)
        blob = os.path.join(d, "model.gguf")
        S.write_gguf(blob, cfg, SEED)
        refdata.run_reference_setup(blob, d)        # index.json by the reference's own gguf_index.py
        lower_expert_exponents(blob, os.path.join(d, "index.json"))
        res = os.path.join(tmp, "out")
        os.makedirs(res)
        r = subprocess.run([sys.executable, REF, blob, os.path.join(d, "index.json"), res], capture_output=True, text=True)
        print(r.stdout[-600:], r.stderr[-600:])
        r.check_returncode()
        np.save(os.path.join(out, "x.npy"), np.fromfile(os.path.join(res, "ffn_x.f32"), np.float32))
        np.save(os.path.join(out, "yref.npy"), np.fromfile(os.path.join(res, "ffn_yref.f32"), np.float32))
        np.save(os.path.join(out, "top.npy"), np.fromfile(os.path.join(res, "ffn_top.i32"), np.int32))
        np.save(os.path.join(out, "w.npy"), np.fromfile(os.path.join(res, "ffn_w.f32"), np.float32))
    print("wrote", out)


if __name__ == "__main__":
    main()
