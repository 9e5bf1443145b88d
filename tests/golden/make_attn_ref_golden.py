"""Generates tests/golden/attn_ref/*.npy by RUNNING THE REFERENCE'S OWN PYTHON CODE:
scripts/attn_reference.py of the reference (a float64 numpy statement of the gpt-oss layer-0 attention
block for one decode step over an 8-entry cache: RMS norm, q/k/v projections with bias, plain NeoX
RoPE at base 150000, the GQA head map, learned sinks in the softmax denominator, o-proj with bias) on
a seeded synthetic one-layer model of the gpt-oss-20b layer shape, written as a GGUF blob by
cpubrrr_b200.synth and indexed by the reference's scripts/gguf_index.py.

    python tests/golden/make_attn_ref_golden.py      # needs the reference checkout

The script applies plain RoPE (no YaRN ramp, no mscale; its header says so), so the tests hand the
engine's attention stage a plain cos/sin table; the YaRN table is checked separately.

Fixture: the script's input h and caches (it draws them itself) and its output.  The model is not
stored: the tests regenerate it from the seed."""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import refdata  # noqa: E402
import cpubrrr_b200 as B  # noqa: E402
from cpubrrr_b200 import synth as S  # noqa: E402

REF = os.path.join(refdata.REF, "scripts", "attn_reference.py")
SEED = 78


def main():
    if not os.path.exists(REF):
        raise SystemExit("reference checkout not present")
    out = os.path.join(HERE, "attn_ref")
    os.makedirs(out, exist_ok=True)
    cfg = B.make_cfg(2880, 1, 64, 8, 4, 4, 256)          # the script reads the attention tensors only: 4 experts keep the blob small
    with tempfile.TemporaryDirectory() as tmp:
        d = os.path.join(tmp, "m")
        os.makedirs(d)
        blob = os.path.join(d, "model.gguf")
        S.write_gguf(blob, cfg, SEED)
        refdata.run_reference_setup(blob, d)
        res = os.path.join(tmp, "out")
        os.makedirs(res)
        r = subprocess.run([sys.executable, REF, blob, os.path.join(d, "index.json"), res], capture_output=True, text=True)
        print(r.stdout[-600:], r.stderr[-600:])
        r.check_returncode()
        for name in ("h", "kcache", "vcache", "attn_yref"):
            np.save(os.path.join(out, name + ".npy"), np.fromfile(os.path.join(res, f"aw_{name}.f32"), np.float32))
    print("wrote", out)


if __name__ == "__main__":
    main()
