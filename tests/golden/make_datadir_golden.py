"""Generates tests/golden/datadir/<case>/{config.txt, manifest.txt, tokens.sha256} by RUNNING THE
REFERENCE'S OWN PREPARATION SCRIPTS (scripts/gguf_index.py, scripts/dump_tokenizer.py and the inline
manifest/config generator of scripts/setup_model.sh, all unmodified) on GGUF blobs of seeded
synthetic models written by cpubrrr_b200.synth.write_gguf.

    python tests/golden/make_datadir_golden.py        # needs the reference checkout

The committed copies let the file-loading tests run where the checkout is absent; where it is
present the tests run the scripts again and compare with these files (tests/refdata.py).
tokens.bin itself is not stored (1.6 MB for the serve case): its SHA-256 is, and the tests rebuild
the file from the toy vocabulary's raw bytes."""
import os
import shutil
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import refdata as R  # noqa: E402


def main():
    if not R.have_reference():
        raise SystemExit("reference checkout not present")
    for case in R.CASES:
        arch, cfg, ktypes = R.case_cfg(case)
        out = os.path.join(R.GOLD, case)
        if os.path.isdir(out):
            shutil.rmtree(out)
        with tempfile.TemporaryDirectory() as tmp:
            blob = os.path.join(tmp, "model.gguf")
            R.S.write_gguf(blob, cfg, 1, arch=arch, ktypes=ktypes)
            R.run_reference_setup(blob, tmp)
            os.makedirs(out)
            for f in ("config.txt", "manifest.txt"):
                shutil.copy(os.path.join(tmp, f), os.path.join(out, f))
            with open(os.path.join(out, "tokens.sha256"), "w") as w:
                w.write(R._sha(os.path.join(tmp, "tokens.bin")) + "\n")
        print("wrote", out)


if __name__ == "__main__":
    main()
