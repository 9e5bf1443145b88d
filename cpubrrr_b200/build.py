"""Build the engine's shared library (cpubrrr_b200/libbrrr.so) with nvcc for sm_100a.

    python -m cpubrrr_b200.build [--force] [--verbose]

The library is built in-tree so that it travels with the source tree.  nvcc cross-compiles
without a GPU.  -fmad=false: kernels fuse multiply-adds only where written explicitly, which
the bit-reproducible float order of the engine depends on.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libbrrr.so")
EXE = os.path.join(HERE, "brrr_engine")

SOURCES = ["kernels_small.cu", "kernels_q8.cu", "kernels_mx.cu", "kernels_router.cu", "kernels_attn.cu", "kernels_ep.cu", "kernels_tile.cu", "kernels_mxt.cu", "kernels_kq.cu", "kernels_qwen.cu", "qwen_model.cu",
           "model.cu", "capi_stage.cu", "capi_noalloc.cu", "host_text.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC,-ffp-contract=off,-O2", "-ccbin", "g++",
]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "brrr.h"), __file__]
    return any(os.path.getmtime(p) > t for p in deps)


def build(force=False, verbose=False):
    """Compile every CUDA source and link libbrrr.so; returns its path."""
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []
    extra += [f"-D{d}" for d in os.environ.get("BRRR_DEFS", "").split()]
    if os.environ.get("BRRR_TIMELINE"):
        extra.append("-DBRRR_TIMELINE")
        if os.environ.get("BRRR_TIMELINE_CTA"):
            extra.append("-DBRRR_TIMELINE_CTA=" + os.environ["BRRR_TIMELINE_CTA"])

    def compile_one(src):
        obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-ccbin", "g++"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    # the command-line front end (reference binary's arguments and protocol), linked against the library
    cmd = ["g++", "-O2", "-o", EXE, os.path.join(CSRC, "engine_main.cpp"), "-L" + HERE, "-lbrrr", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link of brrr_engine failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
