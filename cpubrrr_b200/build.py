"""Build the engine's shared library (cpubrrr_b200/libbrrr.so) with nvcc for sm_100a.

    python -m cpubrrr_b200.build [--force] [--verbose] [--hooks]

--hooks also builds libbrrr_hooks.so: the same sources with -DBRRR_TEST_HOOKS, which compiles in what
only tests and timeline measurements use (a way to spoil the routing estimate, a way to silence the
router's publication, in-kernel clock stamps and the entry point that reads them).  The default
library contains none of it.

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
HOOKS_LIB = os.path.join(HERE, "libbrrr_hooks.so")
EXE = os.path.join(HERE, "brrr_engine")
EXE_QWEN = os.path.join(HERE, "brrr_engine_qwen")

SOURCES = ["kernels_small.cu", "kernels_q8.cu", "kernels_mx.cu", "kernels_router.cu", "kernels_attn.cu", "kernels_ep.cu", "kernels_tile.cu", "kernels_rows.cu", "kernels_mxt.cu", "kernels_kq.cu", "kernels_qwen.cu", "qwen_model.cu",
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


def _stale(lib):
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "brrr.h"), __file__]
    return any(os.path.getmtime(p) > t for p in deps)


def build(force=False, verbose=False, defines=(), out=LIB):
    """Compile every CUDA source with the given -D defines and link the shared library `out`
    (default: libbrrr.so, plus the brrr_engine binary); returns its path."""
    if not force and not _stale(out):
        return out
    nvcc = _nvcc()
    tag = "" if out == LIB else "_" + os.path.splitext(os.path.basename(out))[0]
    objdir = OBJ + tag
    os.makedirs(objdir, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []
    extra += [f"-D{d}" for d in defines]

    def compile_one(src):
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    cmd = [nvcc, "-shared", "-o", out, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-ccbin", "g++"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if out == LIB:
        # the command-line front ends (the reference binaries' arguments and protocols), linked against the library
        for exe, main_src in ((EXE, "engine_main.cpp"), (EXE_QWEN, "engine_qwen_main.cpp")):
            cmd = ["g++", "-O2", "-o", exe, os.path.join(CSRC, main_src), "-L" + HERE, "-lbrrr", "-Wl,-rpath,$ORIGIN"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"link of {os.path.basename(exe)} failed:\n{r.stdout}\n{r.stderr}")
    return out


def build_hooks(force=False):
    """The test-hook build of the library (libbrrr_hooks.so, -DBRRR_TEST_HOOKS)."""
    return build(force=force, defines=("BRRR_TEST_HOOKS",), out=HOOKS_LIB)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--hooks" in sys.argv:
        print(build_hooks(force="--force" in sys.argv))
