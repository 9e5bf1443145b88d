"""The C-ABI library loads on a CPU-only machine and exports every symbol include/brrr.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    src = open(os.path.join(ROOT, "include", "brrr.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(brrr_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_exported(brrr):
    names = declared_symbols()
    assert len(names) >= 30
    L = ctypes.CDLL(brrr.LIB_PATH)
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_binding_covers_header(brrr):
    from cpubrrr_b200._lib import SIGNATURES
    assert sorted(SIGNATURES) == declared_symbols()


def test_error_strings_and_argument_checks(brrr):
    L = brrr.lib()
    assert L.brrr_strerror(0) == b"ok"
    assert b"argument" in L.brrr_strerror(1)
    # argument validation happens before any CUDA call, so it is testable without a GPU
    assert L.brrr_quant_q8(None, 64, None, None, None) == 1
    assert L.brrr_quant_q8(ctypes.c_void_p(16), 33, ctypes.c_void_p(16), ctypes.c_void_p(16), None) == 1
    h = ctypes.c_void_p()
    bad = brrr.make_cfg(100, 1, 4, 2, 8, 4, 512)          # n_embd not a multiple of 64
    assert L.brrr_model_open_synth(ctypes.byref(bad), 1, 0, ctypes.byref(h)) == 1
    bad = brrr.make_cfg(128, 1, 4, 2, 8, 4, 512, head_dim=128)  # reference asserts head_dim == 64
    assert L.brrr_model_open_synth(ctypes.byref(bad), 1, 0, ctypes.byref(h)) == 1
    bad = brrr.make_cfg(128, 1, 4, 2, 8, 9, 512)           # top-k > 8
    assert L.brrr_model_open_synth(ctypes.byref(bad), 1, 0, ctypes.byref(h)) == 1


def test_missing_data_dir_is_an_io_error(brrr, tmp_path):
    L = brrr.lib()
    h = ctypes.c_void_p()
    assert L.brrr_model_open(str(tmp_path).encode(), b"/nonexistent", 0, ctypes.byref(h)) == 2
    assert b"config.txt" in L.brrr_last_cuda_error()


def test_no_cpu_fallback_when_library_missing(monkeypatch, brrr):
    import cpubrrr_b200._lib as _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libbrrr.so")
    import pytest
    with pytest.raises(_lib.BrrrError):
        _lib.lib()


def test_limits_agree_between_header_and_device_code(brrr):
    """BRRR_MAXSEQ and BRRR_TILE_MAX are defined for hosts (include/brrr.h) and for the kernels (csrc/brrr_dev.cuh):
    the two must carry the same values, and the argument checks that need no GPU must follow them."""
    pub = open(os.path.join(ROOT, "include", "brrr.h")).read()
    dev = open(os.path.join(ROOT, "cpubrrr_b200", "csrc", "brrr_dev.cuh")).read()
    for name in ("BRRR_MAXSEQ", "BRRR_TILE_MAX"):
        a = re.search(r"#define\s+%s\s+(\d+)" % name, pub).group(1)
        b = re.search(r"#define\s+%s\s+(\d+)" % name, dev).group(1)
        assert a == b, (name, a, b)
    tile_max = int(re.search(r"#define\s+BRRR_TILE_MAX\s+(\d+)", pub).group(1))
    batch_max = int(re.search(r"#define\s+BRRR_BATCH_MAX\s+(\d+)", pub).group(1))
    L = brrr.lib()
    p = ctypes.c_void_p(16)
    # no model handle: argument errors come before anything touches the device
    assert L.brrr_batch_open(None, 1) == 1
    assert L.brrr_batch_step(None, 1, p, p, p, p) == 1
    assert L.brrr_q8_matmul_rows(None, p, p, 1, p, 16, 0, None) == 1
    assert L.brrr_mx_matmul_tile(None, 0, 16, p, p, tile_max + 1, p, 16, None) == 1
    assert batch_max <= tile_max
