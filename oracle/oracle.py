"""TEST INFRASTRUCTURE — ctypes binding of the CPU oracle (oracle/_build/liboracle.so).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module; the
shipped package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")


def build(force=False):
    """Compile the oracle with the Makefile beside this file (no-op when up to date)."""
    if force and os.path.exists(_SO):
        os.remove(_SO)
    subprocess.run(["make", "-s", "-C", _HERE], check=True)
    return _SO


_REF_SO = os.path.join(_HERE, "_ref", "libref_kq.so")
_REF_DIR = os.environ.get("BRRR_REFERENCE_DIR", "/root/reference")
_REF_SRC = os.path.join(_REF_DIR, "metal", "engine_metal.m")


def build_ref():
    """Build oracle/_ref/libref_kq.so (the reference's own scalar C Q4_K/Q6_K dots) when the reference
    checkout is present; returns the path, or None when neither the checkout nor a prebuilt file exists."""
    if os.path.exists(_REF_SRC):
        subprocess.run(["make", "-s", "-C", _HERE, "ref", "REF=" + _REF_DIR], check=True)
    return _REF_SO if os.path.exists(_REF_SO) else None


_ref = None


def ref_kq():
    """ctypes handle of the reference-built dots, or None when unavailable."""
    global _ref
    if _ref is None:
        so = build_ref()
        if so is None:
            return None
        L = C.CDLL(so)
        L.refkq_q4k_dot.restype = C.c_float
        L.refkq_q6k_dot.restype = C.c_float
        L.refkq_half2f.restype = C.c_float
        L.refkq_half2f.argtypes = [C.c_uint16]
        _ref = L
    return _ref


class Cfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("d", "nh", "nkv", "hd", "nl", "ne", "topk", "nvocab", "swa")] + [
        ("rope_base", C.c_float), ("rms_eps", C.c_float)]


class Q8Mat(C.Structure):
    _fields_ = [("q", C.c_void_p), ("s", C.c_void_p), ("rows", C.c_int), ("cols", C.c_int)]


class QuadMx(C.Structure):
    _fields_ = [("nib", C.c_void_p), ("exps", C.c_void_p), ("rows", C.c_int), ("blocks", C.c_int)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        L.orc_expf_c.restype = C.c_float
        L.orc_expf_c.argtypes = [C.c_float]
        L.orc_ssq.restype = C.c_float
        L.orc_dot_q8_i8.restype = C.c_float
        L.orc_half_to_f32.restype = C.c_float
        L.orc_half_to_f32.argtypes = [C.c_uint16]
        L.orc_q4k_dot.restype = C.c_float
        L.orc_q6k_dot.restype = C.c_float
        L.orc_open_dir.restype = C.c_void_p
        L.orc_open_dir.argtypes = [C.c_char_p, C.c_char_p]
        L.orc_open_synth.restype = C.c_void_p
        L.orc_open_synth.argtypes = [C.POINTER(Cfg), C.c_uint64]
        L.orc_close.argtypes = [C.c_void_p]
        L.orc_get_cfg.argtypes = [C.c_void_p, C.POINTER(Cfg)]
        L.orc_forward.restype = C.c_uint32
        L.orc_forward.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_int]
        L.orc_logits.restype = C.POINTER(C.c_float)
        L.orc_logits.argtypes = [C.c_void_p]
        L.orc_hidden.restype = C.POINTER(C.c_float)
        L.orc_hidden.argtypes = [C.c_void_p]
        L.orc_set_trace.argtypes = [C.c_void_p, C.c_void_p]
        L.orc_layer_q8.restype = C.POINTER(Q8Mat)
        L.orc_layer_q8.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.orc_layer_mx.restype = C.POINTER(QuadMx)
        L.orc_layer_mx.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.orc_layer_f32.restype = C.POINTER(C.c_float)
        L.orc_layer_f32.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.orc_synth_prompt.argtypes = [C.c_uint64, C.c_int, C.c_uint32, C.c_void_p]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


def expf(x):
    x = np.asarray(x, dtype=np.float32)
    L = lib()
    return np.array([L.orc_expf_c(float(v)) for v in x.ravel()], dtype=np.float32).reshape(x.shape)


def quant_q8(x):
    x = _c(x, np.float32)
    q = np.empty(x.size, np.int8)
    s = np.empty(x.size // 32, np.float32)
    lib().orc_quant_q8(_p(x), C.c_int(x.size), _p(q), _p(s))
    return q, s


def ssq(x):
    x = _c(x, np.float32)
    return np.float32(lib().orc_ssq(_p(x), C.c_int(x.size)))


def rmsnorm(x, w, eps):
    x = _c(x, np.float32); w = _c(w, np.float32)
    out = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), C.c_float(eps), C.c_int(x.size), _p(out))
    return out


def q8_from_bf16(w_bits, rows, cols):
    w = _c(w_bits, np.uint16)
    q = np.empty((rows, cols), np.int8)
    s = np.empty((rows, cols // 32), np.float32)
    lib().orc_q8_from_bf16(_p(w), C.c_int(rows), C.c_int(cols), _p(q), _p(s))
    return q, s


def q8_matvec(q, s, xq, xsb):
    rows, cols = q.shape
    q = _c(q, np.int8); s = _c(s, np.float32); xq = _c(xq, np.int8); xsb = _c(xsb, np.float32)
    y = np.empty(rows, np.float32)
    lib().orc_q8_matvec(_p(q), _p(s), C.c_int(rows), C.c_int(cols), _p(xq), _p(xsb), _p(y))
    return y


def repack_mx(raw, rows, blocks):
    raw = _c(raw, np.uint8)
    assert raw.size == rows * blocks * 17
    nib = np.empty(rows * blocks * 16, np.uint8)
    exps = np.empty(rows * blocks, np.uint8)
    lib().orc_repack_mx(_p(raw), C.c_int(rows), C.c_int(blocks), _p(nib), _p(exps))
    return nib, exps


def mx_matvec(nib, exps, rows, blocks, xq, xsb, want_dbg=False):
    xq = _c(xq, np.int8); xsb = _c(xsb, np.float32)
    y = np.empty(rows, np.float32)
    dbg = np.empty((rows // 4, blocks, 4, 4), np.int32) if want_dbg else None
    lib().orc_mx_matvec(_p(nib), _p(exps), C.c_int(rows), C.c_int(blocks), _p(xq), _p(xsb), _p(y), _p(dbg))
    return (y, dbg) if want_dbg else y


def mx_dequant_rows(raw, rows, blocks):
    raw = _c(raw, np.uint8).reshape(rows, blocks * 17)
    out = np.empty((rows, blocks * 32), np.float32)
    for r in range(rows):
        lib().orc_mx_dequant_row(_p(raw[r]), C.c_int(blocks), _p(out[r]))
    return out


def rope_table(cfg):
    tab = np.empty((4096, cfg.hd // 2, 2), np.float32)
    lib().orc_rope_table(C.byref(cfg), _p(tab))
    return tab


def router_topk(w, b, xn, topk):
    ne, d = w.shape
    w = _c(w, np.float32); xn = _c(xn, np.float32)
    b = _c(b, np.float32) if b is not None else None
    logits = np.empty(ne, np.float32); top = np.empty(topk, np.int32); wts = np.empty(topk, np.float32)
    lib().orc_router_topk(_p(w), _p(b), _p(xn), C.c_int(ne), C.c_int(d), C.c_int(topk), _p(logits), _p(top), _p(wts))
    return logits, top, wts


def swiglu_quant(gu, topk, d):
    gu = _c(gu, np.float32)
    hq = np.empty((topk, d), np.int8); hsb = np.empty((topk, d // 32), np.float32); h = np.empty((topk, d), np.float32)
    lib().orc_swiglu_quant(_p(gu), C.c_int(topk), C.c_int(d), _p(hq), _p(hsb), _p(h))
    return hq, hsb, h


def attn_head(q, kc, vc, nkv, hd, kvh, start, pos, sink):
    q = _c(q, np.float32); kc = _c(kc, np.float32); vc = _c(vc, np.float32)
    sc = np.empty(pos - start + 1, np.float32); ao = np.empty(hd, np.float32)
    lib().orc_attn_head(_p(q), _p(kc), _p(vc), C.c_int(nkv), C.c_int(hd), C.c_int(kvh), C.c_int(start), C.c_int(pos),
                        C.c_float(sink), _p(sc), _p(ao))
    return ao


def half_to_f32(h):
    return np.float32(lib().orc_half_to_f32(int(h)))


def quant_q8k(x):
    """Q8_K activation quantiser: int8 quants, one f32 scale per 256, int32 sums per 32."""
    x = _c(x, np.float32)
    q = np.empty(x.size, np.int8); s = np.empty(x.size // 256, np.float32); bs = np.empty(x.size // 32, np.int32)
    lib().orc_quant_q8k(_p(x), C.c_int(x.size), _p(q), _p(s), _p(bs))
    return q, s, bs


def q4k_matvec(w, rows, cols, xq, ys, bsum, want_dbg=False):
    w = _c(w, np.uint8); xq = _c(xq, np.int8); ys = _c(ys, np.float32); bsum = _c(bsum, np.int32)
    assert w.size == rows * (cols // 256) * 144
    y = np.empty(rows, np.float32)
    dbg = np.empty((rows, cols // 256, 2), np.int32) if want_dbg else None
    lib().orc_q4k_matvec(_p(w), C.c_int(rows), C.c_int(cols), _p(xq), _p(ys), _p(bsum), _p(y), _p(dbg))
    return (y, dbg) if want_dbg else y


def q6k_matvec(w, rows, cols, xq, ys, want_dbg=False):
    w = _c(w, np.uint8); xq = _c(xq, np.int8); ys = _c(ys, np.float32)
    assert w.size == rows * (cols // 256) * 210
    y = np.empty(rows, np.float32)
    dbg = np.empty((rows, cols // 256), np.int32) if want_dbg else None
    lib().orc_q6k_matvec(_p(w), C.c_int(rows), C.c_int(cols), _p(xq), _p(ys), _p(y), _p(dbg))
    return (y, dbg) if want_dbg else y


def set_threads(n):
    """OpenMP worker threads of the oracle's parallel loops; returns the count in effect."""
    lib().orc_set_threads(C.c_int(int(n)))
    return int(lib().orc_max_threads())


def synth_prompt(seed, n, bound):
    out = np.empty(n, np.uint32)
    lib().orc_synth_prompt(C.c_uint64(seed), C.c_int(n), C.c_uint32(bound), _p(out))
    return out


def make_cfg(d, nh, nkv, hd, nl, ne, topk, nvocab, swa=128, rope_base=150000.0, rms_eps=1e-5):
    return Cfg(d, nh, nkv, hd, nl, ne, topk, nvocab, swa, rope_base, rms_eps)


class Model:
    """The oracle's model: run(tok, pos, want) -> greedy token, as engine_gpt2.rs:1379."""

    def __init__(self, handle):
        if not handle:
            raise RuntimeError("oracle model open failed")
        self.h = C.c_void_p(handle)
        self.cfg = Cfg()
        lib().orc_get_cfg(self.h, C.byref(self.cfg))
        self._trace = None

    @classmethod
    def synth(cls, cfg, seed):
        return cls(lib().orc_open_synth(C.byref(cfg), C.c_uint64(seed)))

    @classmethod
    def open(cls, data_dir, blob):
        return cls(lib().orc_open_dir(data_dir.encode(), blob.encode()))

    def run(self, tok, pos, want=True):
        return int(lib().orc_forward(self.h, int(tok), int(pos), int(bool(want))))

    def logits(self):
        return np.ctypeslib.as_array(lib().orc_logits(self.h), shape=(self.cfg.nvocab,)).copy()

    def hidden(self):
        return np.ctypeslib.as_array(lib().orc_hidden(self.h), shape=(self.cfg.d,)).copy()

    def enable_trace(self):
        self._trace = np.zeros((self.cfg.nl + 1, self.cfg.d), np.float32)
        lib().orc_set_trace(self.h, _p(self._trace))
        return self._trace

    def layer_q8(self, il, which):
        m = lib().orc_layer_q8(self.h, il, which).contents
        q = np.ctypeslib.as_array(C.cast(m.q, C.POINTER(C.c_int8)), shape=(m.rows, m.cols))
        s = np.ctypeslib.as_array(C.cast(m.s, C.POINTER(C.c_float)), shape=(m.rows, m.cols // 32))
        return q, s

    def layer_mx(self, il, which):
        m = lib().orc_layer_mx(self.h, il, which).contents
        nib = np.ctypeslib.as_array(C.cast(m.nib, C.POINTER(C.c_uint8)), shape=(m.rows * m.blocks * 16,))
        exps = np.ctypeslib.as_array(C.cast(m.exps, C.POINTER(C.c_uint8)), shape=(m.rows * m.blocks,))
        return nib, exps, m.rows, m.blocks

    def layer_f32(self, il, kind, n):
        return np.ctypeslib.as_array(lib().orc_layer_f32(self.h, il, kind), shape=(n,))

    def close(self):
        if self.h:
            lib().orc_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- qwen3moe model ---------------------------------------------------------------------------

class QCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("d", "nh", "nkv", "hd", "nl", "ne", "topk", "ff", "nvocab")] + [
        ("rope_base", C.c_float), ("rms_eps", C.c_float)]


def make_qcfg(d, nh, nkv, hd, nl, ne, topk, ff, nvocab, rope_base=1000000.0, rms_eps=1e-6):
    return QCfg(d, nh, nkv, hd, nl, ne, topk, ff, nvocab, rope_base, rms_eps)


_qready = False


def _qlib():
    global _qready
    L = lib()
    if not _qready:
        L.orcq_open_dir.restype = C.c_void_p
        L.orcq_open_dir.argtypes = [C.c_char_p, C.c_char_p]
        L.orcq_open_synth.restype = C.c_void_p
        L.orcq_open_synth.argtypes = [C.POINTER(QCfg), C.c_uint64]
        L.orcq_close.argtypes = [C.c_void_p]
        L.orcq_get_cfg.argtypes = [C.c_void_p, C.POINTER(QCfg)]
        L.orcq_forward.restype = C.c_uint32
        L.orcq_forward.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_int]
        L.orcq_logits.restype = C.POINTER(C.c_float)
        L.orcq_logits.argtypes = [C.c_void_p]
        L.orcq_hidden.restype = C.POINTER(C.c_float)
        L.orcq_hidden.argtypes = [C.c_void_p]
        L.orcq_set_trace.argtypes = [C.c_void_p, C.c_void_p]
        L.orcq_layer_k.restype = C.POINTER(C.c_uint8)
        L.orcq_layer_k.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.orcq_layer_f32.restype = C.POINTER(C.c_float)
        L.orcq_layer_f32.argtypes = [C.c_void_p, C.c_int, C.c_int]
        _qready = True
    return L


class QwenModel:
    """The oracle's qwen3moe model: run(tok, pos, want) as the reference's run closure."""

    def __init__(self, handle):
        if not handle:
            raise RuntimeError("oracle qwen model failed to open")
        self.h = handle
        self.cfg = QCfg()
        _qlib().orcq_get_cfg(self.h, C.byref(self.cfg))
        self._trace = None

    @classmethod
    def synth(cls, cfg, seed):
        return cls(_qlib().orcq_open_synth(C.byref(cfg), C.c_uint64(seed)))

    @classmethod
    def open(cls, data_dir, blob):
        return cls(_qlib().orcq_open_dir(data_dir.encode(), blob.encode()))

    def run(self, tok, pos, want=True):
        return int(_qlib().orcq_forward(self.h, int(tok), int(pos), int(bool(want))))

    def logits(self):
        return np.ctypeslib.as_array(_qlib().orcq_logits(self.h), shape=(self.cfg.nvocab,)).copy()

    def hidden(self):
        return np.ctypeslib.as_array(_qlib().orcq_hidden(self.h), shape=(self.cfg.d,)).copy()

    def enable_trace(self):
        self._trace = np.zeros((self.cfg.nl + 1, self.cfg.d), np.float32)
        _qlib().orcq_set_trace(self.h, _p(self._trace))
        return self._trace

    def layer_k(self, il, which):
        """Raw K-quant bytes of a matrix: (uint8 array, ggml type, rows, cols)."""
        ty = C.c_uint32(); rows = C.c_int(); cols = C.c_int()
        p = _qlib().orcq_layer_k(self.h, il, which, C.byref(ty), C.byref(rows), C.byref(cols))
        n = rows.value * (cols.value // 256) * (144 if ty.value == 12 else 210)
        return np.ctypeslib.as_array(p, shape=(n,)), ty.value, rows.value, cols.value

    def layer_f32(self, il, kind, n):
        return np.ctypeslib.as_array(_qlib().orcq_layer_f32(self.h, il, kind), shape=(n,))

    def close(self):
        if self.h:
            _qlib().orcq_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
