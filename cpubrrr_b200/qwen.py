"""Host-side mirror of the reference's qwen3moe engine interface.

`QwenEngine.run(tok, pos)` keeps the name, argument meaning and result of the closure `run` in the
reference's src/bin/engine_qwen2.rs:587-595 (the optional `want=False` skips the vocabulary
projection during a prompt, whose result the reference discards); `decode` is the decode loop of
`generate` (613-619) with the token id kept on the device.  Everything executes in libbrrr.so.
"""
import ctypes as C

import numpy as np

from ._lib import QwenCfg, check, lib


def make_qwen_cfg(n_embd, n_layer, n_head, n_head_kv, n_expert, n_expert_used, n_ff_exp, n_vocab, head_dim=128,
                  rope_freq_base=1000000.0, rms_eps=1e-6):
    return QwenCfg(n_embd, n_layer, n_head, n_head_kv, head_dim, n_expert, n_expert_used, n_ff_exp, n_vocab, rope_freq_base, rms_eps)


def qwen3_30b_a3b_cfg():
    """Qwen3-30B-A3B architecture: 48 layers, d 2048, 32/4 heads of 128, 128 experts top-8 of width 768, vocab 151936."""
    return make_qwen_cfg(2048, 48, 32, 4, 128, 8, 768, 151936)


class QwenEngine:
    MAXSEQ = 4096

    def __init__(self, handle):
        self._h = C.c_void_p(handle)
        self.cfg = QwenCfg()
        check(lib().brrr_qwen_cfg_get(self._h, C.byref(self.cfg)), "brrr_qwen_cfg_get")

    @classmethod
    def open(cls, data_dir, blob_path, device=0):
        """The reference's `engine_qwen2 <data-dir> <blob>` arguments."""
        h = C.c_void_p()
        check(lib().brrr_qwen_open(str(data_dir).encode(), str(blob_path).encode(), device, C.byref(h)), "brrr_qwen_open")
        return cls(h.value)

    @classmethod
    def synth(cls, cfg, seed, device=0):
        h = C.c_void_p()
        check(lib().brrr_qwen_open_synth(C.byref(cfg), seed, device, C.byref(h)), "brrr_qwen_open_synth")
        return cls(h.value)

    def close(self):
        if self._h:
            lib().brrr_qwen_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def run(self, tok, pos, want=True):
        out = C.c_uint32(0)
        check(lib().brrr_qwen_forward(self._h, int(tok), int(pos), int(bool(want)), C.byref(out)), "brrr_qwen_forward")
        return int(out.value)

    def prefill(self, ids, pos0=0):
        """Feed a prompt token by token (generate(), engine_qwen2.rs:606-609); returns the first generated token."""
        nxt = 0
        for i, t in enumerate(ids):
            nxt = self.run(t, pos0 + i, i == len(ids) - 1)
        return nxt

    def decode(self, first_tok, pos, n):
        out = np.empty(n, np.uint32)
        check(lib().brrr_qwen_decode(self._h, int(first_tok), int(pos), int(n), out.ctypes.data), "brrr_qwen_decode")
        return out

    def decode_enqueue(self, first_tok, pos, n):
        check(lib().brrr_qwen_decode_enqueue(self._h, int(first_tok), int(pos), int(n)), "brrr_qwen_decode_enqueue")

    def decode_wait(self, n):
        out = np.empty(n, np.uint32)
        check(lib().brrr_qwen_decode_wait(self._h, int(n), out.ctypes.data), "brrr_qwen_decode_wait")
        return out

    def logits(self):
        out = np.empty(self.cfg.n_vocab, np.float32)
        check(lib().brrr_qwen_logits(self._h, out.ctypes.data), "brrr_qwen_logits")
        return out

    def hidden(self):
        out = np.empty(self.cfg.n_embd, np.float32)
        check(lib().brrr_qwen_hidden(self._h, out.ctypes.data), "brrr_qwen_hidden")
        return out

    def run_trace(self, tok, pos):
        out = np.empty((self.cfg.n_layer + 1, self.cfg.n_embd), np.float32)
        check(lib().brrr_qwen_forward_trace(self._h, int(tok), int(pos), out.ctypes.data), "brrr_qwen_forward_trace")
        return out

    @property
    def stream(self):
        return lib().brrr_qwen_stream(self._h)

    def launches_per_step(self, want=True):
        return lib().brrr_qwen_launches_per_step(self._h, int(bool(want)))

    def bytes_per_step(self, pos):
        return int(lib().brrr_qwen_bytes_per_step(self._h, int(pos)))
