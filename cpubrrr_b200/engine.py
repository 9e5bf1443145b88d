"""Host-side mirror of the reference engine's forward-pass interface.

`Engine.run(tok, pos, want)` and `Engine.run_tile(toks, pos0, want)` keep the names, argument
meaning and results of the closures `run` / `run_tile` in the reference's
src/bin/engine_gpt2.rs:1379-1393; `Engine.decode` is the decode loop of `generate` (1431-1438)
with the token id kept on the device.  Everything executes in libbrrr.so.
"""
import ctypes as C

import numpy as np

from ._lib import Cfg, check, lib


def make_cfg(n_embd, n_layer, n_head, n_head_kv, n_expert, n_expert_used, n_vocab, head_dim=64,
             sliding_window=128, rope_freq_base=150000.0, rms_eps=1e-5):
    return Cfg(n_embd, n_layer, n_head, n_head_kv, head_dim, n_expert, n_expert_used, n_embd, sliding_window,
               n_vocab, rope_freq_base, rms_eps)


def gptoss_20b_cfg():
    """gpt-oss-20b architecture: 24 layers, d 2880, 64/8 heads of 64, 32 experts top-4, vocab 201088."""
    return make_cfg(2880, 24, 64, 8, 32, 4, 201088)


class Engine:
    MAXSEQ = 4096

    def __init__(self, handle):
        self._h = C.c_void_p(handle)
        self.cfg = Cfg()
        check(lib().brrr_model_cfg(self._h, C.byref(self.cfg)), "brrr_model_cfg")

    @classmethod
    def open(cls, data_dir, blob_path, device=0):
        """Load config.txt / manifest.txt from data_dir and the GGUF blob (the reference's
        `engine_gpt2 <data-dir> <blob>` arguments)."""
        h = C.c_void_p()
        check(lib().brrr_model_open(str(data_dir).encode(), str(blob_path).encode(), device, C.byref(h)), "brrr_model_open")
        return cls(h.value)

    @classmethod
    def synth(cls, cfg, seed, device=0):
        """Seeded synthetic weights generated on the device."""
        h = C.c_void_p()
        check(lib().brrr_model_open_synth(C.byref(cfg), seed, device, C.byref(h)), "brrr_model_open_synth")
        return cls(h.value)

    def close(self):
        if self._h:
            lib().brrr_model_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- forward-pass interface of the reference
    def run(self, tok, pos, want=True):
        out = C.c_uint32(0)
        check(lib().brrr_forward(self._h, int(tok), int(pos), int(bool(want)), C.byref(out)), "brrr_forward")
        return int(out.value)

    def set_tile_prefill(self, on):
        """run_tile on token tiles of up to 512 rows (True, default) or one graph launch per token (False); same results."""
        check(lib().brrr_model_set_tile_prefill(self._h, int(bool(on))), "brrr_model_set_tile_prefill")

    def run_tile(self, toks, pos0, want=True):
        t = np.ascontiguousarray(toks, dtype=np.uint32)
        out = C.c_uint32(0)
        check(lib().brrr_forward_tile(self._h, t.ctypes.data, t.size, int(pos0), int(bool(want)), C.byref(out)), "brrr_forward_tile")
        return int(out.value)

    # ---- batched decode over independent sequences (one KV cache each)
    def batch_open(self, nseq):
        check(lib().brrr_batch_open(self._h, int(nseq)), "brrr_batch_open")

    def batch_prefill(self, seq, ids, pos0=0):
        t = np.ascontiguousarray(ids, dtype=np.uint32)
        check(lib().brrr_batch_prefill(self._h, int(seq), t.ctypes.data, t.size, int(pos0)), "brrr_batch_prefill")

    def batch_step(self, toks, pos, seq, logits=False):
        """One pass for the rows (toks[i], pos[i], seq[i]); returns the greedy next token of every row
        (and the rows' logits with logits=True)."""
        t = np.ascontiguousarray(toks, dtype=np.uint32)
        p = np.ascontiguousarray(pos, dtype=np.uint32)
        s = np.ascontiguousarray(seq, dtype=np.uint32)
        assert t.size == p.size == s.size
        out = np.empty(t.size, np.uint32)
        if logits:
            lg = np.empty((t.size, self.cfg.n_vocab), np.float32)
            check(lib().brrr_batch_step_logits(self._h, t.size, t.ctypes.data, p.ctypes.data, s.ctypes.data, out.ctypes.data, lg.ctypes.data), "brrr_batch_step_logits")
            return out, lg
        check(lib().brrr_batch_step(self._h, t.size, t.ctypes.data, p.ctypes.data, s.ctypes.data, out.ctypes.data), "brrr_batch_step")
        return out

    def decode(self, first_tok, pos, n):
        out = np.empty(n, np.uint32)
        check(lib().brrr_decode(self._h, int(first_tok), int(pos), int(n), out.ctypes.data), "brrr_decode")
        return out

    def decode_enqueue(self, first_tok, pos, n):
        check(lib().brrr_decode_enqueue(self._h, int(first_tok), int(pos), int(n)), "brrr_decode_enqueue")

    def decode_wait(self, n):
        out = np.empty(n, np.uint32)
        check(lib().brrr_decode_wait(self._h, int(n), out.ctypes.data), "brrr_decode_wait")
        return out

    def prefill(self, ids, pos0=0):
        """Feed a prompt; returns the first generated token (generate(), engine_gpt2.rs:1416-1426)."""
        return self.run_tile(ids, pos0, True)

    # ---- taps
    def logits(self):
        out = np.empty(self.cfg.n_vocab, np.float32)
        check(lib().brrr_logits(self._h, out.ctypes.data), "brrr_logits")
        return out

    def hidden(self):
        out = np.empty(self.cfg.n_embd, np.float32)
        check(lib().brrr_hidden(self._h, out.ctypes.data), "brrr_hidden")
        return out

    def run_trace(self, tok, pos):
        out = np.empty((self.cfg.n_layer + 1, self.cfg.n_embd), np.float32)
        check(lib().brrr_forward_trace(self._h, int(tok), int(pos), out.ctypes.data), "brrr_forward_trace")
        return out

    def moe_ffn_step(self, il, d_xn, d_x, d_top=None, d_wts=None):
        check(lib().brrr_moe_ffn_step(self._h, il, d_xn, d_x, d_top, d_wts), "brrr_moe_ffn_step")

    def moe_ffn_step_tc(self, il, d_xn, d_x, d_top=None, d_wts=None):
        check(lib().brrr_moe_ffn_step_tc(self._h, il, d_xn, d_x, d_top, d_wts), "brrr_moe_ffn_step_tc")

    @property
    def uses_tensor_experts(self):
        return bool(lib().brrr_model_uses_tensor_experts(self._h))

    @property
    def stream(self):
        return lib().brrr_model_stream(self._h)

    def launches_per_step(self, want=True):
        return lib().brrr_model_launches_per_step(self._h, int(bool(want)))

    def wait_fallbacks(self):
        """Times a bounded device wait of the speculative step ran out and the model fell back to the plain step (0 or 1)."""
        return int(lib().brrr_model_wait_fallbacks(self._h))

    def spec_redos(self):
        """Steps re-run because the routing estimate missed an expert (performance counter)."""
        return int(lib().brrr_model_spec_redos(self._h))

    def bytes_per_step(self, pos):
        return int(lib().brrr_model_bytes_per_step(self._h, int(pos)))

    def stage_times(self, pos, reps=20):
        """Per kernel class: (name, ms per launch, algorithmic bytes per launch, launches per step)."""
        L = lib()
        out = []
        for st in range(L.brrr_stage_count()):
            name = L.brrr_stage_name(st).decode()
            if name == "finish_token":
                continue
            ms, by, n = C.c_float(), C.c_uint64(), C.c_int()
            check(L.brrr_stage_time(self._h, st, int(pos), int(reps), C.byref(ms), C.byref(by), C.byref(n)), "brrr_stage_time")
            out.append((name, float(ms.value), int(by.value), int(n.value)))
        return out
