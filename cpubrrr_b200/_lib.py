"""ctypes binding of libbrrr.so — every symbol declared in include/brrr.h."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# BRRR_LIBRARY: another build of the same library (the tests load the test-hook build this way)
LIB_PATH = os.environ.get("BRRR_LIBRARY") or os.path.join(HERE, "libbrrr.so")


class BrrrError(RuntimeError):
    pass


class Cfg(C.Structure):
    """brrr_cfg: the keys of the data directory's config.txt."""
    _fields_ = [(n, C.c_int32) for n in ("n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "n_expert",
                                         "n_expert_used", "n_ff_exp", "sliding_window", "n_vocab")] + [
        ("rope_freq_base", C.c_float), ("rms_eps", C.c_float)]


class QwenCfg(C.Structure):
    """brrr_qwen_cfg: config.txt keys of the qwen3moe engine."""
    _fields_ = [(n, C.c_int32) for n in ("n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "n_expert",
                                         "n_expert_used", "n_ff_exp", "n_vocab")] + [
        ("rope_freq_base", C.c_float), ("rms_eps", C.c_float)]


_P = C.c_void_p
_I = C.c_int
# name -> (restype, argtypes); the authoritative list of exported entry points
SIGNATURES = {
    "brrr_strerror": (C.c_char_p, [_I]),
    "brrr_last_cuda_error": (C.c_char_p, []),
    "brrr_model_open": (_I, [C.c_char_p, C.c_char_p, _I, C.POINTER(_P)]),
    "brrr_model_open_synth": (_I, [C.POINTER(Cfg), C.c_uint64, _I, C.POINTER(_P)]),
    "brrr_model_cfg": (_I, [_P, C.POINTER(Cfg)]),
    "brrr_model_close": (None, [_P]),
    "brrr_forward": (_I, [_P, C.c_uint32, C.c_uint32, _I, C.POINTER(C.c_uint32)]),
    "brrr_forward_tile": (_I, [_P, _P, C.c_uint32, C.c_uint32, _I, C.POINTER(C.c_uint32)]),
    "brrr_model_set_tile_prefill": (_I, [_P, _I]),
    "brrr_batch_open": (_I, [_P, _I]),
    "brrr_batch_prefill": (_I, [_P, C.c_uint32, _P, C.c_uint32, C.c_uint32]),
    "brrr_batch_step": (_I, [_P, _I, _P, _P, _P, _P]),
    "brrr_batch_step_logits": (_I, [_P, _I, _P, _P, _P, _P, _P]),
    "brrr_decode": (_I, [_P, C.c_uint32, C.c_uint32, C.c_uint32, _P]),
    "brrr_decode_enqueue": (_I, [_P, C.c_uint32, C.c_uint32, C.c_uint32]),
    "brrr_decode_wait": (_I, [_P, C.c_uint32, _P]),
    "brrr_logits": (_I, [_P, _P]),
    "brrr_hidden": (_I, [_P, _P]),
    "brrr_forward_trace": (_I, [_P, C.c_uint32, C.c_uint32, _P]),
    "brrr_model_stream": (_P, [_P]),
    "brrr_model_launches_per_step": (_I, [_P, _I]),
    "brrr_model_spec_redos": (C.c_uint64, [_P]),
    "brrr_model_wait_fallbacks": (C.c_uint64, [_P]),
    "brrr_model_bytes_per_step": (C.c_uint64, [_P, C.c_uint32]),
    "brrr_stage_count": (_I, []),
    "brrr_stage_name": (C.c_char_p, [_I]),
    "brrr_stage_time": (_I, [_P, _I, C.c_uint32, _I, C.POINTER(C.c_float), C.POINTER(C.c_uint64), C.POINTER(_I)]),
    "brrr_model_open_synth_ep": (_I, [C.POINTER(Cfg), C.c_uint64, _I, _I, _I, C.POINTER(_P)]),
    "brrr_model_open_ep": (_I, [C.c_char_p, C.c_char_p, _I, _I, _I, C.POINTER(_P)]),
    "brrr_model_ep_handle": (_I, [_P, _P]),
    "brrr_model_ep_attach": (_I, [_P, _P]),
    "brrr_model_ep_info": (_I, [_P, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I), C.POINTER(_I)]),
    "brrr_tokenizer_open": (_I, [C.c_char_p, C.POINTER(_P)]),
    "brrr_tokenizer_close": (None, [_P]),
    "brrr_tokenizer_size": (C.c_uint32, [_P]),
    "brrr_tokenizer_token": (_I, [_P, C.c_uint32, C.POINTER(C.c_char_p), C.POINTER(C.c_uint32)]),
    "brrr_tokenizer_special": (_I, [_P, C.c_char_p, C.POINTER(C.c_uint32)]),
    "brrr_tokenizer_encode": (_I, [_P, C.c_char_p, C.c_size_t, C.c_uint32, _P, C.c_size_t, C.POINTER(C.c_size_t)]),
    "brrr_rng_seed": (C.c_uint64, [C.c_uint64]),
    "brrr_sample_logits": (C.c_uint32, [_P, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint64)]),
    "brrr_chat_prompt": (_I, [_P, C.c_char_p, _P, C.c_size_t, C.POINTER(C.c_size_t)]),
    "brrr_generate": (_I, [_P, _P, _P, C.c_size_t, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint64), _P, _P, _P, C.c_size_t, _P]),
    "brrr_serve_parse": (_I, [C.c_char_p, C.POINTER(C.c_float), C.POINTER(C.c_uint64), C.POINTER(C.c_uint32), C.c_char_p, C.c_size_t]),
    "brrr_cli_main": (_I, [_I, _P]),
    "brrr_qwen_open": (_I, [C.c_char_p, C.c_char_p, _I, C.POINTER(_P)]),
    "brrr_qwen_open_synth": (_I, [C.POINTER(QwenCfg), C.c_uint64, _I, C.POINTER(_P)]),
    "brrr_qwen_cfg_get": (_I, [_P, C.POINTER(QwenCfg)]),
    "brrr_qwen_close": (None, [_P]),
    "brrr_qwen_forward": (_I, [_P, C.c_uint32, C.c_uint32, _I, C.POINTER(C.c_uint32)]),
    "brrr_qwen_decode": (_I, [_P, C.c_uint32, C.c_uint32, C.c_uint32, _P]),
    "brrr_qwen_decode_enqueue": (_I, [_P, C.c_uint32, C.c_uint32, C.c_uint32]),
    "brrr_qwen_decode_wait": (_I, [_P, C.c_uint32, _P]),
    "brrr_qwen_logits": (_I, [_P, _P]),
    "brrr_qwen_hidden": (_I, [_P, _P]),
    "brrr_qwen_forward_trace": (_I, [_P, C.c_uint32, C.c_uint32, _P]),
    "brrr_qwen_stream": (_P, [_P]),
    "brrr_qwen_launches_per_step": (_I, [_P, _I]),
    "brrr_qwen_bytes_per_step": (C.c_uint64, [_P, C.c_uint32]),
    "brrr_qwen_chat_prompt": (_I, [_P, C.c_char_p, _P, C.c_size_t, C.POINTER(C.c_size_t)]),
    "brrr_qwen_generate": (_I, [_P, _P, _P, C.c_size_t, C.c_uint32, _P, _P, _P, C.c_size_t, _P]),
    "brrr_qwen_serve_parse": (_I, [C.c_char_p, C.POINTER(C.c_uint32), C.c_char_p, C.c_size_t]),
    "brrr_qwen_cli_main": (_I, [_I, _P]),
    "brrr_quant_q8": (_I, [_P, _I, _P, _P, _P]),
    "brrr_quant_q8k": (_I, [_P, _I, _P, _P, _P, _P]),
    "brrr_q4k_matvec": (_I, [_P, _I, _I, _P, _P, _P, _P, _P, _P]),
    "brrr_q6k_matvec": (_I, [_P, _I, _I, _P, _P, _P, _P, _P]),
    "brrr_rmsnorm_quant": (_I, [_P, _P, C.c_float, _I, _P, _P, _P, _P]),
    "brrr_fold_norm": (_I, [_P, _P, _I, _I, _P, _P, _P, _P, C.c_float, _P, _P, _I, _P]),
    "brrr_q8mat_from_bf16": (_I, [_P, _I, _I, C.POINTER(_P), _P]),
    "brrr_q8mat_export": (_I, [_P, _P, _P, _P]),
    "brrr_q8mat_free": (None, [_P]),
    "brrr_q8_matvec": (_I, [_P, _P, _P, _P, _P]),
    "brrr_q8_matmul_rows": (_I, [_P, _P, _P, _I, _P, _I, _I, _P]),
    "brrr_mxmat_from_gguf": (_I, [_P, _I, _I, C.POINTER(_P), _P]),
    "brrr_mxmat_free": (None, [_P]),
    "brrr_mx_matvec": (_I, [_P, _I, _I, _P, _P, _P, _P, _P]),
    "brrr_mx_matmul_tile": (_I, [_P, _I, _I, _P, _P, _I, _P, _I, _P]),
    "brrr_moe_ffn_tile": (_I, [_P, _I, _P, _P, _I, _P, _P]),
    "brrr_router_topk": (_I, [_P, _P, _P, _I, _I, _I, _P, _P, _P, _P]),
    "brrr_router_topk_noalloc": (_I, [_P, _P, _P, _I, _I, _I, _P, _P, _P, _P]),
    "brrr_swiglu_quant": (_I, [_P, _I, _I, _P, _P, _P]),
    "brrr_attn_decode": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P]),
    "brrr_rope_table": (_I, [C.POINTER(Cfg), _P]),
    "brrr_moe_ffn_step": (_I, [_P, _I, _P, _P, _P, _P]),
    "brrr_moe_ffn_step_tc": (_I, [_P, _I, _P, _P, _P, _P]),
    "brrr_model_uses_tensor_experts": (_I, [_P]),
    "brrr_synth_tensor": (_I, [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, _P, _P]),
    "brrr_expf": (_I, [_P, _I, _P, _P]),
}

_lib = None


def lib():
    """Load libbrrr.so (built by `python -m cpubrrr_b200.build`). Raises if it is missing: the
    engine has no other execution path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise BrrrError(f"{LIB_PATH} is missing: build it with `python -m cpubrrr_b200.build`")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)      # AttributeError if the library does not export it
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status, what=""):
    if status != 0:
        L = lib()
        msg = L.brrr_strerror(status).decode()
        detail = L.brrr_last_cuda_error().decode()
        raise BrrrError(f"{what}: {msg}" + (f" ({detail})" if detail else ""))
