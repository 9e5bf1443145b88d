"""cpubrrr_b200 — B200-native per-token MoE decode engine (gpt-oss family).

The package is a thin host-side mirror of the reference engine's interface over the C ABI of
libbrrr.so (include/brrr.h).  All computation runs in hand-written sm_100a CUDA kernels; there is
no CPU fallback: importing `cpubrrr_b200.lib()` without the built library raises.
"""
from ._lib import lib, BrrrError, Cfg, QwenCfg, LIB_PATH  # noqa: F401
from .engine import Engine, gptoss_20b_cfg, make_cfg  # noqa: F401
from .qwen import QwenEngine, make_qwen_cfg, qwen3_30b_a3b_cfg  # noqa: F401
