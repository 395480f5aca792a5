"""B200-native flash-attention forward/backward for the autoresearch GPT trainer.

The package is a thin host-side mirror of the attention entry points of the
reference's ``kernels/ops.mojo`` (same names, argument order and layouts) on top
of ``libarattn.so``, a C-ABI library of hand-written sm_100a kernels (tcgen05
MMA, TMEM accumulators, TMA-staged bf16 tiles).  There is no CPU or PyTorch
fallback: every call either runs the CUDA kernels or raises.
"""
from .config import ROPE_BASE, GPTConfig, precompute_rope, window_size  # noqa: F401
from ._lib import ArattnError, lib, lib_path  # noqa: F401
from .ops import (  # noqa: F401
    flash_attn_bwd_dkv,
    flash_attn_bwd_dq,
    flash_attn_bwd_precompute_d,
    flash_attn_fwd,
    linear_bwd_dw,
    linear_bwd_dx,
    linear_fwd,
    rope_bwd,
    rope_fwd,
)
from .attention import AttnParams, attn_bwd, attn_fwd, attention, check_device_status  # noqa: F401
from .sharding import shard_units  # noqa: F401

__all__ = [
    "ROPE_BASE", "GPTConfig", "precompute_rope", "window_size", "ArattnError", "lib", "lib_path",
    "rope_fwd", "rope_bwd", "flash_attn_fwd", "flash_attn_bwd_precompute_d", "flash_attn_bwd_dq",
    "flash_attn_bwd_dkv", "linear_fwd", "linear_bwd_dx", "linear_bwd_dw", "AttnParams", "attn_fwd", "attn_bwd", "attention", "check_device_status", "shard_units",
]
