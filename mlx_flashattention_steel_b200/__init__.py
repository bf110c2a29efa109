"""B200-native flash attention behind the ``mlx_mfa`` operator surface.

Public names follow ``mlx_mfa/__init__.py:96-133`` of the reference for the
attention hot path; everything runs hand-written sm_100a CUDA through
``libb200fa.so`` (C-ABI in ``include/b200fa.h``).
"""
from .attention import (
    flash_attention,
    flash_attention_kvcache,
    flash_attention_paged,
    flash_attention_varlen,
    get_device_info,
    get_supported_configs,
    is_mfa_available,
    kernel_status,
    paged_kv_gather,
    paged_kv_gather_dequant,
)

from .host_pipeline import HostPipeline, flash_attention_from_host
from .kv_cache import PagedKVCache, kv_append
from .packed import (
    flash_attention_kv_packed,
    flash_attention_qkv_packed,
    flash_attention_varlen_kv_packed,
    flash_attention_varlen_qkv_packed,
)
from .sparse import flash_attention_sparse, make_causal_block_mask, make_sliding_window_mask
from .rope import apply_rope, flash_attention_rope, make_rope_3d_tables

__version__ = "0.1.0"

__all__ = [
    "flash_attention",
    "flash_attention_varlen",
    "flash_attention_kvcache",
    "flash_attention_paged",
    "paged_kv_gather",
    "paged_kv_gather_dequant",
    "flash_attention_rope",
    "flash_attention_sparse",
    "make_causal_block_mask",
    "make_sliding_window_mask",
    "flash_attention_qkv_packed",
    "flash_attention_kv_packed",
    "flash_attention_varlen_qkv_packed",
    "flash_attention_varlen_kv_packed",
    "apply_rope",
    "make_rope_3d_tables",
    "PagedKVCache",
    "kv_append",
    "flash_attention_from_host",
    "HostPipeline",
    "kernel_status",
    "is_mfa_available",
    "get_device_info",
    "get_supported_configs",
]
