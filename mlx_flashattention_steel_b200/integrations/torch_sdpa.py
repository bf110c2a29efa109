"""PyTorch integration — drop-in attention for models that call ``torch.nn.functional.scaled_dot_product_attention``.

The reference patches ``mlx_lm.models.base.scaled_dot_product_attention`` so that every mlx-lm model uses its kernel
when the configuration is supported and falls back to the original function otherwise, with call statistics
(mlx_mfa/integrations/mlx_lm.py:66-260).  This module is the same idea for a PyTorch serving or training stack:

    from mlx_flashattention_steel_b200.integrations.torch_sdpa import patch_torch_sdpa
    patch_torch_sdpa()          # F.scaled_dot_product_attention now routes to libb200fa where it can
    ...
    unpatch_torch_sdpa()

Routed to the CUDA kernels: CUDA tensors ``[B, H, N, D]``, f16 / bf16 (float32 too for D in {64, 128}), a supported
head_dim, no dropout, and either no mask or ``is_causal=True`` (the kernel's causal mask is lower-right aligned, which
equals PyTorch's top-left one when N == S; other shapes with ``is_causal`` fall back).  Everything else -- explicit
masks, dropout, unsupported shapes, CPU tensors -- goes to the function that was there before the patch, exactly as
the reference falls back to mlx-lm's own SDPA.  ``register_hf_attention()`` adds the same routing to Hugging Face
transformers as ``attn_implementation="b200fa"``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import flash_attention, get_supported_configs, is_mfa_available

_original_sdpa = None
_stats = {"forward_calls": 0, "steel_calls": 0, "fallback_calls": 0}


def get_stats() -> dict:
    """Copy of the per-session call statistics (mlx_mfa/integrations/mlx_lm.py:42-65, 262-283)."""
    return dict(_stats)


def _reset_stats() -> None:
    for k in _stats:
        _stats[k] = 0


def _eligible(query, key, value, attn_mask, dropout_p, is_causal, enable_gqa) -> bool:
    if attn_mask is not None or dropout_p != 0.0:
        return False
    if not (isinstance(query, torch.Tensor) and query.is_cuda and key.is_cuda and value.is_cuda):
        return False
    if query.ndim != 4 or key.ndim != 4 or value.ndim != 4:
        return False
    D = query.shape[-1]
    if key.shape[-1] != D or value.shape[-1] != D or key.dtype != query.dtype or value.dtype != query.dtype:
        return False
    dims = get_supported_configs()["head_dims"]
    if D not in dims:
        return False
    if query.dtype == torch.float32:
        if D not in (64, 128):
            return False
    elif query.dtype not in (torch.float16, torch.bfloat16):
        return False
    Hq, Hkv = query.shape[1], key.shape[1]
    if Hq != Hkv and not (enable_gqa and Hq % Hkv == 0):
        return False
    if key.shape[2] != value.shape[2] or key.shape[0] != query.shape[0]:
        return False
    if is_causal and query.shape[2] != key.shape[2]:
        return False                      # PyTorch's is_causal is top-left aligned; the kernel's is lower-right
    if query.requires_grad or key.requires_grad or value.requires_grad:
        if query.dtype == torch.float32 or D == 256:
            return False                  # no CUDA backward for these
    return True


def scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p: float = 0.0, is_causal: bool = False,
                                 scale: Optional[float] = None, enable_gqa: bool = False, **kwargs):
    """Signature of ``torch.nn.functional.scaled_dot_product_attention``.  Routes to ``flash_attention`` when the
    call is eligible, else to the original function (PyTorch's own when this module has not been patched in)."""
    _stats["forward_calls"] += 1
    fallback = _original_sdpa if _original_sdpa is not None else torch.nn.functional.scaled_dot_product_attention
    if kwargs or not is_mfa_available() or not _eligible(query, key, value, attn_mask, dropout_p, is_causal, enable_gqa):
        _stats["fallback_calls"] += 1
        if fallback is scaled_dot_product_attention:       # patched in and nothing saved: cannot recurse
            raise RuntimeError("no fallback attention function available")
        extra = dict(kwargs)
        if enable_gqa:
            extra["enable_gqa"] = True
        return fallback(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal, scale=scale, **extra)
    _stats["steel_calls"] += 1
    if scale is None:
        scale = 1.0 / math.sqrt(query.shape[-1])
    return flash_attention(query, key, value, scale=scale, causal=bool(is_causal))


def patch_torch_sdpa(verbose: bool = True) -> bool:
    """Replace ``torch.nn.functional.scaled_dot_product_attention``.  Idempotent; returns False (and leaves PyTorch
    alone) when no B200 / library is available.  Statistics reset at each fresh patch."""
    global _original_sdpa
    if _original_sdpa is not None:
        return True
    if not is_mfa_available():
        if verbose:
            print("[b200fa] Warning: libb200fa / CUDA device not available, torch SDPA patch skipped")
        return False
    _reset_stats()
    _original_sdpa = torch.nn.functional.scaled_dot_product_attention
    torch.nn.functional.scaled_dot_product_attention = scaled_dot_product_attention
    if verbose:
        print(f"[b200fa] Patched torch.nn.functional.scaled_dot_product_attention "
              f"(head_dims={sorted(get_supported_configs()['head_dims'])})")
    return True


def unpatch_torch_sdpa() -> None:
    """Restore the function that was in place before ``patch_torch_sdpa``."""
    global _original_sdpa
    if _original_sdpa is not None:
        torch.nn.functional.scaled_dot_product_attention = _original_sdpa
        _original_sdpa = None


def hf_attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0, scaling: Optional[float] = None,
                         is_causal: Optional[bool] = None, **kwargs):
    """Attention function in the form Hugging Face transformers' ``AttentionInterface`` expects: q/k/v ``[B, H, N, D]``
    in, ``([B, N, H, D], None)`` out.  A 4-D mask or dropout sends the call to PyTorch's SDPA."""
    causal = bool(is_causal) if is_causal is not None else (attention_mask is None and query.shape[2] > 1 and
                                                            getattr(module, "is_causal", True))
    if attention_mask is not None:
        causal = False
    out = scaled_dot_product_attention(query, key, value, attn_mask=attention_mask, dropout_p=dropout, is_causal=causal,
                                       scale=scaling, enable_gqa=query.shape[1] != key.shape[1])
    return out.transpose(1, 2).contiguous(), None


def register_hf_attention(name: str = "b200fa") -> bool:
    """Register ``hf_attention_forward`` with transformers (``attn_implementation=name``).  False when transformers
    (or its AttentionInterface) is not importable."""
    try:
        from transformers import AttentionInterface
    except Exception:
        return False
    AttentionInterface.register(name, hf_attention_forward)
    return True
