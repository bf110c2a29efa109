"""Attention from fused QKV / KV tensors (mlx_mfa/attention.py:3092-3425).

The wrappers only take views: the kernels read q, k and v through their strides (TMA tensor maps over
``[B, H, rows, D]`` with arbitrary 16-byte-multiple strides), so a fused tensor is attended in place where the
reference's path makes contiguous copies first.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .attention import _as_tensor, flash_attention, flash_attention_varlen


def _split_qkv(qkv: torch.Tensor, num_heads: Optional[int], num_kv_heads: Optional[int], who: str) -> Tuple[torch.Tensor, ...]:
    if qkv.ndim == 3:                                     # [B, N, (Hq + 2*Hkv) * D] flat concat
        if num_heads is None:
            raise ValueError(f"{who}: num_heads required for [B,N,3*H*D] layout")
        B, N, fused = qkv.shape
        Hq = num_heads
        Hkv = num_kv_heads if num_kv_heads is not None else Hq
        D = fused // (Hq + 2 * Hkv)
        if D * (Hq + 2 * Hkv) != fused:
            raise ValueError(f"{who}: fused dim {fused} not divisible by (H_q={Hq} + 2*H_kv={Hkv}) * D={D}")
        q_end, k_end = Hq * D, (Hq + Hkv) * D
        q = qkv[..., :q_end].reshape(B, N, Hq, D).permute(0, 2, 1, 3)
        k = qkv[..., q_end:k_end].reshape(B, N, Hkv, D).permute(0, 2, 1, 3)
        v = qkv[..., k_end:].reshape(B, N, Hkv, D).permute(0, 2, 1, 3)
        return q, k, v
    if qkv.ndim == 5:                                     # [B, H, N, 3, D] head-first
        if qkv.shape[3] != 3:
            raise ValueError(f"{who}: expected dim 3 == 3, got {qkv.shape[3]}")
        Hq = qkv.shape[1]
        Hkv = num_kv_heads if num_kv_heads is not None else Hq
        return qkv[:, :Hq, :, 0, :], qkv[:, :Hkv, :, 1, :], qkv[:, :Hkv, :, 2, :]
    raise ValueError(f"{who}: unsupported shape {tuple(qkv.shape)}. Expected [B,N,3*H*D] (ndim=3) or [B,H,N,3,D] (ndim=5).")


def _split_kv(kv: torch.Tensor, num_kv_heads: Optional[int], who: str) -> Tuple[torch.Tensor, torch.Tensor]:
    if kv.ndim == 3:                                      # [B, S, 2*Hkv*D]
        if num_kv_heads is None:
            raise ValueError(f"{who}: num_kv_heads required for [B,S,2*H_kv*D] layout")
        B, S, fused = kv.shape
        Hkv = num_kv_heads
        D = fused // (2 * Hkv)
        if D * 2 * Hkv != fused:
            raise ValueError(f"{who}: fused dim {fused} not divisible by 2*H_kv={Hkv}")
        k = kv[..., :Hkv * D].reshape(B, S, Hkv, D).permute(0, 2, 1, 3)
        v = kv[..., Hkv * D:].reshape(B, S, Hkv, D).permute(0, 2, 1, 3)
        return k, v
    if kv.ndim == 5:                                      # [B, Hkv, S, 2, D]
        if kv.shape[3] != 2:
            raise ValueError(f"{who}: expected dim 3 == 2, got {kv.shape[3]}")
        return kv[:, :, :, 0, :], kv[:, :, :, 1, :]
    raise ValueError(f"{who}: unsupported shape {tuple(kv.shape)}. Expected [B,S,2*H_kv*D] (ndim=3) or [B,H_kv,S,2,D] (ndim=5).")


def flash_attention_qkv_packed(qkv, *, scale: Optional[float] = None, causal: bool = False, num_heads: Optional[int] = None,
                               num_kv_heads: Optional[int] = None, stream=None) -> torch.Tensor:
    """Attention from a fused ``[B, N, 3*H*D]`` or ``[B, H, N, 3, D]`` tensor; returns ``[B, H, N, D]``
    (mlx_mfa/attention.py:3092-3175)."""
    q, k, v = _split_qkv(_as_tensor(qkv, "qkv"), num_heads, num_kv_heads, "flash_attention_qkv_packed")
    return flash_attention(q, k, v, scale=scale, causal=causal, stream=stream)


def flash_attention_kv_packed(q, kv, *, scale: Optional[float] = None, causal: bool = False,
                              num_kv_heads: Optional[int] = None, stream=None) -> torch.Tensor:
    """Attention with K and V fused as ``[B, S, 2*H_kv*D]`` or ``[B, H_kv, S, 2, D]`` (3178-3256)."""
    k, v = _split_kv(_as_tensor(kv, "kv"), num_kv_heads, "flash_attention_kv_packed")
    return flash_attention(q, k, v, scale=scale, causal=causal, stream=stream)


def flash_attention_varlen_qkv_packed(qkv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int, *,
                                      scale: Optional[float] = None, causal: bool = False, num_heads: Optional[int] = None,
                                      num_kv_heads: Optional[int] = None, stream=None) -> torch.Tensor:
    """Packed-sequence attention from ``[1, H, total, 3, D]`` or ``[1, total, 3*H*D]`` (3260-3343)."""
    q, k, v = _split_qkv(_as_tensor(qkv, "qkv"), num_heads, num_kv_heads, "flash_attention_varlen_qkv_packed")
    return flash_attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale=scale,
                                  causal=causal, stream=stream)


def flash_attention_varlen_kv_packed(q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int, *,
                                     scale: Optional[float] = None, causal: bool = False,
                                     num_kv_heads: Optional[int] = None, stream=None) -> torch.Tensor:
    """Packed-sequence attention with K and V fused as ``[1, H_kv, total_kv, 2, D]`` or ``[1, total_kv, 2*H_kv*D]``
    (3347-3425)."""
    k, v = _split_kv(_as_tensor(kv, "kv"), num_kv_heads, "flash_attention_varlen_kv_packed")
    return flash_attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale=scale,
                                  causal=causal, stream=stream)
