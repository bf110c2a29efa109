"""Block-sparse attention: ``flash_attention_sparse`` and the mask builders (mlx_mfa/attention.py:717-810, 1219-1311).

A block mask is a boolean ``[NQ_tiles, NK_tiles]`` grid over (query block, key block) cells whose sizes are the
reference's tile sizes for the head dimension (32 x 32 up to D = 64, 32 x 16 above), so masks built for the reference
mean the same thing here.  Key tiles without an active cell are skipped; cells of a visited tile that are off are
masked element-wise.  The mask rides in the descriptor: the forward runs the tcgen05 kernel's feature instantiation
(head_dim 64 / 128), the backward the portable kernel.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .attention import _DTYPE_CODE, _FlashAttnFn, _SUPPORTED_HDIMS, _as_tensor, _require_cuda


def _steel_block_config(head_dim: int) -> Tuple[int, int]:
    """(BQ, BK) of a mask cell for this head_dim (mlx_mfa/attention.py:717-727)."""
    if head_dim <= 64:
        return (32, 32)
    return (32, 16)


def make_causal_block_mask(seq_len: int, head_dim: int = 128, device=None) -> torch.Tensor:
    """Cell (q, k) is on when the key block's first token <= the query block's last token (734-757)."""
    BQ, BK = _steel_block_config(head_dim)
    NQ, NK = (seq_len + BQ - 1) // BQ, (seq_len + BK - 1) // BK
    q_end = (torch.arange(NQ, dtype=torch.int64) + 1) * BQ - 1
    k_start = torch.arange(NK, dtype=torch.int64) * BK
    mask = k_start[None, :] <= q_end[:, None]
    return mask if device is None else mask.to(device)


def make_sliding_window_mask(seq_len: int, window_size: int, head_dim: int = 128, causal: bool = False,
                             device=None) -> torch.Tensor:
    """Cell (q, k) is on when the key block overlaps ``[centre - window_size, centre + window_size]`` around the query
    block's centre token; with ``causal`` also key block start <= query block end (760-806)."""
    BQ, BK = _steel_block_config(head_dim)
    NQ, NK = (seq_len + BQ - 1) // BQ, (seq_len + BK - 1) // BK
    rows, cols = torch.arange(NQ, dtype=torch.int64), torch.arange(NK, dtype=torch.int64)
    q_centre = rows * BQ + BQ // 2
    k_start = cols * BK
    k_end = k_start + BK - 1
    mask = (k_end[None, :] >= q_centre[:, None] - window_size) & (k_start[None, :] <= q_centre[:, None] + window_size)
    if causal:
        mask = mask & (k_start[None, :] <= ((rows + 1) * BQ - 1)[:, None])
    return mask if device is None else mask.to(device)


def flash_attention_sparse(q, k, v, block_mask, scale: Optional[float] = None, causal: bool = False, stream=None,
                           backward: str = "sdpa") -> torch.Tensor:
    """Attention restricted to the (query block, key block) cells that ``block_mask`` switches on
    (mlx_mfa/attention.py:1219-1311).  ``block_mask``: bool ``[ceil(N/BQ), ceil(S/BK)]`` with (BQ, BK) from
    ``_steel_block_config(D)``; ``causal`` masks additionally inside the active cells.  Rows whose cells are all off
    give zeros.  ``backward`` names the reference's three backward strategies; here one CUDA backward serves them all."""
    q, k, v = _as_tensor(q, "q"), _as_tensor(k, "k"), _as_tensor(v, "v")
    block_mask = _as_tensor(block_mask, "block_mask")
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("flash_attention_sparse expects 4-D tensors [batch, heads, seq, head_dim]")
    B, H, N, D = q.shape
    S = k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"flash_attention_sparse requires float16 or bfloat16; got {q.dtype}. "
                         "For float32, use flash_attention() with a float mask.")
    if D not in _SUPPORTED_HDIMS:
        raise ValueError(f"flash_attention_sparse: head_dim must be in {sorted(_SUPPORTED_HDIMS)}, got {D}")
    if block_mask.ndim != 2:
        raise ValueError(f"block_mask must be 2-D [NQ_tiles, NK_tiles]; got shape {list(block_mask.shape)}")
    BQ, BK = _steel_block_config(D)
    NQ, NK = (N + BQ - 1) // BQ, (S + BK - 1) // BK
    if block_mask.shape[0] != NQ or block_mask.shape[1] != NK:
        raise ValueError(f"block_mask shape {list(block_mask.shape)} does not match expected [{NQ}, {NK}] "
                         f"for seq_len={N}/{S}, head_dim={D} (BQ={BQ}, BK={BK})")
    if backward not in ("sdpa", "sdpa_sparse", "steel_sparse"):
        raise ValueError(f"flash_attention_sparse: unknown backward {backward!r}")
    if k.shape[1] != H and H % k.shape[1] != 0:
        raise ValueError(f"flash_attention GQA: q_heads ({H}) must be divisible by kv_heads ({k.shape[1]}).")
    _require_cuda(q, k, v, block_mask)
    bm = (block_mask != 0).to(torch.uint8).contiguous()
    out, _ = _FlashAttnFn.apply(q, k, v, float(scale), bool(causal), 0.0, -1, False, stream, None, (bm, BQ, BK))
    return out
