"""Rotary position embeddings: the rotation pass, the reference's table builder and ``flash_attention_rope``.

Follows mlx_mfa/attention.py:319-555 (``make_rope_3d_tables``, ``flash_attention_rope``) and 2128-2246
(``_apply_rope_mlx``, ``_apply_rope_to_qk``).  The reference rotates inside its Metal kernel; here
``apply_rope`` is one launch of ``b200fa_rope`` per tensor (per-batch offsets included, where the reference
loops over the batch) followed by the ordinary attention kernels.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import _lib
from .attention import _DTYPE_CODE, _as_tensor, _require_cuda, _stream_ptr, flash_attention


def make_rope_3d_tables(grid_h: int, grid_w: int, num_frames: int, d_h: Optional[int] = None, d_w: Optional[int] = None,
                        d_t: Optional[int] = None, head_dim: int = 128, theta: float = 10000.0,
                        device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(cos, sin)`` float32 ``[N, D/2]`` for video attention, ``N = grid_h*grid_w*num_frames`` tokens in
    (T, H, W) row-major order.  The D/2 pairs split into three consecutive bands: height (position = patch row),
    width (patch column), time (frame); band of width d uses frequencies ``theta**(-2j/d)``
    (mlx_mfa/attention.py:319-417)."""
    if d_h is None:
        d_h = (head_dim // 3) & ~1
    if d_w is None:
        d_w = (head_dim // 3) & ~1
    if d_t is None:
        d_t = head_dim - d_h - d_w
        if d_t % 2:
            d_t -= 1
            d_h += 1
    if d_h % 2 or d_w % 2 or d_t % 2:
        raise ValueError(f"d_h, d_w, d_t must all be even. Got d_h={d_h}, d_w={d_w}, d_t={d_t}.")
    per_frame = grid_h * grid_w
    tok = np.arange(num_frames * per_frame, dtype=np.int64)
    coords = (tok % per_frame // grid_w, tok % per_frame % grid_w, tok // per_frame)      # y, x, t
    cos_parts, sin_parts = [], []
    for pos, d in zip(coords, (d_h, d_w, d_t)):
        j = np.arange(d // 2, dtype=np.float32)
        freq = (1.0 / (theta ** (2.0 * j / d))).astype(np.float32) if d else np.zeros(0, np.float32)
        ang = pos[:, None].astype(np.float32) * freq[None, :]
        cos_parts.append(np.cos(ang))
        sin_parts.append(np.sin(ang))
    cos = torch.from_numpy(np.concatenate(cos_parts, axis=1).astype(np.float32))
    sin = torch.from_numpy(np.concatenate(sin_parts, axis=1).astype(np.float32))
    if device is not None:
        cos, sin = cos.to(device), sin.to(device)
    return cos, sin


def _rope_raw(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, offset, interleaved: bool, rot: int, inverse: bool,
              stream, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    B, H, N, D = x.shape
    if out is None:
        out = torch.empty((B, H, N, D), dtype=x.dtype, device=x.device)
    offs_t, offs_i = None, 0
    if isinstance(offset, torch.Tensor):
        offs_t = offset.to(device=x.device, dtype=torch.int32).contiguous()
        if offs_t.numel() != B:
            raise ValueError(f"cache_seqlens length {offs_t.numel()} must equal batch size B={B}")
    else:
        offs_i = int(offset)
    xs = (C.c_int64 * 3)(*x.stride()[:3])
    os_ = (C.c_int64 * 3)(*out.stride()[:3])
    lib = _lib.load()
    st = lib.b200fa_rope(_DTYPE_CODE[x.dtype], B, H, N, D, rot, 1 if interleaved else 0, 1 if inverse else 0,
                         C.c_void_p(x.data_ptr()), xs, C.c_void_p(out.data_ptr()), os_, C.c_void_p(cos.data_ptr()),
                         C.c_void_p(sin.data_ptr()), cos.shape[0], None if offs_t is None else C.c_void_p(offs_t.data_ptr()),
                         offs_i, C.c_void_p(_stream_ptr(stream, x.device)))
    _lib.check(st, "apply_rope")
    return out


class _RopeFn(torch.autograd.Function):
    """The rotation is orthogonal: its backward is the transposed rotation of the incoming gradient."""

    @staticmethod
    def forward(ctx, x, cos, sin, offset, interleaved, rot, stream):
        ctx.save_for_backward(cos, sin)
        ctx.meta = (offset, interleaved, rot, stream)
        return _rope_raw(x, cos, sin, offset, interleaved, rot, False, stream)

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        offset, interleaved, rot, stream = ctx.meta
        g = g if g.stride(-1) == 1 and all(s % 8 == 0 for s in g.stride()[:3]) and g.data_ptr() % 16 == 0 else g.contiguous()
        return _rope_raw(g, cos, sin, offset, interleaved, rot, True, stream), None, None, None, None, None, None


def apply_rope(x, cos, sin, offset: Union[int, Sequence[int], torch.Tensor] = 0, interleaved: bool = True,
               rotary_dim: Optional[int] = None, stream=None) -> torch.Tensor:
    """Rotate ``x`` ``[B, H, N, D]`` (f16 / bf16) with tables ``cos`` / ``sin`` float32 ``[max_seq_len, rotary_dim/2]``;
    row n of batch b takes position ``offset[b] + n`` (one int for all batches, or one per batch).  Role of
    ``_apply_rope_mlx`` (mlx_mfa/attention.py:2128-2210).  Differentiable with respect to ``x``."""
    x, cos, sin = _as_tensor(x, "x"), _as_tensor(cos, "rotary_cos"), _as_tensor(sin, "rotary_sin")
    if x.ndim != 4:
        raise ValueError(f"apply_rope expects [B, H, N, D], got {x.ndim}D.")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise NotImplementedError("apply_rope takes f16 / bf16 tensors.")
    D = x.shape[-1]
    rot = D if rotary_dim is None else int(rotary_dim)
    if rot <= 0 or rot > D or rot % 2:
        raise ValueError(f"rotary_dim must be even and in (0, {D}], got {rot}.")
    if cos.ndim != 2 or cos.shape != sin.shape or cos.shape[1] != rot // 2:
        raise ValueError(f"rotary_cos / rotary_sin must both be [max_seq_len, {rot // 2}], got {tuple(cos.shape)} and {tuple(sin.shape)}.")
    _require_cuda(x, cos, sin)
    cos, sin = cos.to(torch.float32).contiguous(), sin.to(torch.float32).contiguous()
    N = x.shape[2]
    if isinstance(offset, torch.Tensor) and offset.ndim == 0:
        offset = int(offset)
    if not isinstance(offset, (int, torch.Tensor)):
        offset = [int(o) for o in offset]
        if len(offset) != x.shape[0]:
            raise ValueError(f"cache_seqlens length {len(offset)} must equal batch size B={x.shape[0]}")
        if offset and (min(offset) < 0 or max(offset) + N > cos.shape[0]):
            raise ValueError(f"positions up to {max(offset) + N} exceed the rotary table's {cos.shape[0]} rows.")
        offset = torch.tensor(offset, dtype=torch.int32)
    elif isinstance(offset, torch.Tensor):
        if int(offset.min()) < 0 or int(offset.max()) + N > cos.shape[0]:
            raise ValueError(f"positions exceed the rotary table's {cos.shape[0]} rows.")
    ok = x.stride(-1) == 1 and all(s % 8 == 0 for s in x.stride()[:3]) and x.data_ptr() % 16 == 0
    if not ok:
        x = x.contiguous()
    return _RopeFn.apply(x, cos, sin, offset, bool(interleaved), rot, stream)


def flash_attention_rope(q, k, v, rotary_cos=None, rotary_sin=None, scale: Optional[float] = None, causal: bool = False,
                         cache_seqlens: Union[int, Sequence[int], torch.Tensor] = 0, rope_3d: Optional[dict] = None,
                         interleaved: bool = True, rotary_dim: Optional[int] = None, stream=None) -> torch.Tensor:
    """Attention with rotary embeddings applied to Q (positions ``cache_seqlens + [0, N)``) and K (positions
    ``[0, S)``).  Signature and argument rules of mlx_mfa.flash_attention_rope (mlx_mfa/attention.py:419-555):
    1-D tables ``[max_seq_len, D/2]``, or ``rope_3d={'grid_h', 'grid_w', 'num_frames', ...}`` (tables built by
    :func:`make_rope_3d_tables`, positions start at 0); the two are mutually exclusive."""
    q, k, v = _as_tensor(q, "q"), _as_tensor(k, "k"), _as_tensor(v, "v")
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("flash_attention_rope expects 4-D tensors [batch, heads, seq, head_dim]."
                         f" Got q={q.ndim}D, k={k.ndim}D, v={v.ndim}D.")
    head_dim = q.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    if rope_3d is not None:
        if rotary_cos is not None or rotary_sin is not None:
            raise ValueError("rope_3d and rotary_cos/rotary_sin are mutually exclusive.")
        rotary_cos, rotary_sin = make_rope_3d_tables(
            rope_3d["grid_h"], rope_3d["grid_w"], rope_3d.get("num_frames", 1), d_h=rope_3d.get("d_h"),
            d_w=rope_3d.get("d_w"), d_t=rope_3d.get("d_t"), head_dim=head_dim, theta=rope_3d.get("theta", 10000.0),
            device=q.device)
        cache_seqlens = 0
    if rotary_cos is None or rotary_sin is None:
        raise ValueError("flash_attention_rope requires either rotary_cos/rotary_sin (1D) or rope_3d (3D) to be provided.")
    q_rot = apply_rope(q, rotary_cos, rotary_sin, cache_seqlens, interleaved, rotary_dim, stream)
    k_rot = apply_rope(k, rotary_cos, rotary_sin, 0, interleaved, rotary_dim, stream)
    return flash_attention(q_rot, k_rot, v, scale=scale, causal=causal, stream=stream)
