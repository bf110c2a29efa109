"""Operator front end: the ``mlx_mfa`` attention surface on B200.

Same function names, argument order, defaults and error behaviour as the
reference's ``mlx_mfa/attention.py`` for the attention hot path:

* ``flash_attention``          (mlx_mfa/attention.py:39-316)
* ``flash_attention_varlen``   (mlx_mfa/attention.py:2393-2523)
* ``flash_attention_kvcache``  (mlx_mfa/attention.py:903-1213)
* ``flash_attention_paged``    (mlx_mfa/attention.py:2819-3084)

Arrays are ``torch.Tensor`` on a CUDA device or any object exporting
``__dlpack__``; results are ``torch.Tensor``.  Every operator runs a hand-written
CUDA kernel through the C-ABI of ``libb200fa.so``; where the reference would
silently fall back to ``mx.fast.scaled_dot_product_attention`` this module
raises instead (no second backend, no CPU path).

Deliberate differences from the reference, all on the side of its CPU
(``backend="sdpa"``) semantics:

* causal masks are lower-right aligned per sequence everywhere (the reference's
  varlen kernel and backward are top-left aligned, equal when N == S);
* ``return_lse=True`` honours ``softcap`` and ``window_size`` (the reference
  drops them on that path, mlx_mfa/attention.py:308-314);
* the backward uses the lse saved by the forward instead of recomputing the
  forward (mlx_mfa/attention.py:2009).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence, Tuple, Union

import torch

from . import _lib

_SUPPORTED_HDIMS = (64, 128)
_FWD_ONLY_HDIMS = (256,)       # f16 / bf16 forward through the portable kernel; no backward, no decode kernel
_VALID_BACKENDS = {"auto", "mfa", "sdpa"}
_DTYPE_CODE = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}

__all__ = [
    "flash_attention",
    "flash_attention_varlen",
    "flash_attention_kvcache",
    "flash_attention_paged",
    "paged_kv_gather",
    "paged_kv_gather_dequant",
    "kernel_status",
    "is_mfa_available",
    "get_device_info",
    "get_supported_configs",
]


# ---------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------
def _as_tensor(x, name: str) -> torch.Tensor:
    """Accepts a torch tensor or any DLPack exporter."""
    if x is None:
        raise ValueError(f"{name} is None")
    if not isinstance(x, torch.Tensor):
        if hasattr(x, "__dlpack__"):
            x = torch.from_dlpack(x)
        else:
            raise TypeError(f"{name} must be a torch.Tensor or export __dlpack__, got {type(x)!r}")
    return x


def _require_cuda(*tensors) -> None:
    """Raised just before a launch: there is no CPU implementation to fall back to."""
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                f"tensor on {t.device}: this library only runs CUDA kernels on a B200 and has no CPU path."
            )


def _row_contig(x: torch.Tensor) -> torch.Tensor:
    """Makes the last dim contiguous and the strides / base 16-byte multiples,
    copying only when needed (the reference forces full contiguity,
    mlx_mfa/attention.py:2049-2053)."""
    eb = x.element_size()
    ok = x.stride(-1) == 1 and all((s * eb) % 16 == 0 for s in x.stride()[:-1]) and x.data_ptr() % 16 == 0
    return x if ok else x.contiguous()


def _stream_ptr(stream, device) -> int:
    if stream is None:
        return torch.cuda.current_stream(device).cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    if isinstance(stream, int):
        return stream
    raise TypeError("stream must be None, a torch.cuda.Stream or a raw cudaStream_t integer")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _desc(dtype, kv_dtype, B, Hq, Hkv, N, S, D, scale, causal, softcap=0.0, window_left=-1,
          num_splits=0, flags=0, q=None, k=None, v=None, o=None, alibi=None, bmask=None, kv_lens=None) -> _lib.Desc:
    d = _lib.Desc()
    d.dtype, d.kv_dtype = dtype, kv_dtype
    d.B, d.Hq, d.Hkv, d.N, d.S, d.D = B, Hq, Hkv, N, S, D
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("o_strides", o)):
        arr = getattr(d, name)
        if t is None:
            arr[0] = arr[1] = arr[2] = 0
        else:
            arr[0], arr[1], arr[2] = t.stride(0), t.stride(1), t.stride(2)
    d.scale = float(scale)
    d.softcap = float(softcap)
    d.causal = 1 if causal else 0
    d.window_left = int(window_left)
    d.num_splits = int(num_splits)
    d.flags = int(flags)
    d.alibi_slopes = None if alibi is None else alibi.data_ptr()
    d.kv_lens = None if kv_lens is None else kv_lens.data_ptr()
    if bmask is not None:            # (uint8 tensor [NQ, NK], block rows, block columns)
        d.block_mask = bmask[0].data_ptr()
        d.mask_bq, d.mask_bk, d.mask_nk = int(bmask[1]), int(bmask[2]), int(bmask[0].shape[1])
    return d


_FORCE_FLAGS = 0


def _set_force_flags(flags: int) -> int:
    """Test hook: ORs `flags` (e.g. FLAG_FORCE_MMA_SYNC) into every descriptor."""
    global _FORCE_FLAGS
    old, _FORCE_FLAGS = _FORCE_FLAGS, int(flags)
    return old


# ---------------------------------------------------------------------------
# raw operator calls (C-ABI)
# ---------------------------------------------------------------------------
def _fwd_raw(q, k, v, scale, causal, softcap, window_left, want_lse, stream, out=None, lse=None, alibi=None,
             bmask=None, kv_lens=None):
    """One forward launch.  `out` / `lse` may be caller-owned contiguous buffers (the host pipeline's staging slots).
    `kv_lens` (int32 [B] on the device): batch entry b sees its first kv_lens[b] keys only."""
    _require_cuda(q, k, v)
    lib = _lib.load()
    B, Hq, N, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    q, k, v = _row_contig(q), _row_contig(k), _row_contig(v)
    if Hkv > 1 and S > 0 and k.stride(1) == 0 and v.stride(1) == 0:
        # one kv head broadcast over the head axis (k.expand(...)): that is MQA, and the kernels read the single head
        k, v, Hkv = k[:, :1], v[:, :1], 1
    if out is None:
        out = torch.empty((B, Hq, N, D), dtype=q.dtype, device=q.device)
    if want_lse and lse is None:
        lse = torch.empty((B, Hq, N), dtype=torch.float32, device=q.device)
    if not want_lse:
        lse = None
    code = _DTYPE_CODE[q.dtype]
    d = _desc(code, code, B, Hq, Hkv, N, S, D, scale, causal, softcap, window_left,
              flags=_FORCE_FLAGS, q=q, k=k if S > 0 else None, v=v if S > 0 else None, o=out, alibi=alibi, bmask=bmask,
              kv_lens=kv_lens)
    with torch.cuda.device(q.device):
        # non-zero only for a few query rows against a long cache (N <= 4, S >= 256): the split-KV decode route
        need = lib.b200fa_fwd_workspace_bytes(C.byref(d))
        ws = torch.empty(need, dtype=torch.uint8, device=q.device) if need > 0 else None
        st = lib.b200fa_fwd(C.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), _ptr(ws), need,
                            C.c_void_p(_stream_ptr(stream, q.device)))
    _lib.check(st, "flash_attention")
    return out, lse


def _bwd_raw(q, k, v, out, lse, dout, scale, causal, stream, cu=None, alibi=None, bmask=None, softcap=0.0,
             window_left=-1):
    _require_cuda(q, k, v, out, lse, dout)
    lib = _lib.load()
    B, Hq, N, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    q, k, v = _row_contig(q), _row_contig(k), _row_contig(v)
    out = out.contiguous()
    dout = dout.contiguous()
    dq = torch.empty((B, Hq, N, D), dtype=q.dtype, device=q.device)
    dk = torch.empty((B, Hkv, S, D), dtype=q.dtype, device=q.device)
    dv = torch.empty((B, Hkv, S, D), dtype=q.dtype, device=q.device)
    code = _DTYPE_CODE[q.dtype]
    d = _desc(code, code, B, Hq, Hkv, N, S, D, scale, causal, softcap, window_left, flags=_FORCE_FLAGS, q=q, k=k, v=v,
              o=out, alibi=alibi, bmask=bmask)
    sp = C.c_void_p(_stream_ptr(stream, q.device))
    with torch.cuda.device(q.device):
        if cu is None:
            need = lib.b200fa_bwd_workspace_bytes(C.byref(d))
            ws = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
            st = lib.b200fa_bwd(C.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), _ptr(dout),
                                _ptr(dq), _ptr(dk), _ptr(dv), _ptr(ws), ws.numel(), sp)
        else:
            cu_q, cu_k, nseq, max_q, max_k = cu
            need = lib.b200fa_bwd_varlen_workspace_bytes(C.byref(d), nseq, max_q, max_k)
            ws = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
            st = lib.b200fa_bwd_varlen(C.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse),
                                       _ptr(dout), _ptr(cu_q), _ptr(cu_k), nseq, max_q, max_k,
                                       _ptr(dq), _ptr(dk), _ptr(dv), _ptr(ws), ws.numel(), sp)
    _lib.check(st, "flash_attention backward")
    return dq, dk, dv


class _FlashAttnFn(torch.autograd.Function):
    """Autograd glue; role of _make_mfa_custom (mlx_mfa/attention.py:1931-2030)."""

    @staticmethod
    def forward(ctx, q, k, v, scale, causal, softcap, window_left, want_lse, stream, alibi=None, bmask=None):
        need_grad = q.requires_grad or k.requires_grad or v.requires_grad
        out, lse = _fwd_raw(q, k, v, scale, causal, softcap, window_left, want_lse or need_grad, stream, alibi=alibi,
                            bmask=bmask)
        ctx.bmask = bmask
        ctx.save_for_backward(q, k, v, out, lse if lse is not None else torch.empty(0, device=q.device))
        ctx.cfg = (scale, causal, softcap, window_left, stream)
        ctx.alibi = alibi          # a constant of the graph: the slopes get no gradient (mlx_mfa/attention.py:1909)
        if want_lse:
            ctx.mark_non_differentiable(lse)
            return out, lse
        return out, None

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, v, out, lse = ctx.saved_tensors
        scale, causal, softcap, window_left, stream = ctx.cfg
        if q.shape[-1] in _FWD_ONLY_HDIMS:
            raise NotImplementedError(f"flash_attention backward for head_dim {q.shape[-1]} is not built.")
        if q.dtype == torch.float32:
            raise NotImplementedError(
                "flash_attention backward for float32: the reference differentiates its SDPA fallback "
                "(mlx_mfa/attention.py:2013-2019); the CUDA backward takes f16/bf16."
            )
        # softcap and window_size are differentiated by the kernels (the reference routes them through its SDPA
        # fallback's autodiff, mlx_mfa/attention.py:1976-1992, 2020-2027)
        dq, dk, dv = _bwd_raw(q, k, v, out, lse, dout, scale, causal, stream, alibi=ctx.alibi, bmask=ctx.bmask,
                              softcap=softcap, window_left=window_left)
        return dq, dk, dv, None, None, None, None, None, None, None, None


# ---------------------------------------------------------------------------
# flash_attention
# ---------------------------------------------------------------------------
def flash_attention(
    q,
    k,
    v,
    scale: Optional[float] = None,
    causal: bool = False,
    softcap: float = 0.0,
    alibi_slopes=None,
    dropout_p: float = 0.0,
    return_attn_weights: bool = False,
    window_size: Optional[Tuple[int, int]] = None,
    return_lse: bool = False,
    stream=None,
    attn_bias=None,
    backend: str = "auto",
):
    """Scaled dot-product attention, ``softmax(scale * q k^T + mask) v``.

    Args follow mlx_mfa.flash_attention (mlx_mfa/attention.py:39-54):
    q ``[B, Hq, N, D]``; k, v ``[B, Hkv, S, D]`` with ``Hq % Hkv == 0`` (GQA/MQA);
    ``scale`` defaults to ``1/sqrt(D)``; ``causal`` masks key ``j > i + (S - N)``;
    ``softcap`` applies ``cap * tanh(s / cap)`` before masking;
    ``window_size=(left, right)`` keeps keys ``j >= i + (S - N) - left``; ``right``
    must be -1 or 0 (no right bound, mlx_mfa/attention.py:282-288);
    ``return_lse=True`` returns ``(O, L)``, ``L`` float32 ``[B, Hq, N]`` in base 2.

    Raises ValueError / NotImplementedError / RuntimeError at the conditions the
    reference does; options the reference serves only through its SDPA fallback
    (``alibi_slopes``, ``dropout_p``, ``return_attn_weights``, ``attn_bias``,
    ``backend="sdpa"``, ``D_v != D_qk``) raise NotImplementedError.
    """
    if backend not in _VALID_BACKENDS:
        raise ValueError(
            f"flash_attention: backend must be one of {sorted(_VALID_BACKENDS)}, got {backend!r}."
        )
    if backend == "sdpa":
        raise NotImplementedError(
            "flash_attention(backend='sdpa'): the SDPA fallback of the reference "
            "(mlx_mfa/attention.py:169-180) is not part of this library; it has no CPU path."
        )
    q, k, v = _as_tensor(q, "q"), _as_tensor(k, "k"), _as_tensor(v, "v")
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError(
            f"flash_attention expects 4-D tensors [batch, heads, seq, head_dim]."
            f" Got q={q.ndim}D, k={k.ndim}D, v={v.ndim}D."
        )
    q_dim, k_dim, v_dim = q.shape[-1], k.shape[-1], v.shape[-1]
    if k_dim != q_dim:
        raise ValueError(f"q and k must have the same head_dim. Got q_dim={q_dim}, k_dim={k_dim}.")
    head_dim = q_dim
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    q_heads, kv_heads = q.shape[1], k.shape[1]
    if kv_heads != q_heads and q_heads % kv_heads != 0:
        raise ValueError(
            f"flash_attention GQA: q_heads ({q_heads}) must be divisible by kv_heads ({kv_heads})."
        )
    if k.shape[0] != q.shape[0] or v.shape[:3] != k.shape[:3]:
        raise ValueError(f"flash_attention: inconsistent shapes q={tuple(q.shape)} k={tuple(k.shape)} v={tuple(v.shape)}.")
    if return_attn_weights:
        if return_lse:
            raise ValueError("return_attn_weights and return_lse are mutually exclusive.")
        raise NotImplementedError("return_attn_weights needs the reference's SDPA fallback; not built.")
    if dropout_p > 0.0:
        raise NotImplementedError("dropout_p > 0 needs the reference's SDPA fallback; not built.")
    if attn_bias is not None:
        raise NotImplementedError("attn_bias needs the reference's SDPA fallback; not built.")
    alibi = None
    if alibi_slopes is not None:
        # per-head linear position bias slope[h] * (j - i) (mlx_mfa/attention.py:77-81, 1774-1822); float32 [Hq]
        alibi = _as_tensor(alibi_slopes, "alibi_slopes")
        if alibi.ndim != 1 or alibi.shape[0] != q_heads:
            raise ValueError(f"alibi_slopes must be [H_q] = [{q_heads}], got {tuple(alibi.shape)}.")
        _require_cuda(alibi)
        alibi = alibi.to(torch.float32).contiguous()
    supported = ((head_dim in _SUPPORTED_HDIMS and q.dtype in _DTYPE_CODE) or
                 (head_dim in _FWD_ONLY_HDIMS and q.dtype in (torch.float16, torch.bfloat16))) and v_dim == q_dim
    if not supported:
        msg = (
            f"unsupported configuration — head_dim={head_dim}, dtype={q.dtype}, "
            f"v_dim_mismatch={v_dim != q_dim}. Supported: head_dim∈{{64,128}} with f16/bf16/f32, head_dim=256 with f16/bf16 (forward only)."
        )
        if backend == "mfa":
            raise RuntimeError(f"flash_attention(backend='mfa'): {msg}")
        raise NotImplementedError(f"flash_attention: {msg}")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError(f"flash_attention: q, k, v must share a dtype, got {q.dtype}, {k.dtype}, {v.dtype}.")

    window_left = -1
    if window_size is not None:
        wr = window_size[1] if len(window_size) > 1 else -1
        if wr > 0:
            raise NotImplementedError(
                f"flash_attention: window_size right={wr} is not yet supported. "
                "The STEEL kernel only implements left-side sliding-window masking. "
                "Use causal=True to mask all future tokens, or set right=-1."
            )
        window_left = max(int(window_size[0]), 0)

    out, lse = _FlashAttnFn.apply(q, k, v, float(scale), bool(causal), float(softcap), window_left,
                                  bool(return_lse), stream, alibi)
    if return_lse:
        return out, lse
    return out


# ---------------------------------------------------------------------------
# flash_attention_varlen
# ---------------------------------------------------------------------------
def _varlen_fwd_raw(q, k, v, cu_q, cu_k, nseq, max_q, max_k, scale, causal, want_lse, stream):
    _require_cuda(q, k, v, cu_q, cu_k)
    lib = _lib.load()
    _, Hq, Tq, D = q.shape
    Hkv, Tk = k.shape[1], k.shape[2]
    q, k, v = _row_contig(q), _row_contig(k), _row_contig(v)
    out = torch.zeros((1, Hq, Tq, D), dtype=q.dtype, device=q.device)
    lse = torch.zeros((1, Hq, Tq), dtype=torch.float32, device=q.device) if want_lse else None
    code = _DTYPE_CODE[q.dtype]
    d = _desc(code, code, 1, Hq, Hkv, Tq, Tk, D, scale, causal, flags=_FORCE_FLAGS, q=q, k=k, v=v, o=out)
    with torch.cuda.device(q.device):
        st = lib.b200fa_fwd_varlen(C.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(cu_q), _ptr(cu_k), nseq,
                                   max_q, max_k, _ptr(out), _ptr(lse), None, 0,
                                   C.c_void_p(_stream_ptr(stream, q.device)))
    _lib.check(st, "flash_attention_varlen")
    return out, lse


class _VarlenFn(torch.autograd.Function):
    """One forward launch and one backward launch sequence for all packed
    sequences; replaces _varlen_impl/_varlen_bwd (mlx_mfa/attention.py:2463-2521)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, nseq, max_q, max_k, scale, causal, stream):
        need_grad = q.requires_grad or k.requires_grad or v.requires_grad
        out, lse = _varlen_fwd_raw(q, k, v, cu_q, cu_k, nseq, max_q, max_k, scale, causal, need_grad, stream)
        ctx.save_for_backward(q, k, v, out, lse if lse is not None else torch.empty(0, device=q.device), cu_q, cu_k)
        ctx.cfg = (nseq, max_q, max_k, scale, causal, stream)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        nseq, max_q, max_k, scale, causal, stream = ctx.cfg
        if q.dtype == torch.float32:
            raise NotImplementedError("flash_attention_varlen backward takes f16/bf16.")
        dq, dk, dv = _bwd_raw(q, k, v, out, lse, dout, scale, causal, stream,
                              cu=(cu_q, cu_k, nseq, max_q, max_k))
        return dq, dk, dv, None, None, None, None, None, None, None, None


def flash_attention_varlen(
    q,
    k,
    v,
    cu_seqlens_q,
    cu_seqlens_k,
    max_seqlen_q: int,
    max_seqlen_k: int,
    scale: Optional[float] = None,
    causal: bool = False,
    block_mask=None,
    stream=None,
):
    """Attention over sequences packed along the token axis.

    Signature of mlx_mfa.flash_attention_varlen (mlx_mfa/attention.py:2393-2405):
    q, k, v ``[1, H, total_tokens, D]``; ``cu_seqlens_*`` int32 ``[num_seqs + 1]``
    cumulative lengths; sequences attend only to themselves; ``causal`` is applied
    per sequence.  Returns ``[1, H, total_q, D]``.  ``num_seqs == 0`` returns ``q``
    (mlx_mfa/attention.py:2444-2445).  ``block_mask`` (one block mask valid for every sequence) goes through a
    per-sequence split, as in the reference.
    """
    q, k, v = _as_tensor(q, "q"), _as_tensor(k, "k"), _as_tensor(v, "v")
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("flash_attention_varlen expects 4-D tensors [1, H, total_tokens, D].")
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    cu_q = _as_tensor(cu_seqlens_q, "cu_seqlens_q")
    cu_k = _as_tensor(cu_seqlens_k, "cu_seqlens_k")
    nseq = cu_q.numel() - 1
    if nseq <= 0:
        return q
    if q.shape[0] != 1 or k.shape[0] != 1 or v.shape[0] != 1:
        raise ValueError("flash_attention_varlen expects packed tensors with batch size 1.")
    if cu_k.numel() != cu_q.numel():
        raise ValueError("cu_seqlens_q and cu_seqlens_k must have the same length.")
    if block_mask is not None:
        # The mask has to fit every sequence by itself, so the reference takes it through a per-sequence split and
        # concatenation of flash_attention_sparse calls (mlx_mfa/attention.py:2365-2390, 2448-2453); so does this.
        from .sparse import flash_attention_sparse

        cq, ck = [int(x) for x in cu_q.tolist()], [int(x) for x in cu_k.tolist()]
        outs = [flash_attention_sparse(q[:, :, cq[i]:cq[i + 1]], k[:, :, ck[i]:ck[i + 1]], v[:, :, ck[i]:ck[i + 1]],
                                       block_mask, scale=scale, causal=causal, stream=stream) for i in range(nseq)]
        return torch.cat(outs, dim=2)
    D = q.shape[-1]
    if k.shape[-1] != D or v.shape[-1] != D:
        raise ValueError("q, k, v must have the same head_dim.")
    if q.shape[1] % k.shape[1] != 0:
        raise ValueError(f"flash_attention GQA: q_heads ({q.shape[1]}) must be divisible by kv_heads ({k.shape[1]}).")
    ok = (D in _SUPPORTED_HDIMS and q.dtype in _DTYPE_CODE) or (D in _FWD_ONLY_HDIMS and q.dtype in (torch.float16, torch.bfloat16))
    if not ok:
        raise NotImplementedError(f"flash_attention_varlen: head_dim={D}, dtype={q.dtype} not built.")
    cu_q = cu_q.to(torch.int32).contiguous()
    cu_k = cu_k.to(torch.int32).contiguous()
    return _VarlenFn.apply(q, k, v, cu_q, cu_k, int(nseq), int(max_seqlen_q), int(max_seqlen_k),
                           float(scale), bool(causal), stream)


# ---------------------------------------------------------------------------
# paged KV
# ---------------------------------------------------------------------------
def paged_kv_gather(pool, block_table, seq_lens, max_kv_len: int, stream=None) -> torch.Tensor:
    """``pool [num_pages, block_size, H, D]`` -> ``[B, H, max_kv_len, D]``, zero
    beyond ``seq_lens[b]`` and for ``-1`` table entries.  Bit-exact copy; same
    contract as ``_ext.mfa_paged_kv_gather`` (csrc/bindings.cpp:346-364)."""
    pool = _as_tensor(pool, "pool").contiguous()
    table = _as_tensor(block_table, "block_table").to(torch.int32).contiguous()
    lens = _as_tensor(seq_lens, "seq_lens").to(torch.int32).contiguous()
    if pool.ndim != 4 or table.ndim != 2 or lens.ndim != 1:
        raise ValueError("paged_kv_gather: pool must be 4-D, block_table 2-D, seq_lens 1-D.")
    _require_cuda(pool, table, lens)
    lib = _lib.load()
    _, bs, H, D = pool.shape
    B, max_blocks = table.shape
    out = torch.empty((B, H, max_kv_len, D), dtype=pool.dtype, device=pool.device)
    with torch.cuda.device(pool.device):
        st = lib.b200fa_paged_kv_gather(_ptr(pool), _ptr(table), _ptr(lens), B, H, D, pool.element_size(),
                                        bs, max_blocks, int(max_kv_len), _ptr(out),
                                        C.c_void_p(_stream_ptr(stream, pool.device)))
    _lib.check(st, "paged_kv_gather")
    return out


class _PagedGatherFn(torch.autograd.Function):
    """paged_kv_gather with a backward: the dense gradient is added back into a pool-shaped tensor page by page
    (the role of _gather_contig / _scatter_to_pool in the reference's paged vjp, mlx_mfa/attention.py:2878-2989)."""

    @staticmethod
    def forward(ctx, pool, table, lens, max_kv_len, stream):
        ctx.save_for_backward(table, lens)
        ctx.meta = (tuple(pool.shape), pool.dtype, max_kv_len, stream)
        return paged_kv_gather(pool, table, lens, max_kv_len, stream)

    @staticmethod
    def backward(ctx, g):
        table, lens = ctx.saved_tensors
        shape, dtype, max_kv_len, stream = ctx.meta
        if dtype not in (torch.float16, torch.bfloat16):
            raise NotImplementedError("backward through a page pool takes f16 / bf16 pools.")
        g = g.to(dtype).contiguous()
        grad_pool = torch.zeros(shape, dtype=dtype, device=g.device)
        B, H, _, D = g.shape
        lib = _lib.load()
        with torch.cuda.device(g.device):
            st = lib.b200fa_paged_kv_scatter_add(_ptr(g), _ptr(table), _ptr(lens), B, H, D, _DTYPE_CODE[dtype], shape[1],
                                                 table.shape[1], int(max_kv_len), _ptr(grad_pool),
                                                 C.c_void_p(_stream_ptr(stream, g.device)))
        _lib.check(st, "paged_kv_scatter_add")
        return grad_pool, None, None, None, None


def _fwd_paged_raw(q, k_pages, v_pages, table, lens, max_kv_len, scale, causal, softcap, window_left, want_lse, stream):
    """Forward over a 16-bit page pool for prefill-sized queries: K / V are read through the block table."""
    _require_cuda(q, k_pages, v_pages, table, lens)
    lib = _lib.load()
    B, Hq, N, D = q.shape
    num_pages, block_size, Hkv, _ = k_pages.shape
    q = _row_contig(q)
    out = torch.empty((B, Hq, N, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, N), dtype=torch.float32, device=q.device) if want_lse else None
    code = _DTYPE_CODE[q.dtype]
    d = _desc(code, code, B, Hq, Hkv, N, int(max_kv_len), D, scale, causal, softcap, window_left, flags=_FORCE_FLAGS, q=q, o=out)
    with torch.cuda.device(q.device):
        st = lib.b200fa_fwd_paged(C.byref(d), _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), _ptr(lens), num_pages,
                                  block_size, table.shape[1], int(max_kv_len), _ptr(out), _ptr(lse),
                                  C.c_void_p(_stream_ptr(stream, q.device)))
    _lib.check(st, "flash_attention_paged")
    return out, lse


def paged_kv_gather_dequant(pool, scale, block_table, seq_lens, max_kv_len: int, out_dtype, stream=None) -> torch.Tensor:
    """int8 / float8_e4m3 ``pool [num_pages, block_size, H, D]`` with float16 ``scale [num_pages, block_size, H]`` ->
    ``out_dtype [B, H, max_kv_len, D]``: the page gather and the dense-dequant step of
    mlx_mfa/integrations/mlx_lm.py:97-110 (``mx.dequantize(..., dtype=q.dtype)``) in one pass; zeros beyond
    ``seq_lens[b]`` and for ``-1`` table entries."""
    pool = _as_tensor(pool, "pool").contiguous()
    scale = _as_tensor(scale, "scale").to(torch.float16).contiguous()
    table = _as_tensor(block_table, "block_table").to(torch.int32).contiguous()
    lens = _as_tensor(seq_lens, "seq_lens").to(torch.int32).contiguous()
    if pool.dtype not in _KV_CODE:
        raise ValueError(f"paged_kv_gather_dequant: pool dtype {pool.dtype} is not an 8-bit KV type.")
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("paged_kv_gather_dequant: out_dtype must be float16 or bfloat16.")
    _require_cuda(pool, scale, table, lens)
    lib = _lib.load()
    _, bs, H, D = pool.shape
    B, max_blocks = table.shape
    out = torch.empty((B, H, max_kv_len, D), dtype=out_dtype, device=pool.device)
    with torch.cuda.device(pool.device):
        st = lib.b200fa_paged_kv_gather_dequant(_ptr(pool), _ptr(scale), _ptr(table), _ptr(lens), B, H, D,
                                                _KV_CODE[pool.dtype], _DTYPE_CODE[out_dtype], bs, max_blocks,
                                                int(max_kv_len), _ptr(out), C.c_void_p(_stream_ptr(stream, pool.device)))
    _lib.check(st, "paged_kv_gather_dequant")
    return out


_CHECK_DECODE_STATUS = False   # tests switch this on: one stream sync per call


def _set_check_decode_status(on: bool) -> bool:
    """Debug hook: after each decode launch, wait for it and raise if the kernel set its error word."""
    global _CHECK_DECODE_STATUS
    old, _CHECK_DECODE_STATUS = _CHECK_DECODE_STATUS, bool(on)
    return old


_KV_CODE = {torch.int8: _lib.I8}
if hasattr(torch, "float8_e4m3fn"):
    _KV_CODE[torch.float8_e4m3fn] = _lib.E4M3


def _decode_raw(q, k_pages, v_pages, k_scale, v_scale, table, lens, max_kv_len, scale, causal, softcap,
                block_size, want_lse, stream, num_splits=0, workspace=None, packed=False):
    """One decode launch.  packed=True returns (float32 [B*Hq*Nq, D+4], None): each row is the normalised output in
    fp32 with its base-2 lse at column D -- the per-GPU partial that `parallel.combine_packed` merges."""
    _require_cuda(q, k_pages, v_pages, k_scale, v_scale, table, lens)
    lib = _lib.load()
    B, Hq, Nq, D = q.shape
    num_pages, _, Hkv, _ = k_pages.shape
    q = q.contiguous()
    if packed:
        out = torch.empty((B * Hq * Nq, D + 4), dtype=torch.float32, device=q.device)
        lse = None
    else:
        out = torch.empty((B, Hq, Nq, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, Hq, Nq), dtype=torch.float32, device=q.device) if want_lse else None
    code = _DTYPE_CODE[q.dtype]
    kv_code = _KV_CODE.get(k_pages.dtype, _DTYPE_CODE.get(k_pages.dtype, -1))
    d = _desc(code, kv_code, B, Hq, Hkv, Nq, 0, D, scale, causal, softcap, -1, num_splits,
              _FORCE_FLAGS | (_lib.FLAG_PACKED_F32 if packed else 0))
    with torch.cuda.device(q.device):
        need = lib.b200fa_decode_paged_workspace_bytes(C.byref(d), int(max_kv_len))
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
        st = lib.b200fa_decode_paged(C.byref(d), _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(k_scale),
                                     _ptr(v_scale), _ptr(table), _ptr(lens), num_pages, block_size,
                                     table.shape[1], int(max_kv_len), _ptr(out), _ptr(lse),
                                     _ptr(workspace), workspace.numel(),
                                     C.c_void_p(_stream_ptr(stream, q.device)))
    _lib.check(st, "flash_attention_paged")
    if _CHECK_DECODE_STATUS:
        word = C.c_int32(0)
        _lib.check(lib.b200fa_workspace_status(_ptr(workspace), C.c_void_p(_stream_ptr(stream, q.device)),
                                               C.byref(word)), "decode status")
        if word.value != 0:
            raise RuntimeError(f"flash_attention_paged: decode kernel reported status {word.value} "
                               "(1 = a bounded wait gave up, 2 = block_table entry beyond the pool)")
    return out, lse


def flash_attention_paged(
    q,
    k_pages,
    v_pages,
    block_table,
    seq_lens,
    *,
    scale: Optional[float] = None,
    causal: bool = False,
    block_size: int = 16,
    stream=None,
    k_scale=None,
    v_scale=None,
    softcap: float = 0.0,
    max_kv_len: Optional[int] = None,
    return_lse: bool = False,
    num_splits: int = 0,
):
    """Attention over a paged KV pool.

    Signature of mlx_mfa.flash_attention_paged (mlx_mfa/attention.py:2819-2830) plus
    keyword-only extensions.  q ``[B, Hq, Nq, D]``; ``k_pages``/``v_pages``
    ``[num_pages, block_size, Hkv, D]``; ``block_table`` int32 ``[B, max_blocks]``
    (-1 pads); ``seq_lens`` int32 ``[B]``.  Each sequence sees exactly its first
    ``seq_lens[b]`` tokens; ``causal`` is lower-right aligned per sequence.

    Extensions: ``k_scale``/``v_scale`` float16 ``[num_pages, block_size, Hkv]`` for
    int8 / float8_e4m3 pools (a stored x stands for ``float(x) * scale``, rounded to
    the query dtype as ``mx.dequantize(..., dtype=q.dtype)`` does in
    mlx_mfa/integrations/mlx_lm.py:97-110); ``max_kv_len`` skips the host read of
    ``seq_lens`` that the reference also performs (mlx_mfa/attention.py:2871-2873);
    ``num_splits`` caps how many CTAs share the page list (0 = one per SM).

    Short queries ((Hq/Hkv)*Nq <= 8; D = 128, or D = 64 with 16-bit pools; block_size a multiple
    of 16) run the split-KV decode kernel with in-kernel combine; other shapes gather pages and attend
    per sequence like the reference (mlx_mfa/attention.py:2944-2989).  When gradients are
    wanted (q or a 16-bit pool requires grad) every shape takes the gather route, whose
    backward adds dK / dV back into pool-shaped gradients page by page (2878-2940, 3020-3084).
    """
    q = _as_tensor(q, "q")
    k_pages, v_pages = _as_tensor(k_pages, "k_pages"), _as_tensor(v_pages, "v_pages")
    table = _as_tensor(block_table, "block_table")
    lens = _as_tensor(seq_lens, "seq_lens")
    if q.ndim != 4 or k_pages.ndim != 4 or v_pages.ndim != 4:
        raise ValueError("flash_attention_paged expects q [B,Hq,Nq,D] and pools [num_pages,block_size,Hkv,D].")
    B, Hq, Nq, D = q.shape
    Hkv = k_pages.shape[2]
    if k_pages.shape[1] != block_size or k_pages.shape[3] != D or v_pages.shape != k_pages.shape:
        raise ValueError("flash_attention_paged: pool shape does not match block_size / head_dim.")
    if Hq % Hkv != 0:
        raise ValueError(f"flash_attention GQA: q_heads ({Hq}) must be divisible by kv_heads ({Hkv}).")
    if table.ndim != 2 or table.shape[0] != B or lens.ndim != 1 or lens.shape[0] != B:
        raise ValueError("flash_attention_paged: block_table must be [B, max_blocks] and seq_lens [B].")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    table = table.to(torch.int32).contiguous()
    lens = lens.to(torch.int32).contiguous()
    if max_kv_len is None:
        max_kv_len = int(lens.max().item()) if B > 0 else 0
    if max_kv_len == 0:
        z = torch.zeros((B, Hq, Nq, D), dtype=q.dtype, device=q.device)
        if return_lse:
            return z, torch.full((B, Hq, Nq), float("-inf"), dtype=torch.float32, device=q.device)
        return z
    quant = k_pages.dtype in _KV_CODE
    if quant:
        if k_scale is None or v_scale is None:
            raise ValueError("flash_attention_paged: int8/fp8 pools need k_scale and v_scale.")
        k_scale = _as_tensor(k_scale, "k_scale").to(torch.float16).contiguous()
        v_scale = _as_tensor(v_scale, "v_scale").to(torch.float16).contiguous()
        if tuple(k_scale.shape) != tuple(k_pages.shape[:3]) or tuple(v_scale.shape) != tuple(v_pages.shape[:3]):
            raise ValueError("flash_attention_paged: scales must be [num_pages, block_size, Hkv].")
    elif k_pages.dtype != q.dtype:
        raise ValueError(f"flash_attention_paged: pool dtype {k_pages.dtype} must equal q dtype or be int8/fp8.")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise NotImplementedError("flash_attention_paged takes f16/bf16 queries.")
    k_pages, v_pages = k_pages.contiguous(), v_pages.contiguous()

    # training: gradients flow through the gather route (gather, per-sequence attention, scatter-add into the pools)
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k_pages.requires_grad or v_pages.requires_grad)
    decode_ok = ((Hq // Hkv) * Nq <= 8 and (D == 128 or (D == 64 and not quant)) and block_size % 16 == 0
                 and not needs_grad)
    if decode_ok:
        out, lse = _decode_raw(q, k_pages, v_pages, k_scale, v_scale, table, lens, max_kv_len, float(scale),
                               bool(causal), float(softcap), block_size, return_lse, stream, num_splits)
        return (out, lse) if return_lse else out
    if not needs_grad and D in _SUPPORTED_HDIMS:
        # Prefill-sized queries (chunked prefill over the pool), one launch for all sequences.  16-bit pools: the
        # forward kernel walks the block table itself.  8-bit pools: pages are gathered and dequantised to the query
        # dtype in one pass (the reference's dense-dequant path), then the dense kernel runs with per-sequence key
        # counts -- where the reference slices and launches per sequence (mlx_mfa/attention.py:2950-2989).
        if quant:
            K = paged_kv_gather_dequant(k_pages, k_scale, table, lens, int(max_kv_len), q.dtype, stream)
            V = paged_kv_gather_dequant(v_pages, v_scale, table, lens, int(max_kv_len), q.dtype, stream)
            out, lse = _fwd_raw(q, K, V, float(scale), bool(causal), float(softcap), -1, return_lse, stream, kv_lens=lens)
        else:
            out, lse = _fwd_paged_raw(q, k_pages, v_pages, table, lens, max_kv_len, float(scale), bool(causal),
                                      float(softcap), -1, return_lse, stream)
        return (out, lse) if return_lse else out
    if quant:
        raise NotImplementedError("quantized pools take f16 / bf16 queries at head_dim 64 or 128 and carry no gradient.")
    if return_lse:
        raise NotImplementedError("return_lse on the training (gather) route is not built.")
    # gather route, as the reference: pages -> contiguous, then exact-length slices per sequence
    if needs_grad:
        _require_cuda(q, k_pages, v_pages, table, lens)
        K = _PagedGatherFn.apply(k_pages, table, lens, int(max_kv_len), stream)
        V = _PagedGatherFn.apply(v_pages, table, lens, int(max_kv_len), stream)
    else:
        K = paged_kv_gather(k_pages, table, lens, max_kv_len, stream)
        V = paged_kv_gather(v_pages, table, lens, max_kv_len, stream)
    lens_host = [int(x) for x in lens.tolist()]
    outs = []
    for b in range(B):
        n = lens_host[b]
        if n == 0:
            outs.append(torch.zeros((1, Hq, Nq, D), dtype=q.dtype, device=q.device))
            continue
        outs.append(flash_attention(q[b:b + 1], K[b:b + 1, :, :n], V[b:b + 1, :, :n], scale=scale,
                                    causal=causal, softcap=softcap, stream=stream))
    return torch.cat(outs, dim=0)


def _first_offset(cache_seqlens) -> int:
    """cache_seqlens as one int: the value itself, or the first entry of an array / list (what the reference's
    append and paged routes do, mlx_mfa/attention.py:1077-1082, 1153-1158)."""
    if isinstance(cache_seqlens, torch.Tensor):
        return int(cache_seqlens.reshape(-1)[0])
    if isinstance(cache_seqlens, int):
        return cache_seqlens
    return int(list(cache_seqlens)[0]) if hasattr(cache_seqlens, "__iter__") else int(cache_seqlens)


def flash_attention_kvcache(
    q,
    k_cache,
    v_cache,
    *,
    k_new=None,
    v_new=None,
    block_table=None,
    seq_lens=None,
    block_size: int = 16,
    scale: Optional[float] = None,
    causal: bool = True,
    softcap: float = 0.0,
    alibi_slopes=None,
    window_size: Optional[Tuple[int, int]] = None,
    rotary_cos=None,
    rotary_sin=None,
    cache_seqlens: Union[int, Sequence[int]] = 0,
    interleaved: bool = True,
    rotary_dim: Optional[int] = None,
    cache_batch_idx=None,
    stream=None,
    k_scale=None,
    v_scale=None,
):
    """Attention against a KV cache, dense or paged.

    Signature of mlx_mfa.flash_attention_kvcache (mlx_mfa/attention.py:903-931) plus
    keyword-only ``k_scale``/``v_scale`` for quantized page pools.  Paged mode
    (``block_table`` given) requires ``seq_lens`` and rejects ``window_size`` and
    ``alibi_slopes`` with ValueError, as the reference does
    (mlx_mfa/attention.py:1124-1167).  Dense mode takes caches ``[B, Hkv, S, D]``
    (or a pool indexed by ``cache_batch_idx``).  Append mode (``k_new``/``v_new``, dense only)
    returns ``(out, k_updated, v_updated)`` as the reference does (mlx_mfa/attention.py:1059-1119);
    paged pools are written through ``PagedKVCache.append``.  ``rotary_cos`` / ``rotary_sin`` rotate q at
    ``cache_seqlens`` (and k_new in append mode, the dense cache's keys at ``[0, S)`` in dense mode; a paged pool
    holds rotated keys already).
    """
    q = _as_tensor(q, "q")
    if q.ndim != 4:
        raise ValueError(f"flash_attention_kvcache: q must be 4-D [B, H, N, D], got {q.ndim}D.")
    D = q.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    has_rope = (rotary_cos is not None) or (rotary_sin is not None)
    if has_rope and alibi_slopes is not None:
        raise ValueError("flash_attention_kvcache: rotary_cos/sin and alibi_slopes are mutually exclusive.")
    if k_new is not None or v_new is not None:
        if k_new is None or v_new is None:
            raise ValueError("flash_attention_kvcache: k_new and v_new must both be provided or both be None.")
        if block_table is not None:
            raise ValueError(
                "flash_attention_kvcache: k_new/v_new append is not supported in paged mode.  "
                "Manage the page pool externally and call without k_new."
            )
        if cache_batch_idx is not None:
            raise ValueError(
                "flash_attention_kvcache: k_new/v_new append is not supported together with "
                "cache_batch_idx (continuous-batching pool mode)."
            )
        # Append to the dense cache (or start one from k_new / v_new alone), then attend on the updated cache
        # and hand it back: (out, k_updated, v_updated), mlx_mfa/attention.py:1102-1119.  With rotary tables q and
        # k_new are both rotated at position cache_seqlens first; the cache holds rotated keys (1084-1100).
        k_new, v_new = _as_tensor(k_new, "k_new"), _as_tensor(v_new, "v_new")
        if has_rope:
            if rotary_cos is None or rotary_sin is None:
                raise ValueError("flash_attention_kvcache: both rotary_cos and rotary_sin must be provided together.")
            from .rope import apply_rope

            cs = _first_offset(cache_seqlens)
            q = apply_rope(q, rotary_cos, rotary_sin, cs, interleaved, rotary_dim, stream)
            k_new = apply_rope(k_new, rotary_cos, rotary_sin, cs, interleaved, rotary_dim, stream)
        if k_cache is not None:
            k_cache, v_cache = _as_tensor(k_cache, "k_cache"), _as_tensor(v_cache, "v_cache")
            k_updated = torch.cat([k_cache, k_new.to(k_cache.dtype)], dim=2)
            v_updated = torch.cat([v_cache, v_new.to(v_cache.dtype)], dim=2)
        else:
            k_updated, v_updated = k_new, v_new
        out = flash_attention(q, k_updated, v_updated, scale=scale, causal=causal, softcap=softcap,
                              alibi_slopes=alibi_slopes, window_size=window_size, stream=stream)
        return out, k_updated, v_updated
    if block_table is not None:
        if seq_lens is None:
            raise ValueError("flash_attention_kvcache: paged mode requires seq_lens.")
        if k_cache is None or v_cache is None:
            raise ValueError(
                "flash_attention_kvcache: k_cache and v_cache (page pool) must be provided in paged mode."
            )
        if window_size is not None:
            raise ValueError("flash_attention_kvcache: window_size is not supported in paged mode.")
        if has_rope:
            # keys in the pool are already rotated; only q is, at position cache_seqlens (mlx_mfa/attention.py:1138-1161)
            if rotary_cos is None or rotary_sin is None:
                raise ValueError("flash_attention_kvcache: both rotary_cos and rotary_sin must be provided together.")
            from .rope import apply_rope

            q = apply_rope(q, rotary_cos, rotary_sin, _first_offset(cache_seqlens), interleaved, rotary_dim, stream)
        if alibi_slopes is not None:
            raise ValueError("flash_attention_kvcache: alibi_slopes is not supported in paged mode.")
        # The reference drops softcap here (mlx_mfa/attention.py:1169-1172); it is applied.
        return flash_attention_paged(q, k_cache, v_cache, block_table, seq_lens, scale=scale, causal=causal,
                                     block_size=block_size, stream=stream, k_scale=k_scale, v_scale=v_scale,
                                     softcap=softcap)
    if k_cache is None or v_cache is None:
        raise ValueError(
            "flash_attention_kvcache: k_cache and v_cache must be provided in dense mode "
            "(use block_table to enable paged mode)."
        )
    k_cache, v_cache = _as_tensor(k_cache, "k_cache"), _as_tensor(v_cache, "v_cache")
    if cache_batch_idx is not None:
        idx = _as_tensor(cache_batch_idx, "cache_batch_idx").long()
        k_cache, v_cache = k_cache[idx], v_cache[idx]
    if has_rope:
        # dense cache of unrotated keys: q at cache_seqlens (+ per-batch offsets), keys at [0, S)
        # (the reference routes this to flash_attention_rope and drops softcap / window there, 1195-1203; they apply here)
        if rotary_cos is None or rotary_sin is None:
            raise ValueError("flash_attention_kvcache: both rotary_cos and rotary_sin must be provided together.")
        from .rope import apply_rope

        q = apply_rope(q, rotary_cos, rotary_sin, cache_seqlens, interleaved, rotary_dim, stream)
        k_cache = apply_rope(k_cache, rotary_cos, rotary_sin, 0, interleaved, rotary_dim, stream)
    return flash_attention(q, k_cache, v_cache, scale=scale, causal=causal, softcap=softcap,
                           alibi_slopes=alibi_slopes, window_size=window_size, stream=stream)


# ---------------------------------------------------------------------------
# capability queries (minimal; mlx_mfa/attention.py:558-709)
# ---------------------------------------------------------------------------
def kernel_status(stream=None) -> int:
    """Waits for `stream` and returns (then clears) the device status word of the tcgen05 kernels:
    0 = ok, bit 0 = a bounded wait inside a kernel timed out and that launch's outputs are undefined."""
    lib = _lib.load()
    word = C.c_int32(0)
    dev = torch.device("cuda", torch.cuda.current_device())
    _lib.check(lib.b200fa_kernel_status(C.c_void_p(_stream_ptr(stream, dev)), C.byref(word)), "kernel_status")
    return int(word.value)


def is_mfa_available() -> bool:
    """True when libb200fa.so is built and a CUDA device of compute capability 10.x is visible."""
    if not _lib.is_built() or not torch.cuda.is_available():
        return False
    return torch.cuda.get_device_capability()[0] == 10


def get_device_info() -> dict:
    info = _lib.DeviceInfo()
    _lib.check(_lib.load().b200fa_device_info(-1, C.byref(info)), "get_device_info")
    return {
        "device_name": info.name.decode(),
        "compute_capability": (info.cc_major, info.cc_minor),
        "sm_count": info.sm_count,
        "smem_per_block_optin": info.smem_per_block_optin,
        "total_mem": info.total_mem,
        "has_tcgen05": bool(info.has_tcgen05),
    }


def get_supported_configs() -> dict:
    return {
        "head_dims": list(_SUPPORTED_HDIMS) + list(_FWD_ONLY_HDIMS),
        "dtypes": ["float16", "bfloat16", "float32"],
        "kv_dtypes": ["float16", "bfloat16", "int8", "float8_e4m3fn"],
        "features": {
            "causal": True, "gqa": True, "softcap": True, "window_left": True, "return_lse": True,
            "varlen": True, "paged": True, "quantized_kv": True, "native_backward": True,
            "alibi": True, "dropout": False, "block_sparse": True, "rope": True,
        },
    }
