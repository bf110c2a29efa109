"""Paged KV cache: block allocator on the host, pools on the GPU, writes by one scatter kernel.

Mirrors the reference's ``PagedKVCache`` (mlx_mfa/attention.py:2531-2816): same constructor
arguments, methods and return conventions (pool layout ``[num_blocks, block_size, H, D]``,
block tables padded with ``-1``, ``seq_lengths`` as a dict).  Differences, all additions:

* ``append`` launches ``b200fa_kv_append`` once instead of splicing the pool block by block,
  and ``append_batch`` writes one step of many sequences in the same single launch;
* ``kv_dtype="int8"`` / ``"e4m3"`` keeps 8-bit pools with per-(token, head) f16 scales
  (``k_scale`` / ``v_scale``), the format ``flash_attention_paged`` reads for decode.

The allocator (free list, block tables, write pointers) is host Python as in the reference;
nothing in it touches the device.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib
from .attention import _DTYPE_CODE, _as_tensor, _require_cuda, _stream_ptr

_POOL_DTYPES = {"int8": torch.int8}
if hasattr(torch, "float8_e4m3fn"):
    _POOL_DTYPES["e4m3"] = torch.float8_e4m3fn
_POOL_CODE = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.int8: _lib.I8}
if hasattr(torch, "float8_e4m3fn"):
    _POOL_CODE[torch.float8_e4m3fn] = _lib.E4M3


def kv_append(k_new, v_new, slot_mapping, k_pool, v_pool, k_scale=None, v_scale=None, stream=None) -> None:
    """Scatter new tokens into page pools in place.

    k_new / v_new: ``[T, Hkv, D]`` f16 / bf16 (any token / head strides whose rows are contiguous);
    slot_mapping: int64 ``[T]`` on the device, ``page * block_size + offset`` (negative = skip);
    pools ``[P, block_size, Hkv, D]`` of f16 / bf16 / int8 / float8_e4m3fn, 8-bit pools with f16
    scales ``[P, block_size, Hkv]``."""
    _require_cuda(k_new, v_new, slot_mapping, k_pool, v_pool)
    if k_new.dtype not in (torch.float16, torch.bfloat16) or v_new.dtype != k_new.dtype:
        raise NotImplementedError("kv_append takes f16/bf16 tokens, K and V of one dtype.")
    if k_pool.dtype not in _POOL_CODE or v_pool.dtype != k_pool.dtype:
        raise NotImplementedError(f"kv_append: pool dtype {k_pool.dtype} not built.")
    if k_new.ndim != 3 or k_new.shape != v_new.shape:
        raise ValueError("kv_append: k_new and v_new must both be [T, Hkv, D].")
    T, H, D = k_new.shape
    P, bs, Hp, Dp = k_pool.shape
    if (Hp, Dp) != (H, D) or v_pool.shape != k_pool.shape:
        raise ValueError("kv_append: pools must be [P, block_size, Hkv, D] with the tokens' Hkv and D.")
    if slot_mapping.dtype != torch.int64 or slot_mapping.numel() != T:
        raise ValueError("kv_append: slot_mapping must be int64 [T].")
    if not (k_pool.is_contiguous() and v_pool.is_contiguous() and slot_mapping.is_contiguous()):
        raise ValueError("kv_append: pools and slot_mapping must be contiguous.")
    quant = k_pool.dtype not in (torch.float16, torch.bfloat16)
    if quant:
        for s in (k_scale, v_scale):
            if s is None or s.dtype != torch.float16 or tuple(s.shape) != (P, bs, H) or not s.is_contiguous():
                raise ValueError("kv_append: 8-bit pools need contiguous f16 scales [P, block_size, Hkv].")
    def rows_ok(x):   # the kernel reads rows with 16-byte loads
        return x.stride(2) == 1 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0 and x.data_ptr() % 16 == 0

    if not (rows_ok(k_new) and rows_ok(v_new)) or v_new.stride() != k_new.stride():
        k_new, v_new = k_new.contiguous(), v_new.contiguous()
    if T == 0:
        return
    lib = _lib.load()
    st = lib.b200fa_kv_append(
        _DTYPE_CODE[k_new.dtype], _POOL_CODE[k_pool.dtype], T, H, D, bs, P,
        C.c_void_p(k_new.data_ptr()), C.c_void_p(v_new.data_ptr()), k_new.stride(0), k_new.stride(1),
        C.c_void_p(slot_mapping.data_ptr()), C.c_void_p(k_pool.data_ptr()), C.c_void_p(v_pool.data_ptr()),
        C.c_void_p(k_scale.data_ptr()) if quant else None, C.c_void_p(v_scale.data_ptr()) if quant else None,
        C.c_void_p(_stream_ptr(stream, k_pool.device)))
    _lib.check(st, "kv_append")


class PagedKVCache:
    """Paged KV cache manager — dual-pool block allocator (mlx_mfa/attention.py:2531-2816).

    Args:
        num_blocks:  pages in each pool.
        block_size:  tokens per page.
        H:           KV heads.
        D:           head dimension (64 or 128).
        dtype:       dtype of the tokens handed to ``append`` and of 16-bit pools (default float16).
        kv_dtype:    ``None`` (pools in ``dtype``), ``"int8"`` or ``"e4m3"``.
        device:      CUDA device of the pools (default the current one).
    """

    def __init__(self, num_blocks: int, block_size: int, H: int, D: int, dtype=None, kv_dtype: Optional[str] = None,
                 device=None) -> None:
        if dtype is None:
            dtype = torch.float16
        if dtype not in (torch.float16, torch.bfloat16):
            raise NotImplementedError("PagedKVCache pools take float16 / bfloat16 tokens.")
        if kv_dtype is not None and kv_dtype not in _POOL_DTYPES:
            raise ValueError(f"PagedKVCache: kv_dtype must be None, 'int8' or 'e4m3', got {kv_dtype!r}.")
        if num_blocks <= 0 or block_size <= 0:
            raise ValueError("PagedKVCache: num_blocks and block_size must be positive.")
        self.num_blocks, self.block_size, self.H, self.D = num_blocks, block_size, H, D
        self.dtype = dtype
        self.kv_dtype = kv_dtype
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        pool_dtype = dtype if kv_dtype is None else _POOL_DTYPES[kv_dtype]
        if pool_dtype in (torch.float16, torch.bfloat16, torch.int8):
            self._k_pool = torch.zeros((num_blocks, block_size, H, D), dtype=pool_dtype, device=self.device)
            self._v_pool = torch.zeros((num_blocks, block_size, H, D), dtype=pool_dtype, device=self.device)
        else:   # float8 tensors are created through their byte view
            self._k_pool = torch.zeros((num_blocks, block_size, H, D), dtype=torch.uint8, device=self.device).view(pool_dtype)
            self._v_pool = torch.zeros((num_blocks, block_size, H, D), dtype=torch.uint8, device=self.device).view(pool_dtype)
        self._k_scale = self._v_scale = None
        if kv_dtype is not None:
            self._k_scale = torch.ones((num_blocks, block_size, H), dtype=torch.float16, device=self.device)
            self._v_scale = torch.ones((num_blocks, block_size, H), dtype=torch.float16, device=self.device)
        self._free: List[int] = list(range(num_blocks))      # stack of available block ids
        self._block_table: Dict[int, List[int]] = {}          # seq_id -> block ids
        self._write_ptr: Dict[int, int] = {}                  # seq_id -> write pointer inside the last block

    # ── internal ──────────────────────────────────────────────────────────
    def _allocate_block(self) -> int:
        if not self._free:
            raise RuntimeError("PagedKVCache: out of blocks — increase num_blocks")
        return self._free.pop()

    def _ensure_seq(self, seq_id: int) -> None:
        if seq_id not in self._block_table:
            self._block_table[seq_id] = [self._allocate_block()]
            self._write_ptr[seq_id] = 0

    def _reserve(self, seq_id: int, T: int) -> List[int]:
        """Advance seq_id by T tokens (allocating blocks as they fill) and return the T slots."""
        self._ensure_seq(seq_id)
        slots = []
        blks = self._block_table[seq_id]
        ptr = self._write_ptr[seq_id]
        for _ in range(T):
            if ptr == self.block_size:
                blks.append(self._allocate_block())
                ptr = 0
            slots.append(blks[-1] * self.block_size + ptr)
            ptr += 1
        self._write_ptr[seq_id] = ptr
        return slots

    # ── pool properties ───────────────────────────────────────────────────
    @property
    def k_pool(self) -> torch.Tensor:
        """Key page pool ``[num_blocks, block_size, H, D]``."""
        return self._k_pool

    @property
    def v_pool(self) -> torch.Tensor:
        """Value page pool ``[num_blocks, block_size, H, D]``."""
        return self._v_pool

    @property
    def k_scale(self) -> Optional[torch.Tensor]:
        """f16 scales ``[num_blocks, block_size, H]`` of an 8-bit key pool, else None."""
        return self._k_scale

    @property
    def v_scale(self) -> Optional[torch.Tensor]:
        return self._v_scale

    # ── public API ────────────────────────────────────────────────────────
    def append(self, k, v, seq_id: int = 0, stream=None) -> None:
        """Append new K/V tokens ``[1, H, T, D]`` for ``seq_id`` (mlx_mfa/attention.py:2642-2711)."""
        k, v = _as_tensor(k, "k"), _as_tensor(v, "v")
        if k.ndim != 4 or k.shape[0] != 1 or k.shape[1] != self.H or k.shape[3] != self.D or v.shape != k.shape:
            raise ValueError(f"PagedKVCache.append: k and v must be [1, {self.H}, T, {self.D}].")
        T = k.shape[2]
        if T == 0:
            self._ensure_seq(seq_id)
            return
        slots = self._reserve(seq_id, T)
        k_tok = k[0].to(self.dtype).permute(1, 0, 2)       # [T, H, D] view: token stride D, head stride T*D
        v_tok = v[0].to(self.dtype).permute(1, 0, 2)
        slot_t = torch.tensor(slots, dtype=torch.int64).to(self.device, non_blocking=True)
        kv_append(k_tok, v_tok, slot_t, self._k_pool, self._v_pool, self._k_scale, self._v_scale, stream)

    def append_batch(self, k, v, seq_ids: Sequence[int], stream=None) -> None:
        """One decode step for many sequences: k, v ``[B, H, T, D]``, row b appended to ``seq_ids[b]``.
        A single launch writes all ``B*T`` tokens (no counterpart in the reference, which loops over append)."""
        k, v = _as_tensor(k, "k"), _as_tensor(v, "v")
        if k.ndim != 4 or k.shape[0] != len(seq_ids) or k.shape[1] != self.H or k.shape[3] != self.D or v.shape != k.shape:
            raise ValueError(f"PagedKVCache.append_batch: k and v must be [{len(seq_ids)}, {self.H}, T, {self.D}].")
        B, _, T, _ = k.shape
        if B == 0 or T == 0:
            return
        slots: List[int] = []
        for s in seq_ids:
            slots.extend(self._reserve(s, T))
        k_tok = k.to(self.dtype).permute(0, 2, 1, 3).reshape(B * T, self.H, self.D)
        v_tok = v.to(self.dtype).permute(0, 2, 1, 3).reshape(B * T, self.H, self.D)
        slot_t = torch.tensor(slots, dtype=torch.int64).to(self.device, non_blocking=True)
        kv_append(k_tok, v_tok, slot_t, self._k_pool, self._v_pool, self._k_scale, self._v_scale, stream)

    def gather(self, seq_id: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
        """Contiguous ``(k, v)`` ``[1, H, S, D]`` of ``seq_id`` (mlx_mfa/attention.py:2713-2743).  8-bit pools are
        dequantised to ``dtype`` (value * scale)."""
        blks = self._block_table.get(seq_id, [])
        seqlen = self.seq_lengths.get(seq_id, 0)
        if not blks or seqlen == 0:
            z = torch.zeros((1, self.H, 0, self.D), dtype=self.dtype, device=self.device)
            return z, z.clone()
        idx = torch.tensor(blks, dtype=torch.int64, device=self.device)
        outs = []
        for pool, scale in ((self._k_pool, self._k_scale), (self._v_pool, self._v_scale)):
            flat = pool[idx].reshape(-1, self.H, self.D)[:seqlen]
            if scale is not None:
                sc = scale[idx].reshape(-1, self.H)[:seqlen]
                flat = (flat.to(torch.float32) * sc.to(torch.float32).unsqueeze(-1)).to(self.dtype)
            outs.append(flat.permute(1, 0, 2)[None])
        return outs[0], outs[1]

    def get_block_table(self, seq_ids: Optional[List[int]] = None) -> torch.Tensor:
        """int32 ``[B, max_blocks_per_seq]`` on the cache's device, unused slots ``-1`` (2745-2769)."""
        if seq_ids is None:
            seq_ids = sorted(self._block_table.keys())
        if not seq_ids:
            return torch.zeros((0, 0), dtype=torch.int32, device=self.device)
        max_blks = max(len(self._block_table[s]) for s in seq_ids)
        table = [self._block_table[s] + [-1] * (max_blks - len(self._block_table[s])) for s in seq_ids]
        return torch.tensor(table, dtype=torch.int32).to(self.device)

    def get_seq_lens(self, seq_ids: Optional[List[int]] = None) -> torch.Tensor:
        """int32 ``[B]`` token counts (2771-2788)."""
        if seq_ids is None:
            seq_ids = sorted(self._block_table.keys())
        lens = [self.seq_lengths.get(s, 0) for s in seq_ids]
        return torch.tensor(lens, dtype=torch.int32).to(self.device)

    def block_table_and_seq_lens(self, seq_ids: List[int]) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.get_block_table(seq_ids), self.get_seq_lens(seq_ids)

    @property
    def seq_lengths(self) -> Dict[int, int]:
        """``{seq_id: tokens written}`` for all active sequences."""
        return {sid: (len(blks) - 1) * self.block_size + self._write_ptr[sid] for sid, blks in self._block_table.items()}

    def free_seq(self, seq_id: int) -> None:
        """Release all blocks held by ``seq_id`` back to the free list."""
        if seq_id in self._block_table:
            self._free.extend(self._block_table.pop(seq_id))
            self._write_ptr.pop(seq_id, None)

    def __repr__(self) -> str:
        used = self.num_blocks - len(self._free)
        return (f"PagedKVCache(blocks={self.num_blocks}, block_size={self.block_size}, H={self.H}, D={self.D}, "
                f"kv_dtype={self.kv_dtype}, used={used}/{self.num_blocks})")
