"""Multi-GPU host logic: one process per GPU, `torch.distributed` for the plumbing.

The reference is single-device (no rank, world size or collective anywhere in it), so
nothing here mirrors a reference file; it is the layer a serving or training stack puts
around the operators on an 8-GPU box.

* (batch, kv-head) shards are independent in forward, backward and decode — each query
  head reads exactly one kv head — so the batched operators need no collective:
  ``shard_units`` deals the (batch, kv-head) units out and each rank runs the ordinary
  operators on views of its shard.
* One very long decode sequence is the exception: its page list is split across ranks,
  every rank runs the same split-KV decode kernel over its pages, which leaves its partial
  (fp32 rows with their base-2 lse) in one packed buffer; ``combine_packed`` merges the ranks'
  partials with one small NCCL all-gather (Hq*(D+4) floats per rank) and one launch of the
  library's combine kernel -- the log-sum-exp rule the decode kernel itself uses between CTAs
  (``L = log2 sum_r 2^lse_r``, ``O = sum_r 2^(lse_r - L) O_r``).  ``combine_partials`` is the
  same rule in torch ops for host tensors (the gloo tests of the host logic).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous balanced split of ``range(n)``: the first ``n % world`` ranks get one extra."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_by_load(loads, world: int) -> List[List[int]]:
    """Deals items with unequal cost (sequences by their KV length) out to ``world`` ranks so that the heaviest rank is
    as light as a greedy pass makes it: items in order of decreasing load, each to the rank that is lightest so far
    (ties: the lower rank; equal loads: the lower index first).  Returns each rank's item indices in increasing order.
    Every rank computes the same deal from the same ``loads``; nothing is exchanged."""
    if world <= 0:
        raise ValueError(f"bad world: {world}")
    loads = [int(x) for x in loads]
    order = sorted(range(len(loads)), key=lambda i: (-loads[i], i))
    total = [0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (total[j], j))
        owned[r].append(i)
        total[r] += loads[i]
    return [sorted(o) for o in owned]


def shard_units(B: int, Hkv: int, world: int, rank: int) -> List[Tuple[int, int]]:
    """(batch, kv-head) units owned by ``rank``; unit u = b * Hkv + h, dealt contiguously so a
    rank's units are a few whole batches plus a contiguous head range (views, no copies)."""
    lo, hi = shard_range(B * Hkv, world, rank)
    return [(u // Hkv, u % Hkv) for u in range(lo, hi)]


def shard_blocks(B: int, Hkv: int, world: int, rank: int) -> List[Tuple[int, int, int]]:
    """The units of ``shard_units`` merged into (batch, first kv head, end kv head) blocks: a rank's units are
    contiguous, so they are at most a partial batch, some whole batches and another partial batch -- one launch each."""
    blocks: List[Tuple[int, int, int]] = []
    for b, h in shard_units(B, Hkv, world, rank):
        if blocks and blocks[-1][0] == b and blocks[-1][2] == h:
            blocks[-1] = (b, blocks[-1][1], h + 1)
        else:
            blocks.append((b, h, h + 1))
    return blocks


def shard_views(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, world: int, rank: int):
    """Yields (b, h, q_view, k_view, v_view) per owned unit: q heads [h*g, (h+1)*g) of batch b with
    kv head h.  Views only; the kernels take the strides as they are."""
    B, Hq = q.shape[0], q.shape[1]
    Hkv = k.shape[1]
    g = Hq // Hkv
    for b, h in shard_units(B, Hkv, world, rank):
        yield b, h, q[b:b + 1, h * g:(h + 1) * g], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1]


def split_pages(num_pages_of_seq: int, world: int, rank: int, block_size: int, seq_len: int) -> Tuple[int, int, int]:
    """Page range [lo, hi) of one long sequence owned by ``rank`` and the number of valid tokens in it."""
    lo, hi = shard_range(num_pages_of_seq, world, rank)
    tok_lo = min(seq_len, lo * block_size)
    tok_hi = min(seq_len, hi * block_size)
    return lo, hi, tok_hi - tok_lo


def combine_partials(out: torch.Tensor, lse: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                     out_dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merges per-rank partial attention results over disjoint key ranges.

    out [..., D] (any float dtype), lse [...] float32 base-2 (``-inf`` where the rank saw no key).
    Returns (O, L) on every rank.  One all-gather of the packed (O fp32, lse) — 4*(D+1) bytes per row
    per rank — then a local weighted sum; the formula is the split combine of the reference's
    flash-decode reduce (csrc/mfa_steel_fwd.cpp:2066-2101) in base 2."""
    world = dist.get_world_size(group)
    packed = torch.cat([out.float(), lse.float().unsqueeze(-1)], dim=-1).contiguous()
    gathered = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(gathered, packed, group=group)
    allp = torch.stack(gathered, dim=0)                    # [world, ..., D+1]
    o_r, l_r = allp[..., :-1], allp[..., -1]
    m = l_r.max(dim=0).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp2(l_r - m_safe)                           # [world, ...]
    wsum = w.sum(dim=0)
    o = (w.unsqueeze(-1) * o_r).sum(dim=0) / torch.where(wsum > 0, wsum, torch.ones_like(wsum)).unsqueeze(-1)
    L = torch.where(wsum > 0, m_safe + torch.log2(torch.where(wsum > 0, wsum, torch.ones_like(wsum))),
                    torch.full_like(m, float("-inf")))
    return o.to(out_dtype or out.dtype), L


def combine_packed(packed: torch.Tensor, D: int, out_dtype: torch.dtype, group: Optional[dist.ProcessGroup] = None,
                   stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merges the per-rank packed partials of the decode kernel (float32 [rows, D+4]: the normalised row in fp32, its
    base-2 lse at column D) into (O [rows, D] out_dtype, L [rows] float32) on every rank: one NCCL all-gather of the
    packed rows -- the partials stay fp32 across ranks -- and one launch of the library's combine kernel."""
    import ctypes as C

    from . import _lib
    from .attention import _DTYPE_CODE, _stream_ptr

    world = dist.get_world_size(group)
    rows = packed.shape[0]
    gathered = torch.empty((world,) + tuple(packed.shape), dtype=torch.float32, device=packed.device)
    dist.all_gather_into_tensor(gathered, packed, group=group)
    out = torch.empty((rows, D), dtype=out_dtype, device=packed.device)
    lse = torch.empty((rows,), dtype=torch.float32, device=packed.device)
    with torch.cuda.device(packed.device):
        st = _lib.load().b200fa_combine_partials(C.c_void_p(gathered.data_ptr()), world, rows, D, _DTYPE_CODE[out_dtype],
                                                 C.c_void_p(out.data_ptr()), C.c_void_p(lse.data_ptr()),
                                                 C.c_void_p(_stream_ptr(stream, packed.device)))
    _lib.check(st, "combine_partials")
    return out, lse


def decode_long_sequence(q, k_pages, v_pages, block_table_local, seq_lens_local, *, group=None, scale=None,
                         k_scale=None, v_scale=None, softcap: float = 0.0, max_kv_len=None, block_size: int = 16):
    """Decode step for sequences whose pages are spread over the ranks of ``group``: every rank passes
    the block table rows and token counts of ITS part of each sequence (q is replicated).  Three launches and one
    collective per step: the paged decode kernel on the local pages, leaving fp32 partials with their lse in one
    packed buffer; an all-gather of that buffer; the combine kernel.  causal is irrelevant for a single query
    token (the reference notes N=1 causal == non-causal, tests/test_attention.py:1472-1487)."""
    import math

    from .attention import _decode_raw

    if q.shape[2] != 1:
        raise NotImplementedError("decode_long_sequence takes one query token per sequence")
    B, Hq, _, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    table = block_table_local.to(torch.int32).contiguous()
    lens = seq_lens_local.to(torch.int32).contiguous()
    if max_kv_len is None:
        max_kv_len = table.shape[1] * block_size        # no host read of seq_lens: the table's width bounds the length
    if k_scale is not None:
        k_scale, v_scale = k_scale.to(torch.float16).contiguous(), v_scale.to(torch.float16).contiguous()
    packed, _ = _decode_raw(q, k_pages.contiguous(), v_pages.contiguous(), k_scale, v_scale, table, lens, int(max_kv_len),
                            float(scale), False, float(softcap), block_size, True, None, packed=True)
    o, l = combine_packed(packed, D, q.dtype, group=group)
    return o.view(B, Hq, 1, D), l.view(B, Hq, 1)
