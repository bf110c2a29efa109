"""CPU tests of the KV-cache write path's host side: the oracle's quantiser against the format the decode tests
use, the oracle's scatter against the reference's splice semantics, and the block allocator's bookkeeping
(mlx_mfa/attention.py:2531-2816; the reference's own checks are tests/test_attention.py:3946-3961 for
page-crossing appends)."""
import numpy as np
import pytest
import torch

from oracle import sdpa_oracle as orc

from .util import make_paged


@pytest.mark.parametrize("kind", ["int8", "e4m3"])
def test_quantiser_matches_the_pool_format_of_the_decode_tests(kind):
    """make_paged builds quantised pools from float32 rows; the oracle quantiser must give the same bytes and scales."""
    pg = make_paged(2, 2, 128, 16, [40, 9], torch.bfloat16, 77, quant=kind)
    g = torch.Generator().manual_seed(78)
    P = pg["num_pages"]
    kf = torch.randn((P, 16, 2, 128), generator=g)
    q, sc = orc.quantise_kv(kf, kind)
    assert torch.equal(q.view(torch.uint8), pg["k"].view(torch.uint8))
    assert torch.equal(sc, pg["k_scale"])


@pytest.mark.parametrize("kind", ["int8", "e4m3"])
def test_quantise_dequantise_round_trip(kind):
    g = torch.Generator().manual_seed(5)
    x = torch.randn((7, 3, 128), generator=g).to(torch.bfloat16)
    q, sc = orc.quantise_kv(x, kind)
    back = orc.dequant(q, sc, torch.float32)
    step = sc.float().unsqueeze(-1) * (0.5 if kind == "int8" else 16.0)   # half a step / half an e4m3 ulp at the top binade
    assert bool(((back - x.float()).abs() <= step + 1e-6).all())
    z, zs = orc.quantise_kv(torch.zeros((2, 1, 64)), kind)
    assert float(zs.max()) == 1.0 and int(z.view(torch.uint8).max()) == 0


def test_scatter_oracle_crosses_pages_and_skips_negative_slots():
    P, bs, H, D = 4, 4, 2, 64
    kp = torch.zeros((P, bs, H, D), dtype=torch.float16)
    vp = torch.zeros_like(kp)
    g = torch.Generator().manual_seed(6)
    kn = torch.randn((6, H, D), generator=g).to(torch.float16)
    vn = torch.randn((6, H, D), generator=g).to(torch.float16)
    slots = [2 * bs + 2, 2 * bs + 3, 0 * bs + 0, -1, 0 * bs + 1, 99]     # page 2 fills up, continues on page 0; one padding, one outside
    orc.kv_append(kp, vp, kn, vn, slots)
    assert torch.equal(kp[2, 2], kn[0]) and torch.equal(kp[2, 3], kn[1]) and torch.equal(kp[0, 0], kn[2])
    assert torch.equal(vp[0, 1], vn[4])
    assert int((kp != 0).any(-1).any(-1).sum()) == 4          # nothing else written


def test_allocator_bookkeeping_without_a_gpu(monkeypatch):
    """Slots handed out by the cache follow the reference's allocation order: a stack of free blocks popped from the
    end, a new block only when the last one is full, blocks returned on free_seq."""
    from mlx_flashattention_steel_b200 import kv_cache as kc

    cache = kc.PagedKVCache.__new__(kc.PagedKVCache)
    cache.num_blocks, cache.block_size, cache.H, cache.D = 5, 4, 1, 64
    cache._free = list(range(5))
    cache._block_table, cache._write_ptr = {}, {}
    s0 = cache._reserve(0, 6)        # blocks 4 then 3
    assert s0 == [16, 17, 18, 19, 12, 13]
    s1 = cache._reserve(7, 1)        # block 2
    assert s1 == [8]
    assert cache.seq_lengths == {0: 6, 7: 1}
    assert cache._reserve(0, 3) == [14, 15, 4]               # fills block 3, continues on block 1
    cache.free_seq(0)
    assert sorted(cache._free) == [0, 1, 3, 4] and cache.seq_lengths == {7: 1}
    with pytest.raises(RuntimeError):
        cache._reserve(9, 4 * 4 + 1)
