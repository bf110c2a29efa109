"""CPU tests (gloo, world_size 2) of the multi-GPU host logic: shard planning and the
cross-rank log-sum-exp combine of split-KV partials, checked against the oracle."""
import os

import pytest
import torch
import torch.distributed as dist

from mlx_flashattention_steel_b200 import parallel as par
from oracle import sdpa_oracle as orc

from .util import run_ranks


def test_shard_range_covers_everything_once():
    for n in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = par.shard_range(n, world, r)
                assert 0 <= lo <= hi <= n
                seen += list(range(lo, hi))
            assert seen == list(range(n))
    with pytest.raises(ValueError):
        par.shard_range(4, 2, 2)


def test_shard_by_load_balances_and_covers():
    import numpy as np

    rng = np.random.default_rng(4)
    lens = rng.integers(512, 32769, size=128)
    for world in (1, 2, 3, 4, 8):
        deal = par.shard_by_load(lens, world)
        assert len(deal) == world
        flat = sorted(i for d in deal for i in d)
        assert flat == list(range(128))                       # every sequence exactly once
        assert all(d == sorted(d) for d in deal)
        totals = [int(lens[d].sum()) for d in deal]
        # a greedy deal is within one item of even: no rank exceeds the mean by more than the longest sequence
        assert max(totals) - sum(totals) / world <= int(lens.max())
        assert par.shard_by_load(lens, world) == deal          # deterministic: every rank computes the same deal
    # contiguous dealing of the same lengths is visibly worse at eight ranks
    contiguous = [int(lens[slice(*par.shard_range(128, 8, r))].sum()) for r in range(8)]
    assert max(int(lens[d].sum()) for d in par.shard_by_load(lens, 8)) < max(contiguous)
    assert par.shard_by_load([], 2) == [[], []]
    assert par.shard_by_load([5, 5, 5], 2) == [[0, 2], [1]]
    with pytest.raises(ValueError):
        par.shard_by_load([1], 0)


def test_shard_units_config2():
    # 4 batches x 8 kv heads over 8 GPUs -> 4 units each, whole number of heads of one batch
    all_units = []
    for r in range(8):
        u = par.shard_units(4, 8, 8, r)
        assert len(u) == 4 and len({b for b, _ in u}) == 1
        all_units += u
    assert sorted(all_units) == [(b, h) for b in range(4) for h in range(8)]


def test_shard_blocks_merge_contiguous_units():
    # 4 batches x 8 kv heads: one GPU takes every batch whole; 8 GPUs take half a batch each; 3 GPUs cut batches
    assert par.shard_blocks(4, 8, 1, 0) == [(0, 0, 8), (1, 0, 8), (2, 0, 8), (3, 0, 8)]
    assert par.shard_blocks(4, 8, 8, 5) == [(2, 4, 8)]
    seen = []
    for r in range(3):
        for b, h0, h1 in par.shard_blocks(4, 8, 3, r):
            assert 0 <= h0 < h1 <= 8
            seen += [(b, h) for h in range(h0, h1)]
    assert seen == [(b, h) for b in range(4) for h in range(8)]


def test_shard_views_are_views():
    q, k, v = torch.zeros(2, 8, 4, 16), torch.zeros(2, 2, 6, 16), torch.zeros(2, 2, 6, 16)
    got = list(par.shard_views(q, k, v, 2, 1))
    assert [(b, h) for b, h, *_ in got] == [(1, 0), (1, 1)]
    _, _, qv, kv, _ = got[1]
    assert qv.shape == (1, 4, 4, 16) and kv.shape == (1, 1, 6, 16)
    assert qv.data_ptr() == q[1, 4].data_ptr()


def test_split_pages():
    # 100 tokens, 7 pages of 16, over 2 ranks: pages [0,4) and [4,7) -> 64 and 36 tokens
    assert par.split_pages(7, 2, 0, 16, 100) == (0, 4, 64)
    assert par.split_pages(7, 2, 1, 16, 100) == (4, 7, 36)


def _worker(rank, world, port, q, k, v, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        S = k.shape[2]
        lo, hi = par.shard_range(S, world, rank)
        if rank == 1:
            hi = lo            # rank 1 holds no key at all: lse = -inf must drop out of the combine
        elif world == 2:
            hi = S
        if hi > lo:
            o, l, _ = orc.sdpa(q, k[:, :, lo:hi], v[:, :, lo:hi])
        else:
            o = torch.zeros(q.shape, dtype=torch.float64)
            l = torch.full(q.shape[:3], float("-inf"), dtype=torch.float64)
        O, L = par.combine_partials(o.float(), l.float())
        # second round: a real split
        lo, hi = par.shard_range(S, world, rank)
        o, l, _ = orc.sdpa(q, k[:, :, lo:hi], v[:, :, lo:hi])
        O2, L2 = par.combine_partials(o.float(), l.float())
        if rank == 0:
            ret.put((O, L, O2, L2))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_combine_partials_over_gloo():
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 4, 1, 32), torch.randn(2, 2, 77, 32), torch.randn(2, 2, 77, 32)
    O, L, O2, L2 = run_ranks(_worker, 2, (q, k, v), timeout=120)
    ref, lref, _ = orc.sdpa(q, k, v)
    for o, l in ((O, L), (O2, L2)):
        assert float((o.double() - ref).abs().max()) < 1e-5
        assert float((l.double() - lref).abs().max()) < 1e-4
