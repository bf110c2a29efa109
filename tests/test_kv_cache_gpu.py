"""GPU parity of the KV-cache write path: the scatter / quantise kernel against the CPU oracle (bit-exact: it is
byte and integer work), PagedKVCache against the reference's behaviour (append across pages, gather, block
tables: mlx_mfa/attention.py:2531-2816, tests/test_attention.py:3946-3961 in the reference), the cache feeding the
decode kernel, and the dense append mode of flash_attention_kvcache (mlx_mfa/attention.py:1059-1119)."""
import numpy as np
import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from oracle import sdpa_oracle as orc

from .util import assert_close, randn

pytestmark = pytest.mark.gpu

POOL = {"f16": torch.float16, "bf16": torch.bfloat16, "int8": torch.int8, "e4m3": torch.float8_e4m3fn}


def _empty_pool(P, bs, H, D, dtype, dev):
    if dtype == torch.float8_e4m3fn:
        return torch.zeros((P, bs, H, D), dtype=torch.uint8, device=dev).view(dtype)
    return torch.zeros((P, bs, H, D), dtype=dtype, device=dev)


@pytest.mark.parametrize("pool", ["f16", "bf16", "int8", "e4m3"])
@pytest.mark.parametrize("src", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128])
def test_scatter_kernel_is_bit_exact(dev, pool, src, D):
    P, bs, H, T = 9, 16, 3, 41
    pdt = POOL[pool]
    quant = pool in ("int8", "e4m3")
    g = torch.Generator().manual_seed(600 + D)
    # tokens live in a [1, H, T, D] tensor (the layout append() receives); the kernel reads the permuted view
    k4 = (3.0 * torch.randn((1, H, T, D), generator=g)).to(src)
    v4 = torch.randn((1, H, T, D), generator=g).to(src)
    k4[0, 1, 5] = 0                                       # an all-zero row: scale must become 1
    slots = torch.randperm(P * bs, generator=g)[:T].to(torch.int64)
    slots[7] = -1
    kp, vp = _empty_pool(P, bs, H, D, pdt, dev), _empty_pool(P, bs, H, D, pdt, dev)
    ks = vs = None
    if quant:
        ks = torch.full((P, bs, H), 7.0, dtype=torch.float16, device=dev)
        vs = torch.full((P, bs, H), 7.0, dtype=torch.float16, device=dev)
    fa.kv_append(k4[0].permute(1, 0, 2).to(dev), v4[0].permute(1, 0, 2).to(dev), slots.to(dev), kp, vp, ks, vs)
    torch.cuda.synchronize()
    rk, rv = _empty_pool(P, bs, H, D, pdt, "cpu"), _empty_pool(P, bs, H, D, pdt, "cpu")
    rks = rvs = None
    if quant:
        rks = torch.full((P, bs, H), 7.0, dtype=torch.float16)
        rvs = torch.full((P, bs, H), 7.0, dtype=torch.float16)
    orc.kv_append(rk, rv, k4[0].permute(1, 0, 2), v4[0].permute(1, 0, 2), slots.tolist(), rks, rvs)
    bits = torch.uint8 if pdt.itemsize == 1 else torch.int16
    assert torch.equal(kp.cpu().view(bits), rk.view(bits))
    assert torch.equal(vp.cpu().view(bits), rv.view(bits))
    if quant:
        assert torch.equal(ks.cpu(), rks) and torch.equal(vs.cpu(), rvs)


def test_scatter_rejects_bad_arguments(dev):
    kp = torch.zeros((2, 16, 2, 128), dtype=torch.int8, device=dev)
    k = torch.zeros((3, 2, 128), dtype=torch.bfloat16, device=dev)
    slots = torch.zeros(3, dtype=torch.int64, device=dev)
    with pytest.raises(ValueError):
        fa.kv_append(k, k, slots, kp, kp.clone())                      # 8-bit pool without scales
    with pytest.raises(ValueError):
        fa.kv_append(k, k, slots.int(), kp, kp.clone(), torch.ones((2, 16, 2), dtype=torch.float16, device=dev),
                     torch.ones((2, 16, 2), dtype=torch.float16, device=dev))   # int32 slots
    with pytest.raises(NotImplementedError):
        fa.kv_append(k.float(), k.float(), slots, kp, kp.clone())
    with pytest.raises(RuntimeError):
        fa.kv_append(k.cpu(), k.cpu(), slots.cpu(), kp.cpu(), kp.cpu())   # no CPU path


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_cache_append_gather_round_trip(dev, dtype):
    cache = fa.PagedKVCache(num_blocks=12, block_size=16, H=2, D=128, dtype=dtype, device=dev)
    k_all = randn((1, 2, 50, 128), dtype, 610).to(dev)
    v_all = randn((1, 2, 50, 128), dtype, 611).to(dev)
    cache.append(k_all[:, :, :37], v_all[:, :, :37], seq_id=3)         # prefill crossing two page boundaries
    for t in range(37, 50):                                             # decode, one token per call
        cache.append(k_all[:, :, t:t + 1], v_all[:, :, t:t + 1], seq_id=3)
    k, v = cache.gather(3)
    assert torch.equal(k, k_all) and torch.equal(v, v_all)
    assert cache.seq_lengths == {3: 50}
    table, lens = cache.block_table_and_seq_lens([3])
    assert table.shape == (1, 4) and table.dtype == torch.int32 and lens.tolist() == [50]
    cache.free_seq(3)
    assert cache.seq_lengths == {} and "used=0/12" in repr(cache)
    ek, ev = cache.gather(3)
    assert ek.shape == (1, 2, 0, 128)


@pytest.mark.parametrize("kind", [None, "int8", "e4m3"])
def test_cache_feeds_the_decode_kernel(dev, kind):
    """Three sequences of different length are prefilled and extended with append_batch, then one decode step runs on
    the cache's pools; the oracle attends on the same tokens (quantised by its own quantiser for 8-bit pools)."""
    H, D, bs = 2, 128, 16
    lens = [45, 16, 130]
    cache = fa.PagedKVCache(num_blocks=20, block_size=bs, H=H, D=D, dtype=torch.bfloat16, kv_dtype=kind, device=dev)
    toks = [(randn((1, H, n + 2, D), torch.bfloat16, 620 + i), randn((1, H, n + 2, D), torch.bfloat16, 630 + i)) for i, n in enumerate(lens)]
    for i, n in enumerate(lens):
        cache.append(toks[i][0][:, :, :n].to(dev), toks[i][1][:, :, :n].to(dev), seq_id=10 + i)
    for step in range(2):                                               # two batched decode-step appends
        kb = torch.cat([toks[i][0][:, :, lens[i] + step:lens[i] + step + 1] for i in range(3)], dim=0)
        vb = torch.cat([toks[i][1][:, :, lens[i] + step:lens[i] + step + 1] for i in range(3)], dim=0)
        cache.append_batch(kb.to(dev), vb.to(dev), [10, 11, 12])
    table, sl = cache.block_table_and_seq_lens([10, 11, 12])
    assert sl.tolist() == [n + 2 for n in lens]
    q = randn((3, 8, 1, D), torch.bfloat16, 640)
    out = fa.flash_attention_paged(q.to(dev), cache.k_pool, cache.v_pool, table, sl, causal=True, block_size=bs,
                                   k_scale=cache.k_scale, v_scale=cache.v_scale)
    torch.cuda.synchronize()
    # oracle: the same tokens written by the oracle's scatter into pools of its own, with the cache's block table
    P = cache.num_blocks
    pdt = torch.bfloat16 if kind is None else POOL[kind]
    rk, rv = _empty_pool(P, bs, H, D, pdt, "cpu"), _empty_pool(P, bs, H, D, pdt, "cpu")
    rks = rvs = None
    if kind is not None:
        rks, rvs = torch.ones((P, bs, H), dtype=torch.float16), torch.ones((P, bs, H), dtype=torch.float16)
    tb = table.cpu()
    for i, n in enumerate(lens):
        slots = [int(tb[i, t // bs]) * bs + t % bs for t in range(n + 2)]
        orc.kv_append(rk, rv, toks[i][0][0].permute(1, 0, 2), toks[i][1][0].permute(1, 0, 2), slots, rks, rvs)
    bits = torch.uint8 if pdt.itemsize == 1 else torch.int16
    assert torch.equal(cache.k_pool.cpu().view(bits), rk.view(bits))   # the pools themselves agree byte for byte
    O, _ = orc.paged_attention(q, rk, rv, tb, sl.cpu(), causal=True, k_scale=rks, v_scale=rvs)
    assert_close(out, O, torch.bfloat16)
    if kind is not None:
        gk, _ = cache.gather(11)
        assert gk.shape == (1, H, 18, D) and float((gk.float().cpu() - toks[1][0].float()).abs().max()) < 0.2


def test_dense_append_mode_returns_the_updated_cache(dev):
    """flash_attention_kvcache(k_new=, v_new=) concatenates, attends and returns (out, k_updated, v_updated)."""
    q = randn((2, 4, 1, 128), torch.float16, 650)
    kc, vc = randn((2, 2, 70, 128), torch.float16, 651), randn((2, 2, 70, 128), torch.float16, 652)
    kn, vn = randn((2, 2, 1, 128), torch.float16, 653), randn((2, 2, 1, 128), torch.float16, 654)
    out, ku, vu = fa.flash_attention_kvcache(q.to(dev), kc.to(dev), vc.to(dev), k_new=kn.to(dev), v_new=vn.to(dev))
    assert ku.shape == (2, 2, 71, 128) and torch.equal(ku.cpu(), torch.cat([kc, kn], 2)) and torch.equal(vu.cpu(), torch.cat([vc, vn], 2))
    O, _, _ = orc.sdpa(q, torch.cat([kc, kn], 2), torch.cat([vc, vn], 2), causal=True)
    assert_close(out, O, torch.float16)
    out2, k2, _ = fa.flash_attention_kvcache(q.to(dev), None, None, k_new=kn.to(dev), v_new=vn.to(dev))
    assert k2.shape == (2, 2, 1, 128)
    assert_close(out2, vn.repeat_interleave(2, 1), torch.float16)       # one key: the output is its value
    with pytest.raises(ValueError):
        fa.flash_attention_kvcache(q.to(dev), kc.to(dev), vc.to(dev), k_new=kn.to(dev))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_backward_through_the_page_pool(dev, dtype):
    """dQ and pool-shaped dK / dV through flash_attention_paged: two sequences of different length, -1 padding, and a
    page shared by both sequences (its gradient is the sum of both), against float64 autograd through the same
    gather written with index operations (the reference's vjp: gather, per-sequence vjp, _scatter_to_pool;
    mlx_mfa/attention.py:2878-2940, 3020-3084)."""
    P, bs, H, D = 10, 16, 2, 64
    lens = [40, 23]
    table = torch.tensor([[7, 2, 5], [7, 4, -1]], dtype=torch.int32)         # page 7 is a shared prefix
    kp, vp = randn((P, bs, H, D), dtype, 660), randn((P, bs, H, D), dtype, 661)
    q, do = randn((2, 4, 24, D), dtype, 662), randn((2, 4, 24, D), dtype, 663)
    qg, kg, vg = (x.to(dev).requires_grad_(True) for x in (q, kp, vp))
    out = fa.flash_attention_paged(qg, kg, vg, table.to(dev), torch.tensor(lens, dtype=torch.int32, device=dev),
                                   causal=True, block_size=bs)
    out.backward(do.to(dev))
    torch.cuda.synchronize()
    # oracle
    qr, kr, vr = (x.double().requires_grad_(True) for x in (q, kp, vp))
    outs = []
    for b, n in enumerate(lens):
        pages = table[b, : (n + bs - 1) // bs].long()
        K = kr[pages].reshape(-1, H, D)[:n].permute(1, 0, 2)[None]
        V = vr[pages].reshape(-1, H, D)[:n].permute(1, 0, 2)[None]
        O, _, _ = orc.sdpa(qr[b:b + 1], K, V, causal=True)
        outs.append(O)
    ref = torch.cat(outs, 0)
    assert_close(out, ref.detach(), dtype)
    ref.backward(do.double())
    from .util import assert_close_grad
    assert_close_grad(qg.grad, qr.grad, dtype, "dQ")
    assert_close_grad(kg.grad, kr.grad, dtype, "dK pages")
    assert_close_grad(vg.grad, vr.grad, dtype, "dV pages")
    assert kg.grad.shape == kp.shape and float(kg.grad[0].abs().max()) == 0.0       # an unused page gets no gradient
    assert float(kg.grad[5, 8:].abs().max()) == 0.0                                  # nor do slots beyond seq_lens
