"""GPU parity of the paged split-KV decode kernel against the CPU oracle (gather pages,
dequantise to the query dtype, attend per sequence to its exact length), 2e-2 max-abs.
Cases follow the reference's paged tests (tests/test_attention.py in the reference:
two sequences of different length with -1 padding 3812-3857, decode rows 1525-1598)."""
import numpy as np
import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from mlx_flashattention_steel_b200 import attention as A
from oracle import sdpa_oracle as orc

from .util import assert_close, make_paged, randn

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_checks():
    old = A._set_check_decode_status(True)
    yield
    A._set_check_decode_status(old)


def _run(dev, qdtype, quant, B, Hq, Hkv, Nq, lens, seed, causal=True, softcap=0.0, num_splits=0, holes=False, tol=2e-2,
         D=128, block_size=16):
    pg = make_paged(B, Hkv, D, block_size, lens, qdtype, seed, quant=quant)
    table = pg["block_table"].clone()
    if holes:
        table[B - 1, 1] = -1
    q = randn((B, Hq, Nq, D), qdtype, seed + 7)
    ks, vs = pg["k_scale"], pg["v_scale"]
    out, lse = fa.flash_attention_paged(
        q.to(dev), pg["k"].to(dev), pg["v"].to(dev), table.to(dev), pg["seq_lens"].to(dev), causal=causal,
        k_scale=None if ks is None else ks.to(dev), v_scale=None if vs is None else vs.to(dev), softcap=softcap,
        return_lse=True, num_splits=num_splits, block_size=block_size)
    torch.cuda.synchronize()
    O, L = orc.paged_attention(q, pg["k"], pg["v"], table, pg["seq_lens"], causal=causal, softcap=softcap,
                               k_scale=ks, v_scale=vs)
    assert out.shape == q.shape and out.dtype == qdtype
    assert_close(out, O, qdtype, "out", tol)
    assert_close(lse, L, qdtype, "lse", tol)


LENS = [1, 16, 17, 500, 3000]


@pytest.mark.parametrize("qdtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("quant", [None, "int8", "e4m3"])
@pytest.mark.parametrize("num_splits", [0, 1, 3])
def test_decode_kinds(dev, qdtype, quant, num_splits):
    _run(dev, qdtype, quant, len(LENS), 32, 8, 1, LENS, 400, num_splits=num_splits)


@pytest.mark.parametrize("Hq,Hkv", [(4, 1), (4, 2), (8, 4), (16, 16), (48, 24), (8, 1)])
@pytest.mark.parametrize("quant", [None, "int8"])
def test_decode_head_layouts(dev, Hq, Hkv, quant):
    _run(dev, torch.bfloat16, quant, 3, Hq, Hkv, 1, [33, 700, 129], 410)


@pytest.mark.parametrize("Nq,Hq,Hkv", [(2, 8, 2), (4, 4, 2), (8, 2, 2), (5, 3, 3)])
@pytest.mark.parametrize("causal", [False, True])
def test_decode_several_query_rows(dev, Nq, Hq, Hkv, causal):
    _run(dev, torch.float16, "int8", 4, Hq, Hkv, Nq, [16, 40, 333, 8], 420, causal=causal)
    _run(dev, torch.bfloat16, None, 4, Hq, Hkv, Nq, [16, 40, 333, 8], 421, causal=causal)


def test_decode_empty_sequences_and_holes(dev):
    _run(dev, torch.bfloat16, "int8", 5, 32, 8, 1, [0, 100, 0, 48, 64], 430, holes=True)
    _run(dev, torch.float16, None, 5, 8, 8, 1, [0, 100, 0, 48, 64], 431, holes=True)


@pytest.mark.parametrize("quant", [None, "int8", "e4m3"])
def test_decode_ignores_garbage_beyond_the_sequence_end(dev, quant):
    """Slots of a sequence's last page beyond seq_lens hold whatever the pool's owner left there (a pool from
    cudaMalloc or torch.empty, a recycled page).  NaN patterns in those K / V rows and scales must not reach the
    output: their probabilities are zero, but 0 * NaN is NaN unless the values are masked too."""
    lens = [5, 17, 100, 33]
    qdtype = torch.bfloat16
    pg = make_paged(4, 2, 128, 16, lens, qdtype, 77, quant=quant)
    table = pg["block_table"]
    for b, n in enumerate(lens):
        page = int(table[b, (n - 1) // 16])
        first = n % 16
        if first == 0:
            continue
        if quant is None:
            pg["k"][page, first:] = float("nan")
            pg["v"][page, first:] = float("nan")
        else:
            pg["k_scale"][page, first:] = float("nan")
            pg["v_scale"][page, first:] = float("inf")
            if quant == "e4m3":
                pg["v"].view(torch.uint8)[page, first:] = 0x7F        # e4m3 NaN
                pg["k"].view(torch.uint8)[page, first:] = 0xFF
    q = randn((4, 8, 1, 128), qdtype, 78)
    ks, vs = pg["k_scale"], pg["v_scale"]
    out, lse = fa.flash_attention_paged(
        q.to(dev), pg["k"].to(dev), pg["v"].to(dev), table.to(dev), pg["seq_lens"].to(dev), causal=True,
        k_scale=None if ks is None else ks.to(dev), v_scale=None if vs is None else vs.to(dev), return_lse=True)
    O, L = orc.paged_attention(q, pg["k"], pg["v"], table, pg["seq_lens"], causal=True, k_scale=ks, v_scale=vs)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    assert_close(out, O, qdtype)
    assert_close(lse, L, qdtype, "lse")


@pytest.mark.parametrize("block_size", [32, 64, 48])
@pytest.mark.parametrize("quant", [None, "int8", "e4m3"])
def test_decode_page_sizes(dev, block_size, quant):
    """The reference takes any block_size (mlx_mfa/attention.py:914, 2828; its docstring recommends 16, 32 or 64):
    pages of several 16-token units, ragged last pages, holes and split sequences."""
    _run(dev, torch.bfloat16, quant, 5, 8, 2, 1, [1, 31, 33, 700, 2900], 480, block_size=block_size, holes=True)
    _run(dev, torch.float16, quant, 3, 4, 4, 2, [64, 65, 1500], 481, block_size=block_size, num_splits=3)


@pytest.mark.parametrize("qdtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("block_size", [16, 64])
def test_decode_head_dim_64(dev, qdtype, block_size):
    """head_dim 64 pools (16-bit): GQA groups, several query rows, split sequences."""
    _run(dev, qdtype, None, 5, 8, 2, 1, LENS, 485, D=64, block_size=block_size)
    _run(dev, qdtype, None, 3, 6, 3, 4, [70, 900, 2000], 486, D=64, block_size=block_size, causal=True, softcap=20.0)
    _run(dev, qdtype, None, 2, 16, 16, 1, [300, 5000], 487, D=64, block_size=block_size, num_splits=2)


@pytest.mark.parametrize("N", [1, 4, 5])
@pytest.mark.parametrize("S", [255, 256, 1000, 4099])
@pytest.mark.parametrize("D", [64, 128])
def test_dense_cache_decode_route(dev, N, S, D):
    """Plain flash_attention / dense flash_attention_kvcache calls with a few query rows against a long cache: the
    reference switches to flash-decoding at N <= 4 and S >= 256 (csrc/mfa_attention.cpp:150-151; its own threshold
    cases are tests/test_attention.py:1525-1598 in the reference).  Both sides of the threshold, ragged S, causal and
    not, GQA, soft cap, and a cache that is a view of a longer buffer, against the oracle."""
    dtype = torch.bfloat16
    B, Hq, Hkv = 2, 8, 4
    q = randn((B, Hq, N, D), dtype, 490)
    kbuf = randn((B, Hkv, S + 37, D), dtype, 491)
    vbuf = randn((B, Hkv, S + 37, D), dtype, 492)
    k, v = kbuf[:, :, :S], vbuf[:, :, :S]                       # strided views: batch / head strides of the longer buffer
    for causal, softcap in ((True, 0.0), (False, 0.0), (True, 30.0)):
        out, lse = fa.flash_attention(q.to(dev), kbuf.to(dev)[:, :, :S], vbuf.to(dev)[:, :, :S], causal=causal,
                                      softcap=softcap, return_lse=True)
        O, L, _ = orc.sdpa(q, k, v, causal=causal, softcap=softcap)
        assert_close(out, O, dtype)
        assert_close(lse, L, dtype, "lse")
    out = fa.flash_attention_kvcache(q.to(dev), k.to(dev), v.to(dev), causal=True)
    O, _, _ = orc.sdpa(q, k, v, causal=True)
    assert_close(out, O, dtype)


def test_dense_cache_decode_matches_prefill_kernel(dev):
    """The decode route and the prefill kernel must agree on the same call (different bits show both really ran)."""
    from mlx_flashattention_steel_b200 import _lib

    q = randn((3, 16, 2, 128), torch.float16, 495).to(dev)
    k, v = (randn((3, 4, 3000, 128), torch.float16, 496 + i).to(dev) for i in range(2))
    a, la = fa.flash_attention(q, k, v, causal=True, return_lse=True)
    old = A._set_force_flags(_lib.FLAG_FORCE_MMA_SYNC)          # keeps the call off the decode route
    try:
        b, lb = fa.flash_attention(q, k, v, causal=True, return_lse=True)
    finally:
        A._set_force_flags(old)
    assert float((a.float() - b.float()).abs().max()) <= 2e-2 and float((la - lb).abs().max()) <= 2e-2
    assert not torch.equal(a, b)


def test_decode_softcap(dev):
    _run(dev, torch.bfloat16, "int8", 3, 32, 8, 1, [100, 2000, 31], 440, softcap=30.0)


def test_decode_via_kvcache_entry(dev):
    pg = make_paged(2, 8, 128, 16, [48, 32], torch.float16, 450)
    q = randn((2, 32, 1, 128), torch.float16, 451)
    out = fa.flash_attention_kvcache(q.to(dev), pg["k"].to(dev), pg["v"].to(dev), block_table=pg["block_table"].to(dev),
                                     seq_lens=pg["seq_lens"].to(dev))
    O, _ = orc.paged_attention(q, pg["k"], pg["v"], pg["block_table"], pg["seq_lens"], causal=True)
    assert_close(out, O, torch.float16)


def test_gather_route_for_long_queries(dev):
    # (Hq/Hkv)*Nq > 8 -> gather + per-sequence attention, as the reference routes it
    pg = make_paged(2, 2, 128, 16, [48, 100], torch.bfloat16, 460)
    q = randn((2, 8, 16, 128), torch.bfloat16, 461)
    out = fa.flash_attention_paged(q.to(dev), pg["k"].to(dev), pg["v"].to(dev), pg["block_table"].to(dev),
                                   pg["seq_lens"].to(dev), causal=True)
    O, _ = orc.paged_attention(q, pg["k"], pg["v"], pg["block_table"], pg["seq_lens"], causal=True)
    assert_close(out, O, torch.bfloat16)


@pytest.mark.parametrize("quant", [None, "int8", "e4m3"])
@pytest.mark.parametrize("block_size,D", [(16, 128), (32, 128), (64, 64), (16, 64)])
def test_paged_prefill_chunks(dev, quant, block_size, D):
    """Prefill-sized queries over a page pool (chunked prefill): sequences of different length with -1 padding (the
    reference's paged cases, tests/test_attention.py:3812-3857 in the reference), a hole in a table, GQA, causal
    lower-right alignment per sequence, soft cap, lse.  16-bit pools are read through the block table by the forward
    kernel; 8-bit pools are gathered and dequantised first.  Both against the oracle's gather + per-sequence attention."""
    if quant is not None and D == 64 and block_size == 16:
        pytest.skip("one 8-bit head_dim-64 case is enough")
    dtype = torch.bfloat16
    lens = [48, 100, 700, 0, 1030]
    B, Hq, Hkv = len(lens), 8, 2
    pg = make_paged(B, Hkv, D, block_size, lens, dtype, 600, quant=quant)
    table = pg["block_table"].clone()
    table[2, 1] = -1                                   # a hole: its tokens count as zeros
    ks, vs = pg["k_scale"], pg["v_scale"]
    for Nq, causal, softcap in ((16, True, 0.0), (40, True, 30.0), (130, False, 0.0)):
        q = randn((B, Hq, Nq, D), dtype, 601 + Nq)
        out, lse = fa.flash_attention_paged(
            q.to(dev), pg["k"].to(dev), pg["v"].to(dev), table.to(dev), pg["seq_lens"].to(dev), causal=causal,
            block_size=block_size, k_scale=None if ks is None else ks.to(dev), v_scale=None if vs is None else vs.to(dev),
            softcap=softcap, return_lse=True)
        O, L = orc.paged_attention(q, pg["k"], pg["v"], table, pg["seq_lens"], causal=causal, softcap=softcap,
                                   k_scale=ks, v_scale=vs)
        # rows of a causal chunk longer than its sequence see no key: zeros and -inf on both sides
        assert_close(out, O, dtype)
        assert_close(lse, L, dtype, "lse")


@pytest.mark.parametrize("quant", ["int8", "e4m3"])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16])
def test_gather_dequant_is_bit_exact(dev, quant, out_dtype):
    """out = out_dtype(float(x) * float(scale)), one rounding: equal to the oracle's dequantise-then-gather bit for bit."""
    lens = [5, 33, 200]
    pg = make_paged(3, 4, 128, 16, lens, out_dtype, 610, quant=quant)
    got = fa.paged_kv_gather_dequant(pg["k"].to(dev), pg["k_scale"].to(dev), pg["block_table"].to(dev),
                                     pg["seq_lens"].to(dev), 200, out_dtype)
    deq = orc.dequant(pg["k"], pg["k_scale"], out_dtype)
    ref = orc.paged_gather(deq.view(torch.int16).numpy(), pg["block_table"].numpy(), pg["seq_lens"].numpy(), 200)
    assert np.array_equal(got.cpu().view(torch.int16).numpy(), ref)


def test_dense_attention_with_per_sequence_key_counts(dev):
    """kv_lens through the raw forward: each batch entry attends to its own number of keys of a padded dense cache."""
    dtype = torch.float16
    lens = [300, 1, 0, 257]
    q = randn((4, 4, 70, 128), dtype, 620)
    k, v = randn((4, 2, 300, 128), dtype, 621), randn((4, 2, 300, 128), dtype, 622)
    lt = torch.tensor(lens, dtype=torch.int32, device=dev)
    out, lse = A._fwd_raw(q.to(dev), k.to(dev), v.to(dev), 128 ** -0.5, True, 0.0, -1, True, None, kv_lens=lt)
    for b, n in enumerate(lens):
        if n == 0:
            assert not out[b].any() and torch.isinf(lse[b]).all()
            continue
        O, L, _ = orc.sdpa(q[b:b + 1], k[b:b + 1, :, :n], v[b:b + 1, :, :n], causal=True)
        assert_close(out[b:b + 1], O, dtype)
        assert_close(lse[b:b + 1], L, dtype, "lse")


@pytest.mark.parametrize("parts", [2, 3])
def test_packed_partials_and_combine_kernel(dev, parts):
    """What the multi-GPU long-sequence path does, on one GPU: the page list of each sequence is cut into `parts`
    ranges, the decode kernel leaves an fp32 partial with its lse for each range (one packed buffer per range), and the
    combine kernel merges them.  The result must equal the decode of the whole sequences and the oracle.  One range
    is left empty for one sequence (lse = -inf drops out of the combine)."""
    import ctypes as C

    from mlx_flashattention_steel_b200 import _lib
    from mlx_flashattention_steel_b200 import parallel as par

    dtype, D, bs = torch.bfloat16, 128, 16
    lens = [5000, 130, 16]
    B, Hq, Hkv = len(lens), 16, 4
    pg = make_paged(B, Hkv, D, bs, lens, dtype, 630, quant="int8")
    pgd = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in pg.items()}
    q = randn((B, Hq, 1, D), dtype, 631)
    qd = q.to(dev)
    packed = []
    for r in range(parts):
        rows, counts = [], []
        for b, n in enumerate(lens):
            lo, hi, ntok = par.split_pages((n + bs - 1) // bs, parts, r, bs, n)
            rows.append(pg["block_table"][b, lo:hi])
            counts.append(ntok)
        width = max(1, max(len(x) for x in rows))
        tbl = torch.full((B, width), -1, dtype=torch.int32)
        for b, x in enumerate(rows):
            tbl[b, :len(x)] = x
        lt = torch.tensor(counts, dtype=torch.int32)
        pk, _ = A._decode_raw(qd, pgd["k"], pgd["v"], pgd["k_scale"], pgd["v_scale"], tbl.to(dev), lt.to(dev),
                              max(max(counts), 1), D ** -0.5, False, 0.0, bs, True, None, packed=True)
        assert pk.shape == (B * Hq, D + 4) and pk.dtype == torch.float32
        packed.append(pk)
    gathered = torch.stack(packed, dim=0).contiguous()
    out = torch.empty((B * Hq, D), dtype=dtype, device=dev)
    lse = torch.empty((B * Hq,), dtype=torch.float32, device=dev)
    st = _lib.load().b200fa_combine_partials(C.c_void_p(gathered.data_ptr()), parts, B * Hq, D, _lib.BF16,
                                             C.c_void_p(out.data_ptr()), C.c_void_p(lse.data_ptr()),
                                             C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == _lib.OK, _lib.last_error()
    O, L = orc.paged_attention(q, pg["k"], pg["v"], pg["block_table"], pg["seq_lens"], k_scale=pg["k_scale"],
                               v_scale=pg["v_scale"])
    assert_close(out.view(B, Hq, 1, D), O, dtype)
    assert_close(lse.view(B, Hq, 1), L, dtype, "lse")
    # the short sequences leave whole ranges empty: their partial lse must be -inf, not NaN
    assert torch.isinf(gathered[parts - 1, 2 * Hq:, D]).all()


def test_config4_shaped_reduced(dev):
    """Config-4 shape with fewer, shorter sequences: B=24, lens ~ U[512, 6144], int8 KV, bf16 q."""
    rng = np.random.default_rng(4)
    lens = rng.integers(512, 6145, size=24).tolist()
    _run(dev, torch.bfloat16, "int8", 24, 32, 8, 1, lens, 470)


def test_full_size_properties(dev):
    """Config 4 at full size (B=128, lens ~ U[512, 32768]) without the oracle:
    (1) pools holding one constant value v (int8 x * scale) give O = v for every head;
    (2) the int8 kernel agrees with the 16-bit kernel run on the dequantised pools."""
    rng = np.random.default_rng(4)
    B, Hq, Hkv, D, bs = 128, 32, 8, 128, 16
    lens = rng.integers(512, 32769, size=B).astype(np.int32)
    pages_per = (lens + bs - 1) // bs
    P = int(pages_per.sum()) + 8
    perm = rng.permutation(P)
    table = -np.ones((B, int(pages_per.max())), dtype=np.int32)
    pos = 0
    for b in range(B):
        table[b, :pages_per[b]] = perm[pos:pos + pages_per[b]]
        pos += pages_per[b]
    gd = torch.Generator(device=dev).manual_seed(4)
    kq = torch.randint(-127, 128, (P, bs, Hkv, D), generator=gd, device=dev, dtype=torch.int8)
    vq = torch.randint(-127, 128, (P, bs, Hkv, D), generator=gd, device=dev, dtype=torch.int8)
    ksc = (torch.rand((P, bs, Hkv), generator=gd, device=dev) * 0.01 + 0.005).to(torch.float16)
    vsc = (torch.rand((P, bs, Hkv), generator=gd, device=dev) * 0.02 + 0.01).to(torch.float16)
    q = torch.randn((B, Hq, 1, D), generator=gd, device=dev).to(torch.bfloat16)
    tt, lt = torch.from_numpy(table).to(dev), torch.from_numpy(lens).to(dev)
    out = fa.flash_attention_paged(q, kq, vq, tt, lt, causal=True, k_scale=ksc, v_scale=vsc, max_kv_len=int(lens.max()))
    # (2) same pools dequantised to bf16, 16-bit kernel
    kd = (kq.float() * ksc.float().unsqueeze(-1)).to(torch.bfloat16)
    vd = (vq.float() * vsc.float().unsqueeze(-1)).to(torch.bfloat16)
    ref = fa.flash_attention_paged(q, kd, vd, tt, lt, causal=True, max_kv_len=int(lens.max()))
    assert float((out.float() - ref.float()).abs().max()) <= 2e-2
    del kd, vd
    # (1) constant values
    vq.fill_(50)
    vsc.fill_(0.02)
    outc = fa.flash_attention_paged(q, kq, vq, tt, lt, causal=True, k_scale=ksc, v_scale=vsc, max_kv_len=int(lens.max()))
    assert float((outc.float() - 1.0).abs().max()) <= 1e-2
