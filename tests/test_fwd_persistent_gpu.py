"""The forward kernel with persistent CTAs (each CTA walks many query tiles; barriers, rings and TMEM live across
them) against the oracle.  The launcher picks that mode for shapes with few key tiles per query tile and many query
tiles (large packed-sequence launches); here it is forced through the descriptor flag on shapes small enough
for the CPU oracle yet with more items than resident CTAs, so that every CTA goes through several items, including
items without any visible key and query tiles beyond a packed sequence's end."""
import numpy as np
import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from mlx_flashattention_steel_b200 import _lib, attention as A
from oracle import sdpa_oracle as orc

from .util import LSE_TOL, assert_close, randn

pytestmark = pytest.mark.gpu


@pytest.fixture
def persistent():
    old = A._set_force_flags(_lib.FLAG_FWD_PERSISTENT)
    yield
    A._set_force_flags(old)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("kw", [dict(causal=True), dict(causal=True, window_size=(100, 0)), dict(causal=False),
                                dict(causal=True, softcap=30.0, window_size=(300, 0))])
def test_persistent_dense(dev, persistent, dtype, D, kw):
    B, Hq, Hkv, N, S = 3, 32, 8, 600, 650            # 5 query tiles x 96 heads = 480 items on at most 296 CTAs
    q, k, v = randn((B, Hq, N, D), dtype, 800), randn((B, Hkv, S, D), dtype, 801), randn((B, Hkv, S, D), dtype, 802)
    out, lse = fa.flash_attention(q.to(dev), k.to(dev), v.to(dev), return_lse=True, **kw)
    ws = kw.get("window_size")
    O, L, _ = orc.sdpa(q, k, v, causal=kw.get("causal", False), softcap=kw.get("softcap", 0.0),
                       window_left=-1 if ws is None else ws[0])
    assert_close(out, O, dtype)
    assert_close(lse, L, dtype, "lse", LSE_TOL[dtype])
    assert fa.kernel_status() == 0


def test_persistent_matches_one_item_per_cta_bitwise(dev, persistent):
    """Same arithmetic in the same order: the two launch modes must give identical bits."""
    q, k, v = (randn((2, 64, 700, 128), torch.bfloat16, 810 + i).to(dev) for i in range(3))
    k, v = k[:, :16].contiguous(), v[:, :16].contiguous()
    a, la = fa.flash_attention(q, k, v, causal=True, window_size=(200, 0), softcap=50.0, return_lse=True)
    A._set_force_flags(_lib.FLAG_FWD_ONE_ITEM)
    b, lb = fa.flash_attention(q, k, v, causal=True, window_size=(200, 0), softcap=50.0, return_lse=True)
    assert torch.equal(a, b) and torch.equal(la, lb)


def test_persistent_rows_without_keys_and_short_tiles(dev, persistent):
    # N > S with a causal mask: the first query tiles see no key at all (zero rows, lse = -inf), later ones a few
    q = randn((2, 96, 520, 64), torch.float16, 820)
    k, v = randn((2, 96, 130, 64), torch.float16, 821), randn((2, 96, 130, 64), torch.float16, 822)
    out, lse = fa.flash_attention(q.to(dev), k.to(dev), v.to(dev), causal=True, return_lse=True)
    O, L, _ = orc.sdpa(q, k, v, causal=True)
    assert_close(out, O, torch.float16)
    assert_close(lse, L, torch.float16, "lse", LSE_TOL[torch.float16])


@pytest.mark.parametrize("D,dtype", [(64, torch.bfloat16), (128, torch.float16)])
def test_persistent_varlen(dev, persistent, D, dtype):
    rng = np.random.default_rng(8)
    lens = [int(x) for x in rng.integers(1, 700, size=12)] + [128, 256, 1]
    cu = [0] + list(np.cumsum(lens))
    T = cu[-1]
    q, k, v = randn((1, 8, T, D), dtype, 830), randn((1, 4, T, D), dtype, 831), randn((1, 4, T, D), dtype, 832)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    out = fa.flash_attention_varlen(q.to(dev), k.to(dev), v.to(dev), cu_t, cu_t, max(lens), max(lens), causal=True)
    O, _ = orc.varlen(q, k, v, cu, cu, causal=True)
    assert_close(out, O, dtype)
    assert fa.kernel_status() == 0
