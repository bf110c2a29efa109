"""GPU parity of the rotary-embedding pass and of the attention routes that use it, against the CPU oracle
(rotation in float64, then the SDPA oracle).  Cases follow the reference's RoPE tests (tests/test_attention.py in
the reference: 1-D tables with cache_seqlens offsets, per-batch offsets, interleaved and split-half layouts, partial
rotary_dim, 3-D tables, the kv-cache routes)."""
import math

import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from oracle import sdpa_oracle as orc

from .util import ULP, assert_close, randn

pytestmark = pytest.mark.gpu


def _tables(n, half, theta=10000.0):
    j = torch.arange(half, dtype=torch.float32)
    ang = torch.arange(n, dtype=torch.float32)[:, None] * (theta ** (-2.0 * j / (2 * half)))[None, :]
    return torch.cos(ang), torch.sin(ang)


def _close_1ulp(got, ref, dtype):
    """float32 arithmetic with one rounding: within one unit in the last place of the storage type."""
    a, b = got.double().cpu(), ref.double()
    assert float(((a - b).abs() - (ULP[dtype] * b.abs() + 1e-6)).max()) <= 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("D,rot", [(128, None), (64, None), (128, 64), (64, 32), (128, 20)])
def test_rotation_kernel(dev, dtype, interleaved, D, rot):
    if not interleaved and rot is not None and rot % 16:
        pytest.skip("split-half mode takes rotary_dim in multiples of 16")
    half = (D if rot is None else rot) // 2
    cos, sin = _tables(300, half)
    x = randn((2, 3, 37, D), dtype, 700)
    got = fa.apply_rope(x.to(dev), cos.to(dev), sin.to(dev), offset=11, interleaved=interleaved, rotary_dim=rot)
    _close_1ulp(got, orc.rope(x, cos, sin, 11, interleaved, rot), dtype)
    got = fa.apply_rope(x.to(dev), cos.to(dev), sin.to(dev), offset=[0, 250], interleaved=interleaved, rotary_dim=rot)
    _close_1ulp(got, orc.rope(x, cos, sin, [0, 250], interleaved, rot), dtype)


def test_rotation_of_a_strided_view_and_table_bounds(dev):
    cos, sin = _tables(64, 64)
    big = randn((2, 4, 50, 128), torch.bfloat16, 701).to(dev)
    view = big[:, 1:3, 8:40]                                   # non-contiguous batch / head / row strides
    got = fa.apply_rope(view, cos.to(dev), sin.to(dev), offset=5)
    _close_1ulp(got, orc.rope(view.cpu(), cos, sin, 5), torch.bfloat16)
    with pytest.raises(ValueError):
        fa.apply_rope(view, cos.to(dev), sin.to(dev), offset=40)            # 40 + 32 > 64 table rows
    with pytest.raises(ValueError):
        fa.apply_rope(view, cos.to(dev), sin.to(dev), offset=[1, 2, 3])


@pytest.mark.parametrize("interleaved", [True, False])
def test_rotation_backward_is_the_inverse_rotation(dev, interleaved):
    cos, sin = _tables(128, 32)
    x = randn((1, 2, 40, 64), torch.float16, 702).to(dev).requires_grad_(True)
    g = randn((1, 2, 40, 64), torch.float16, 703)
    fa.apply_rope(x, cos.to(dev), sin.to(dev), offset=3, interleaved=interleaved).backward(g.to(dev))
    xr = x.detach().cpu().double().requires_grad_(True)
    orc.rope(xr, cos, sin, 3, interleaved).backward(g.double())
    _close_1ulp(x.grad, xr.grad, torch.float16)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal,N,S,cs", [(False, 64, 64, 0), (True, 200, 200, 0), (True, 1, 77, 76), (True, 5, 133, 128)])
def test_attention_with_rope(dev, dtype, causal, N, S, cs):
    cos, sin = _tables(512, 64)
    q, k, v = randn((2, 4, N, 128), dtype, 710), randn((2, 2, S, 128), dtype, 711), randn((2, 2, S, 128), dtype, 712)
    out = fa.flash_attention_rope(q.to(dev), k.to(dev), v.to(dev), cos.to(dev), sin.to(dev), causal=causal, cache_seqlens=cs)
    qr = orc.rope(q, cos, sin, cs).to(dtype)
    kr = orc.rope(k, cos, sin, 0).to(dtype)
    O, _, _ = orc.sdpa(qr, kr, v, causal=causal)
    assert_close(out, O, dtype)


def test_attention_with_per_batch_offsets_and_3d_tables(dev):
    cos, sin = _tables(512, 32)
    q, k, v = randn((3, 2, 1, 64), torch.bfloat16, 720), randn((3, 2, 90, 64), torch.bfloat16, 721), randn((3, 2, 90, 64), torch.bfloat16, 722)
    out = fa.flash_attention_rope(q.to(dev), k.to(dev), v.to(dev), cos.to(dev), sin.to(dev), causal=True, cache_seqlens=[89, 40, 300])
    O, _, _ = orc.sdpa(orc.rope(q, cos, sin, [89, 40, 300]).to(torch.bfloat16), orc.rope(k, cos, sin, 0).to(torch.bfloat16), v, causal=True)
    assert_close(out, O, torch.bfloat16)
    # video tokens: 2 frames of 4 x 6 patches
    q, k, v = (randn((1, 2, 48, 128), torch.float16, 730 + i) for i in range(3))
    out = fa.flash_attention_rope(q.to(dev), k.to(dev), v.to(dev), rope_3d={"grid_h": 4, "grid_w": 6, "num_frames": 2})
    c3, s3 = fa.make_rope_3d_tables(4, 6, 2, head_dim=128)
    O, _, _ = orc.sdpa(orc.rope(q, c3, s3).to(torch.float16), orc.rope(k, c3, s3).to(torch.float16), v)
    assert_close(out, O, torch.float16)


def test_kvcache_routes_with_rotary_tables(dev):
    cos, sin = _tables(256, 64)
    cd, sd = cos.to(dev), sin.to(dev)
    q = randn((1, 4, 1, 128), torch.bfloat16, 740)
    kc, vc = randn((1, 2, 60, 128), torch.bfloat16, 741), randn((1, 2, 60, 128), torch.bfloat16, 742)
    kn, vn = randn((1, 2, 1, 128), torch.bfloat16, 743), randn((1, 2, 1, 128), torch.bfloat16, 744)
    # dense: unrotated cache, q at position 59
    out = fa.flash_attention_kvcache(q.to(dev), kc.to(dev), vc.to(dev), rotary_cos=cd, rotary_sin=sd, cache_seqlens=59)
    O, _, _ = orc.sdpa(orc.rope(q, cos, sin, 59).to(torch.bfloat16), orc.rope(kc, cos, sin, 0).to(torch.bfloat16), vc, causal=True)
    assert_close(out, O, torch.bfloat16)
    # append: the cache holds rotated keys; q and k_new are rotated at position 60
    kc_rot = orc.rope(kc, cos, sin, 0).to(torch.bfloat16)
    out, ku, vu = fa.flash_attention_kvcache(q.to(dev), kc_rot.to(dev), vc.to(dev), k_new=kn.to(dev), v_new=vn.to(dev),
                                             rotary_cos=cd, rotary_sin=sd, cache_seqlens=60)
    kn_rot = orc.rope(kn, cos, sin, 60).to(torch.bfloat16)
    assert ku.shape == (1, 2, 61, 128) and float((ku[:, :, 60:].float().cpu() - kn_rot.float()).abs().max()) <= 2.0 ** -6
    O, _, _ = orc.sdpa(orc.rope(q, cos, sin, 60).to(torch.bfloat16), torch.cat([kc_rot, kn_rot], 2), torch.cat([vc, vn], 2), causal=True)
    assert_close(out, O, torch.bfloat16)
    # paged: rotated keys live in a PagedKVCache, q is rotated at its position
    cache = fa.PagedKVCache(num_blocks=8, block_size=16, H=2, D=128, dtype=torch.bfloat16, device=dev)
    cache.append(kc_rot.to(dev), vc.to(dev), seq_id=0)
    table, lens = cache.block_table_and_seq_lens([0])
    out = fa.flash_attention_kvcache(q.to(dev), cache.k_pool, cache.v_pool, block_table=table, seq_lens=lens,
                                     rotary_cos=cd, rotary_sin=sd, cache_seqlens=59)
    O, _, _ = orc.sdpa(orc.rope(q, cos, sin, 59).to(torch.bfloat16), kc_rot, vc, causal=True)
    assert_close(out, O, torch.bfloat16)
    with pytest.raises(ValueError):
        fa.flash_attention_kvcache(q.to(dev), kc.to(dev), vc.to(dev), rotary_cos=cd)
