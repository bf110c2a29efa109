"""Fused QKV / KV wrappers (mlx_mfa/attention.py:3092-3425; tests/test_attention.py's packed-format tests in the
reference): each layout must give exactly what the unpacked call gives on the same values, read in place."""
import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from oracle import sdpa_oracle as orc

from .util import assert_close, randn


def test_argument_rules():
    x = torch.zeros((2, 16, 3 * 4 * 64), dtype=torch.float16)
    with pytest.raises(ValueError):
        fa.flash_attention_qkv_packed(x)                              # flat layout needs num_heads
    with pytest.raises(ValueError):
        fa.flash_attention_qkv_packed(x, num_heads=5)                 # 768 not divisible by 15 heads
    with pytest.raises(ValueError):
        fa.flash_attention_qkv_packed(torch.zeros((2, 4, 16, 2, 64)))
    with pytest.raises(ValueError):
        fa.flash_attention_kv_packed(torch.zeros((2, 4, 16, 64)), torch.zeros((2, 16, 512)))
    with pytest.raises(ValueError):
        fa.flash_attention_kv_packed(torch.zeros((2, 4, 16, 64)), torch.zeros((2, 16, 4, 64)))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_qkv_layouts_match_the_unpacked_call(dev, dtype):
    B, Hq, Hkv, N, D = 2, 4, 2, 200, 64
    flat = randn((B, N, (Hq + 2 * Hkv) * D), dtype, 800).to(dev)
    q = flat[..., :Hq * D].reshape(B, N, Hq, D).permute(0, 2, 1, 3).contiguous()
    k = flat[..., Hq * D:(Hq + Hkv) * D].reshape(B, N, Hkv, D).permute(0, 2, 1, 3).contiguous()
    v = flat[..., (Hq + Hkv) * D:].reshape(B, N, Hkv, D).permute(0, 2, 1, 3).contiguous()
    ref = fa.flash_attention(q, k, v, causal=True)
    out = fa.flash_attention_qkv_packed(flat, causal=True, num_heads=Hq, num_kv_heads=Hkv)
    assert out.shape == (B, Hq, N, D) and torch.equal(out, ref)
    O, _, _ = orc.sdpa(q.cpu(), k.cpu(), v.cpu(), causal=True)
    assert_close(out, O, dtype)
    head_first = randn((B, Hq, N, 3, D), dtype, 801).to(dev)
    out = fa.flash_attention_qkv_packed(head_first, num_kv_heads=Hkv)
    ref = fa.flash_attention(head_first[:, :, :, 0].contiguous(), head_first[:, :Hkv, :, 1].contiguous(), head_first[:, :Hkv, :, 2].contiguous())
    assert torch.equal(out, ref)


@pytest.mark.gpu
def test_kv_and_varlen_layouts(dev):
    dtype = torch.bfloat16
    q = randn((2, 4, 33, 128), dtype, 810).to(dev)
    kv = randn((2, 70, 2 * 2 * 128), dtype, 811).to(dev)
    k = kv[..., :256].reshape(2, 70, 2, 128).permute(0, 2, 1, 3).contiguous()
    v = kv[..., 256:].reshape(2, 70, 2, 128).permute(0, 2, 1, 3).contiguous()
    assert torch.equal(fa.flash_attention_kv_packed(q, kv, num_kv_heads=2), fa.flash_attention(q, k, v))
    kv5 = randn((2, 2, 70, 2, 128), dtype, 812).to(dev)
    assert torch.equal(fa.flash_attention_kv_packed(q, kv5, causal=True),
                       fa.flash_attention(q, kv5[:, :, :, 0].contiguous(), kv5[:, :, :, 1].contiguous(), causal=True))
    # packed sequences [33, 64, 17]
    cu = torch.tensor([0, 33, 97, 114], dtype=torch.int32, device=dev)
    qkv = randn((1, 2, 114, 3, 64), dtype, 813).to(dev)
    ref = fa.flash_attention_varlen(qkv[:, :, :, 0].contiguous(), qkv[:, :, :, 1].contiguous(), qkv[:, :, :, 2].contiguous(), cu, cu, 64, 64, causal=True)
    assert torch.equal(fa.flash_attention_varlen_qkv_packed(qkv, cu, cu, 64, 64, causal=True), ref)
    flat = randn((1, 114, 3 * 2 * 64), dtype, 814).to(dev)
    out = fa.flash_attention_varlen_qkv_packed(flat, cu, cu, 64, 64, num_heads=2)
    qf, kf, vf = (flat[..., i * 128:(i + 1) * 128].reshape(1, 114, 2, 64).permute(0, 2, 1, 3).contiguous() for i in range(3))
    assert torch.equal(out, fa.flash_attention_varlen(qf, kf, vf, cu, cu, 64, 64))
    qv = randn((1, 4, 114, 64), dtype, 815).to(dev)
    kvp = randn((1, 2, 114, 2, 64), dtype, 816).to(dev)
    assert torch.equal(fa.flash_attention_varlen_kv_packed(qv, kvp, cu, cu, 64, 64, causal=True),
                       fa.flash_attention_varlen(qv, kvp[:, :, :, 0].contiguous(), kvp[:, :, :, 1].contiguous(), cu, cu, 64, 64, causal=True))
