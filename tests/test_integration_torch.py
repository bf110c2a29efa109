"""The PyTorch SDPA integration (role of mlx_mfa/integrations/mlx_lm.py and the reference's
tests/test_mlx_lm_integration.py: routing rules, fallback, statistics, patch / unpatch idempotence)."""
import pytest
import torch
import torch.nn.functional as F

from mlx_flashattention_steel_b200.integrations import torch_sdpa as integ

from .util import assert_close, randn


def test_cpu_calls_fall_back_and_are_counted():
    integ._reset_stats()
    q = torch.randn(1, 2, 8, 64)
    ref = F.scaled_dot_product_attention(q, q, q, is_causal=True)
    out = integ.scaled_dot_product_attention(q, q, q, is_causal=True)
    assert torch.equal(out, ref)
    st = integ.get_stats()
    assert st["forward_calls"] == 1 and st["fallback_calls"] == 1 and st["steel_calls"] == 0


def test_eligibility_rules():
    q = torch.zeros(1, 4, 16, 128, dtype=torch.bfloat16)
    e = lambda **kw: integ._eligible(kw.get("q", q), kw.get("k", q), kw.get("v", q), kw.get("mask"), kw.get("p", 0.0),
                                     kw.get("causal", False), kw.get("gqa", False))
    assert not e()                                                    # CPU tensors
    assert not e(mask=torch.ones(16, 16, dtype=torch.bool))
    assert not e(p=0.1)


@pytest.mark.gpu
def test_routes_to_the_kernel_and_matches_torch(dev):
    integ._reset_stats()
    q, k, v = (randn((2, 8, 200, 128), torch.bfloat16, 990 + i).to(dev) for i in range(3))
    ref = F.scaled_dot_product_attention(q, k, v, is_causal=True)
    out = integ.scaled_dot_product_attention(q, k, v, is_causal=True)
    assert_close(out, ref.double().cpu(), torch.bfloat16)
    kg = k[:, :2].contiguous()
    out = integ.scaled_dot_product_attention(q, kg, kg, enable_gqa=True)          # GQA, no mask
    ref = F.scaled_dot_product_attention(q, kg, kg, enable_gqa=True)
    assert_close(out, ref.double().cpu(), torch.bfloat16)
    assert integ.get_stats()["steel_calls"] == 2
    # masks, dropout, causal with N != S and mismatched heads without enable_gqa go to the original function
    m = torch.ones(200, 200, dtype=torch.bool, device=dev).tril()
    out = integ.scaled_dot_product_attention(q, k, v, attn_mask=m)
    assert_close(out, F.scaled_dot_product_attention(q, k, v, attn_mask=m).double().cpu(), torch.bfloat16)
    integ.scaled_dot_product_attention(q[:, :, :5], k, v, is_causal=True)
    st = integ.get_stats()
    assert st["fallback_calls"] == 2 and st["forward_calls"] == 4


@pytest.mark.gpu
def test_patch_is_idempotent_and_reversible(dev):
    orig = F.scaled_dot_product_attention
    try:
        assert integ.patch_torch_sdpa(verbose=False) and integ.patch_torch_sdpa(verbose=False)
        assert torch.nn.functional.scaled_dot_product_attention is integ.scaled_dot_product_attention
        q = randn((1, 4, 64, 64), torch.float16, 995).to(dev).requires_grad_(True)
        out = torch.nn.functional.scaled_dot_product_attention(q, q, q, is_causal=True)
        out.sum().backward()                                                     # the CUDA backward runs too
        assert q.grad is not None and integ.get_stats()["steel_calls"] == 1
        mha = torch.nn.MultiheadAttention(64, 4, batch_first=True, device=dev, dtype=torch.float16)
        x = randn((2, 32, 64), torch.float16, 996).to(dev)
        y, _ = mha(x, x, x, need_weights=False)                                  # a stock module keeps working
        assert y.shape == x.shape
    finally:
        integ.unpatch_torch_sdpa()
    assert torch.nn.functional.scaled_dot_product_attention is orig
    integ.unpatch_torch_sdpa()                                                   # a second call is a no-op


@pytest.mark.gpu
def test_hf_attention_interface_shape_contract(dev):
    q, k, v = (randn((1, 4, 50, 64), torch.bfloat16, 997 + i).to(dev) for i in range(3))
    out, w = integ.hf_attention_forward(None, q, k, v, None, is_causal=True)
    assert w is None and out.shape == (1, 50, 4, 64)
    ref = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2)
    assert_close(out, ref.double().cpu(), torch.bfloat16)
    assert isinstance(integ.register_hf_attention(), bool)
