"""CPU tests of the Python front end: the argument checks and error classes of the
reference's operators (mlx_mfa/attention.py; tests/test_attention.py:96-102, 487-493,
552-558, 795-819, 5120-5156 in the reference) reproduced without a GPU."""
import pytest
import torch

import mlx_flashattention_steel_b200 as fa


def _qkv(B=1, Hq=4, Hkv=4, N=8, S=8, D=64, dtype=torch.float16):
    return (torch.zeros(B, Hq, N, D, dtype=dtype), torch.zeros(B, Hkv, S, D, dtype=dtype),
            torch.zeros(B, Hkv, S, D, dtype=dtype))


def test_public_names():
    for n in ("flash_attention", "flash_attention_varlen", "flash_attention_kvcache", "flash_attention_paged"):
        assert callable(getattr(fa, n))


def test_invalid_backend():
    q, k, v = _qkv()
    with pytest.raises(ValueError, match="backend must be one of"):
        fa.flash_attention(q, k, v, backend="metal")
    with pytest.raises(NotImplementedError):
        fa.flash_attention(q, k, v, backend="sdpa")


def test_rank_and_dim_checks():
    q, k, v = _qkv()
    with pytest.raises(ValueError, match="expects 4-D"):
        fa.flash_attention(q[0], k[0], v[0])
    with pytest.raises(ValueError, match="same head_dim"):
        fa.flash_attention(q, torch.zeros(1, 4, 8, 128, dtype=q.dtype), v)
    with pytest.raises(ValueError, match="divisible"):
        fa.flash_attention(*_qkv(Hq=6, Hkv=4))


def test_unsupported_head_dim_and_options():
    with pytest.raises(NotImplementedError):
        fa.flash_attention(*_qkv(D=96))
    with pytest.raises(RuntimeError, match="unsupported configuration"):
        fa.flash_attention(*_qkv(D=96), backend="mfa")
    q, k, v = _qkv()
    with pytest.raises(ValueError, match="mutually exclusive"):
        fa.flash_attention(q, k, v, return_attn_weights=True, return_lse=True)
    with pytest.raises(NotImplementedError):
        fa.flash_attention(q, k, v, dropout_p=0.1)
    with pytest.raises(NotImplementedError):
        fa.flash_attention(q, k, v, attn_bias=torch.zeros(8, 8))
    with pytest.raises(NotImplementedError, match="right=3"):
        fa.flash_attention(q, k, v, window_size=(4, 3))


def test_no_cpu_path():
    q, k, v = _qkv()
    with pytest.raises(RuntimeError, match="no CPU path"):
        fa.flash_attention(q, k, v)


def test_varlen_checks():
    q, k, v = _qkv()
    cu = torch.tensor([0], dtype=torch.int32)
    assert fa.flash_attention_varlen(q, k, v, cu, cu, 0, 0) is q      # num_seqs == 0 returns q
    cu = torch.tensor([0, 8], dtype=torch.int32)
    with pytest.raises(ValueError, match="block_mask shape"):   # the mask must fit every sequence: [1, 1] for 8 tokens ...
        fa.flash_attention_varlen(q, k, v, cu, cu, 8, 8, block_mask=torch.ones(2, 2))
    with pytest.raises(ValueError, match="batch size 1"):
        fa.flash_attention_varlen(*_qkv(B=2), cu, cu, 8, 8)


def test_kvcache_checks():
    q, k, v = _qkv(N=1)
    table = torch.zeros(1, 2, dtype=torch.int32)
    with pytest.raises(ValueError, match="4-D"):
        fa.flash_attention_kvcache(q[0], k, v)
    with pytest.raises(ValueError, match="requires seq_lens"):
        fa.flash_attention_kvcache(q, k, v, block_table=table)
    with pytest.raises(ValueError, match="window_size is not supported in paged"):
        fa.flash_attention_kvcache(q, k, v, block_table=table, seq_lens=torch.tensor([4]), window_size=(4, 0))
    with pytest.raises(ValueError, match="alibi_slopes is not supported in paged"):
        fa.flash_attention_kvcache(q, k, v, block_table=table, seq_lens=torch.tensor([4]), alibi_slopes=torch.ones(4))
    with pytest.raises(ValueError, match="must both be provided"):
        fa.flash_attention_kvcache(q, k, v, k_new=k)
    with pytest.raises(ValueError, match="not supported in paged mode"):
        fa.flash_attention_kvcache(q, k, v, k_new=k, v_new=v, block_table=table, seq_lens=torch.tensor([4]))
    with pytest.raises(ValueError, match="must be provided in dense mode"):
        fa.flash_attention_kvcache(q, None, None)
    with pytest.raises(ValueError, match="mutually exclusive"):
        fa.flash_attention_kvcache(q, k, v, rotary_cos=torch.ones(1), alibi_slopes=torch.ones(4))


def test_paged_zero_length_returns_zeros():
    # mlx_mfa/attention.py:2875-2876
    q = torch.ones(2, 4, 1, 128, dtype=torch.float16)
    pool = torch.zeros(3, 16, 2, 128, dtype=torch.float16)
    out = fa.flash_attention_paged(q, pool, pool, torch.full((2, 2), -1, dtype=torch.int32),
                                   torch.zeros(2, dtype=torch.int32))
    assert out.shape == q.shape and not out.any()


def test_paged_checks():
    q = torch.ones(2, 4, 1, 128, dtype=torch.float16)
    pool8 = torch.zeros(3, 16, 2, 128, dtype=torch.int8)
    table = torch.zeros(2, 2, dtype=torch.int32)
    lens = torch.tensor([4, 4], dtype=torch.int32)
    with pytest.raises(ValueError, match="need k_scale"):
        fa.flash_attention_paged(q, pool8, pool8, table, lens)
    with pytest.raises(ValueError, match="block_size"):
        fa.flash_attention_paged(q, pool8, pool8, table, lens, block_size=32)
