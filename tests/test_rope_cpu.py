"""CPU tests of the rotary-embedding oracle and the 3-D table builder (mlx_mfa/attention.py:319-417, 2128-2210;
the reference's own checks are tests/test_attention.py's TestRoPE classes: rotation by known angles, norm
preservation, interleaved versus split-half layouts, partial rotary_dim)."""
import math

import numpy as np
import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from oracle import sdpa_oracle as orc


def _tables(n, half, theta=10000.0):
    j = torch.arange(half, dtype=torch.float32)
    ang = torch.arange(n, dtype=torch.float32)[:, None] * (theta ** (-2.0 * j / (2 * half)))[None, :]
    return torch.cos(ang), torch.sin(ang)


def test_quarter_turn_and_identity():
    x = torch.tensor([1.0, 2.0, 3.0, 4.0]).reshape(1, 1, 1, 4)
    zero, one = torch.zeros(1, 2), torch.ones(1, 2)
    assert torch.equal(orc.rope(x, one, zero).float(), x)                                  # angle 0
    assert torch.allclose(orc.rope(x, zero, one).float(), torch.tensor([-2.0, 1.0, -4.0, 3.0]).reshape(1, 1, 1, 4))
    assert torch.allclose(orc.rope(x, zero, one, interleaved=False).float(), torch.tensor([-3.0, -4.0, 1.0, 2.0]).reshape(1, 1, 1, 4))


@pytest.mark.parametrize("interleaved", [True, False])
def test_rotation_preserves_norm_and_relative_position(interleaved):
    g = torch.Generator().manual_seed(1)
    cos, sin = _tables(64, 8)
    q = torch.randn((1, 1, 1, 16), generator=g)
    k = torch.randn((1, 1, 1, 16), generator=g)
    r = orc.rope(q.expand(1, 1, 20, 16), cos, sin, offset=3, interleaved=interleaved)
    assert torch.allclose(r.norm(dim=-1), q.double().norm(dim=-1).expand(1, 1, 20), atol=1e-6)
    # q.k after rotation depends only on the distance between their positions
    d1 = (orc.rope(q, cos, sin, 10, interleaved) * orc.rope(k, cos, sin, 4, interleaved)).sum()
    d2 = (orc.rope(q, cos, sin, 30, interleaved) * orc.rope(k, cos, sin, 24, interleaved)).sum()
    assert abs(float(d1 - d2)) < 1e-5


def test_partial_rotary_dim_and_per_batch_offsets():
    g = torch.Generator().manual_seed(2)
    cos, sin = _tables(32, 4)
    x = torch.randn((2, 2, 5, 16), generator=g)
    r = orc.rope(x, cos, sin, offset=[0, 7], rotary_dim=8)
    assert torch.equal(r[..., 8:].float(), x[..., 8:])                                     # tail untouched
    assert torch.allclose(r[1:2], orc.rope(x[1:2], cos, sin, offset=7, rotary_dim=8))
    assert torch.allclose(r[0, :, 0, :8].float(), x[0, :, 0, :8])                          # position 0: identity


def test_3d_tables_bands_and_positions():
    cos, sin = fa.make_rope_3d_tables(3, 4, 2, head_dim=64)
    assert cos.shape == (24, 32) and cos.dtype == torch.float32
    d_h = d_w = (64 // 3) & ~1                                                              # 20, 20, 24
    # token 17 = frame 1, row 1, column 1
    for band, (lo, d, pos) in enumerate(((0, d_h, 1), (d_h // 2, d_w, 1), (d_h // 2 + d_w // 2, 64 - d_h - d_w, 1))):
        j = np.arange(d // 2, dtype=np.float32)
        ang = np.float32(pos) * (1.0 / (10000.0 ** (2.0 * j / d))).astype(np.float32)
        assert np.allclose(cos[17, lo:lo + d // 2].numpy(), np.cos(ang), atol=1e-6)
        assert np.allclose(sin[17, lo:lo + d // 2].numpy(), np.sin(ang), atol=1e-6)
    assert torch.equal(cos[0], torch.ones(32)) and torch.equal(sin[0], torch.zeros(32))
    with pytest.raises(ValueError):
        fa.make_rope_3d_tables(2, 2, 1, d_h=3, d_w=2, d_t=2, head_dim=8)


def test_front_end_argument_rules_without_a_gpu():
    q = torch.zeros((1, 2, 4, 64), dtype=torch.float16)
    with pytest.raises(ValueError):
        fa.flash_attention_rope(q[0], q, q, torch.ones(4, 32), torch.zeros(4, 32))
    with pytest.raises(ValueError):
        fa.flash_attention_rope(q, q, q)                                                   # no tables, no rope_3d
    with pytest.raises(ValueError):
        fa.flash_attention_rope(q, q, q, torch.ones(4, 32), torch.zeros(4, 32), rope_3d={"grid_h": 2, "grid_w": 2})
    with pytest.raises(RuntimeError):
        fa.apply_rope(q, torch.ones(4, 32), torch.zeros(4, 32))                            # CPU tensors: no CPU path
    with pytest.raises(ValueError):
        fa.apply_rope(q, torch.ones(4, 16), torch.zeros(4, 32))
