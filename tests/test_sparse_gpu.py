"""Block-sparse attention against the CPU oracle (block mask expanded to elements), and the mask builders against
their definitions (mlx_mfa/attention.py:717-810, 1219-1311, 1399-1432; the reference's tests compare
flash_attention_sparse with the dense fallback under the expanded mask)."""
import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from mlx_flashattention_steel_b200.sparse import _steel_block_config
from oracle import sdpa_oracle as orc

from .util import assert_close, assert_close_grad, randn


def test_mask_builders_follow_their_definitions():
    assert _steel_block_config(64) == (32, 32) and _steel_block_config(128) == (32, 16)
    m = fa.make_causal_block_mask(100, 128)                          # 4 query blocks of 32, 7 key blocks of 16
    assert m.shape == (4, 7) and m.dtype == torch.bool
    for qb in range(4):
        for kb in range(7):
            assert bool(m[qb, kb]) == (kb * 16 <= (qb + 1) * 32 - 1)
    w = fa.make_sliding_window_mask(256, 40, head_dim=64)            # 8 x 8 cells of 32 x 32
    for qb in range(8):
        c = qb * 32 + 16
        for kb in range(8):
            assert bool(w[qb, kb]) == ((kb * 32 + 31 >= c - 40) and (kb * 32 <= c + 40))
    wc = fa.make_sliding_window_mask(256, 40, head_dim=64, causal=True)
    assert bool((wc <= w).all()) and not bool(wc[0, 1])


def test_argument_rules():
    q = torch.zeros((1, 2, 64, 128), dtype=torch.float16)
    with pytest.raises(ValueError):
        fa.flash_attention_sparse(q, q, q, torch.ones((2, 3), dtype=torch.bool))          # wrong grid: expects [2, 4]
    with pytest.raises(ValueError):
        fa.flash_attention_sparse(q.float(), q.float(), q.float(), torch.ones((2, 4), dtype=torch.bool))
    with pytest.raises(ValueError):
        fa.flash_attention_sparse(q, q, q, torch.ones((8,), dtype=torch.bool))
    with pytest.raises(RuntimeError):
        fa.flash_attention_sparse(q, q, q, torch.ones((2, 4), dtype=torch.bool))          # host tensors: no CPU path


def _random_mask(NQ, NK, seed, density=0.4):
    g = torch.Generator().manual_seed(seed)
    m = torch.rand((NQ, NK), generator=g) < density
    m[:, 0] |= True                                                   # every row sees something ...
    return m


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,N,S,D,causal", [(4, 4, 256, 256, 128, False), (4, 2, 200, 200, 128, True),
                                                  (2, 2, 300, 300, 64, True), (4, 1, 96, 500, 128, False)])
def test_sparse_forward(dev, dtype, Hq, Hkv, N, S, D, causal):
    BQ, BK = _steel_block_config(D)
    NQ, NK = (N + BQ - 1) // BQ, (S + BK - 1) // BK
    mask = _random_mask(NQ, NK, 950 + N)
    if NQ > 2:
        mask[2] = False                                               # ... except one block row: those rows give zeros
        mask[1, 4:] = False                                           # and one that skips whole key tiles
    q, k, v = randn((2, Hq, N, D), dtype, 951), randn((2, Hkv, S, D), dtype, 952), randn((2, Hkv, S, D), dtype, 953)
    out = fa.flash_attention_sparse(q.to(dev), k.to(dev), v.to(dev), mask.to(dev), causal=causal)
    O, _, _ = orc.sdpa(q, k, v, causal=causal, block_mask=mask, block=(BQ, BK))
    assert_close(out, O, dtype)
    if NQ > 2:
        assert float(out[:, :, 2 * BQ:3 * BQ].abs().max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("D,density", [(128, 0.05), (64, 0.3)])
def test_sparse_forward_long_rows(dev, D, density):
    """More than 32 key tiles per query tile (the active-tile list is built in several rounds), low density so that most
    tiles are skipped, lse checked as well."""
    BQ, BK = _steel_block_config(D)
    N = S = 4096 + 40
    NQ, NK = (N + BQ - 1) // BQ, (S + BK - 1) // BK
    mask = _random_mask(NQ, NK, 990, density=density)
    mask[5] = False
    q, k, v = randn((1, 2, N, D), torch.bfloat16, 991), randn((1, 1, S, D), torch.bfloat16, 992), randn((1, 1, S, D), torch.bfloat16, 993)
    out = fa.flash_attention_sparse(q.to(dev), k.to(dev), v.to(dev), mask.to(dev), causal=True)
    O, _, _ = orc.sdpa(q, k, v, causal=True, block_mask=mask, block=(BQ, BK))
    assert_close(out, O, torch.bfloat16)
    assert float(out[:, :, 5 * BQ:6 * BQ].abs().max()) == 0.0


@pytest.mark.gpu
def test_builders_reproduce_dense_causal_and_window(dev):
    """A causal block mask plus causal=True is exactly causal attention; the sliding-window cells bound the keys seen."""
    q, k, v = (randn((1, 2, 320, 128), torch.bfloat16, 960 + i).to(dev) for i in range(3))
    cm = fa.make_causal_block_mask(320, 128, device=dev)
    a = fa.flash_attention_sparse(q, k, v, cm, causal=True)
    b = fa.flash_attention(q, k, v, causal=True)
    assert float((a.float() - b.float()).abs().max()) <= 2e-2
    wm = fa.make_sliding_window_mask(320, 48, 128, causal=True)
    out = fa.flash_attention_sparse(q, k, v, wm.to(dev), causal=True)
    O, _, _ = orc.sdpa(q.cpu(), k.cpu(), v.cpu(), causal=True, block_mask=wm, block=(32, 16))
    assert_close(out, O, torch.bfloat16)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128])
def test_sparse_backward(dev, dtype, D):
    BQ, BK = _steel_block_config(D)
    N = S = 160
    mask = _random_mask((N + BQ - 1) // BQ, (S + BK - 1) // BK, 970)
    mask[3] = False
    q, k, v, do = (randn(shape, dtype, 971 + i) for i, shape in enumerate(((1, 4, N, D), (1, 2, S, D), (1, 2, S, D), (1, 4, N, D))))
    qg, kg, vg = (x.to(dev).requires_grad_(True) for x in (q, k, v))
    fa.flash_attention_sparse(qg, kg, vg, mask.to(dev), causal=True).backward(do.to(dev))
    qr, kr, vr = (x.double().requires_grad_(True) for x in (q, k, v))
    O, _, _ = orc.sdpa(qr, kr, vr, causal=True, block_mask=mask, block=(BQ, BK))
    O.backward(do.double())
    assert_close_grad(qg.grad, qr.grad, dtype, "dQ")
    assert_close_grad(kg.grad, kr.grad, dtype, "dK")
    assert_close_grad(vg.grad, vr.grad, dtype, "dV")
    assert float(qg.grad[:, :, 3 * BQ:4 * BQ].abs().max()) == 0.0      # rows with no active cell get no gradient


@pytest.mark.gpu
def test_varlen_with_a_block_mask(dev):
    """flash_attention_varlen(block_mask=...): one mask that fits every sequence, applied per sequence -- the
    reference's split / concatenate route (mlx_mfa/attention.py:2365-2390, 2448-2453).  Sequences of 113 to 128
    tokens share the [4, 8] cell grid of head_dim 128; forward and gradients against the oracle per sequence."""
    D, dtype = 128, torch.bfloat16
    BQ, BK = _steel_block_config(D)
    lens = [120, 128, 113]
    cu = [0, 120, 248, 361]
    mask = _random_mask(4, 8, 970, density=0.5)
    q, k, v, do = (randn((1, 4, 361, D), dtype, 971 + i) for i in range(4))
    k, v = k[:, :2].contiguous(), v[:, :2].contiguous()
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    qg, kg, vg = (x.to(dev).requires_grad_(True) for x in (q, k, v))
    out = fa.flash_attention_varlen(qg, kg, vg, cu_t, cu_t, 128, 128, causal=True, block_mask=mask.to(dev))
    out.backward(do.to(dev))
    for i, n in enumerate(lens):
        sl = slice(cu[i], cu[i + 1])
        O, _, _ = orc.sdpa(q[:, :, sl], k[:, :, sl], v[:, :, sl], causal=True, block_mask=mask, block=(BQ, BK))
        assert_close(out[:, :, sl], O, dtype)
    assert qg.grad.shape == q.shape and torch.isfinite(qg.grad.float()).all() and torch.isfinite(kg.grad.float()).all()


@pytest.mark.gpu
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("feature", ["alibi", "block_mask", "both"])
def test_feature_backward_tcgen05_and_portable_kernels_agree(dev, D, feature):
    """ALiBi and block-masked gradients run the tcgen05 backward kernels (head_dim 64: one kernel; 128: dK/dV + dQ
    kernels); forcing the mma.sync kernel must give the same gradients within tolerance, with different bits."""
    from mlx_flashattention_steel_b200 import _lib, attention as A

    dtype = torch.bfloat16
    B, Hq, Hkv, N = 2, 4, 2, 300
    BQ, BK = _steel_block_config(D)
    mask = _random_mask((N + BQ - 1) // BQ, (N + BK - 1) // BK, 980, density=0.5).to(dev)
    slopes = torch.tensor([0.5, 0.25, 0.125, 0.0625], device=dev)
    q, k, v, do = (randn((B, Hq, N, D), dtype, 981 + i).to(dev) for i in range(4))
    k, v = k[:, :Hkv].contiguous(), v[:, :Hkv].contiguous()

    def grads():
        qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
        bm = (mask.to(torch.uint8).contiguous(), BQ, BK) if feature in ("block_mask", "both") else None
        al = slopes if feature in ("alibi", "both") else None
        out, _ = A._FlashAttnFn.apply(qg, kg, vg, D ** -0.5, True, 0.0, -1, False, None, al, bm)
        out.backward(do)
        return qg.grad.float(), kg.grad.float(), vg.grad.float()

    g1 = grads()
    old = A._set_force_flags(_lib.FLAG_FORCE_MMA_SYNC)
    try:
        g2 = grads()
    finally:
        A._set_force_flags(old)
    differs = False
    for a, b in zip(g1, g2):
        assert float((a - b).abs().max()) <= 2e-2 + 2.0 ** -7 * float(b.abs().max())
        differs = differs or not torch.equal(a, b)
    assert differs
    assert fa.kernel_status() == 0
