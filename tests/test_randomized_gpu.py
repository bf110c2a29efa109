"""Seeded random shapes through both implementations of each path: the tcgen05 kernels (default) against the portable
mma.sync kernels (forced), forward and backward, dense and packed, with the masks and the soft cap drawn at random.
The two families share no device code beyond the helpers, so an edge case that one of them gets wrong shows as a
disagreement; the fixed cases of the other modules pin both to the oracle.  (A run of this kind found the portable
forward's race on query tiles without a visible key.)"""
import random

import numpy as np
import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from mlx_flashattention_steel_b200 import _lib
from mlx_flashattention_steel_b200 import attention as fa_attn

pytestmark = pytest.mark.gpu

TOL = 2e-2


def _both(fn):
    a = fn()
    old = fa_attn._set_force_flags(_lib.FLAG_FORCE_MMA_SYNC)
    try:
        b = fn()
    finally:
        fa_attn._set_force_flags(old)
    return a, b


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-3))


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_forward_kernels_agree_on_random_shapes(dev, seed):
    rnd = random.Random(seed)
    gd = torch.Generator(device=dev).manual_seed(500 + seed)
    for case in range(60):
        D = rnd.choice([64, 128, 128, 256])
        Hkv = rnd.choice([1, 2, 3])
        Hq = Hkv * rnd.choice([1, 1, 2, 4, 8])
        B = rnd.choice([1, 2, 3])
        N = rnd.choice([1, 3, 17, 64, 127, 128, 129, 200, 256, 300, 511, 640, 900, 1300, 2049])
        S = N if rnd.random() < 0.5 else rnd.choice([1, 63, 64, 129, 257, 500, 777, 1024, 1500, 2500])
        kw = dict(causal=rnd.random() < 0.6, softcap=rnd.choice([0.0, 0.0, 30.0, 50.0, 100.0]),
                  window_size=rnd.choice([None, None, (7, 0), (100, 0), (300, -1)]), return_lse=True)
        dt = rnd.choice([torch.bfloat16, torch.float16])
        q, k, v = (torch.randn(s, generator=gd, device=dev).to(dt) for s in ((B, Hq, N, D), (B, Hkv, S, D), (B, Hkv, S, D)))
        (o1, l1), (o2, l2) = _both(lambda: fa.flash_attention(q, k, v, **kw))
        what = f"case {case}: D={D} B={B} Hq={Hq} Hkv={Hkv} N={N} S={S} {kw} {dt}"
        assert not bool(torch.isnan(o1.float()).any()), what
        assert float((o1.float() - o2.float()).abs().max()) <= TOL, what
        fin = torch.isfinite(l2)
        assert torch.equal(torch.isfinite(l1), fin), what
        if bool(fin.any()):
            assert float((l1[fin] - l2[fin]).abs().max()) <= TOL, what
    assert fa.kernel_status() == 0


@pytest.mark.parametrize("seed", [0, 1])
def test_backward_kernels_agree_on_random_shapes(dev, seed):
    """head_dim 128 (the split dK/dV and dQ kernels) and 64 (the fused kernel), dense, with soft cap and window."""
    rnd = random.Random(10 + seed)
    gd = torch.Generator(device=dev).manual_seed(600 + seed)
    for case in range(60):
        D = rnd.choice([64, 128])
        Hkv = rnd.choice([1, 2, 3])
        Hq = Hkv * rnd.choice([1, 1, 2, 4])
        B = rnd.choice([1, 2, 3])
        N = rnd.choice([1, 17, 64, 127, 128, 129, 200, 256, 300, 511, 640, 900, 1300, 2049])
        S = N if rnd.random() < 0.6 else rnd.choice([64, 129, 257, 500, 777, 1024, 1500, 2500])
        causal = rnd.random() < 0.6
        cap = rnd.choice([0.0, 0.0, 30.0, 100.0])
        win = rnd.choice([-1, -1, 7, 100, 300]) if causal or rnd.random() < 0.5 else -1
        dt = rnd.choice([torch.bfloat16, torch.float16])
        q, k, v, do = (torch.randn(s, generator=gd, device=dev).to(dt)
                       for s in ((B, Hq, N, D), (B, Hkv, S, D), (B, Hkv, S, D), (B, Hq, N, D)))
        sc = D ** -0.5
        out, lse = fa_attn._fwd_raw(q, k, v, sc, causal, cap, win, True, None)
        g1, g2 = _both(lambda: fa_attn._bwd_raw(q, k, v, out, lse, do, sc, causal, None, softcap=cap, window_left=win))
        what = f"case {case}: D={D} B={B} Hq={Hq} Hkv={Hkv} N={N} S={S} causal={causal} cap={cap} win={win} {dt}"
        for a, b, name in zip(g1, g2, ("dq", "dk", "dv")):
            assert not bool(torch.isnan(a.float()).any()), f"{what} {name}"
            assert _rel(a, b) <= TOL, f"{what} {name}"
    assert fa.kernel_status() == 0


def test_packed_sequences_agree_on_random_lengths(dev):
    rnd = random.Random(20)
    gd = torch.Generator(device=dev).manual_seed(700)
    for case in range(40):
        D = rnd.choice([64, 128])
        Hkv = rnd.choice([1, 2])
        Hq = Hkv * rnd.choice([1, 2, 4])
        lens = [rnd.choice([1, 5, 63, 64, 65, 127, 128, 129, 200, 300, 513, 900]) for _ in range(rnd.choice([1, 2, 3, 5, 9]))]
        klens = lens if rnd.random() < 0.7 else [rnd.choice([1, 64, 100, 257, 700]) for _ in lens]
        causal = rnd.random() < 0.6
        dt = rnd.choice([torch.bfloat16, torch.float16])
        tq, tk = sum(lens), sum(klens)
        q, k, v, do = (torch.randn(s, generator=gd, device=dev).to(dt)
                       for s in ((1, Hq, tq, D), (1, Hkv, tk, D), (1, Hkv, tk, D), (1, Hq, tq, D)))
        cuq = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=dev)
        cuk = torch.tensor([0] + list(np.cumsum(klens)), dtype=torch.int32, device=dev)

        def fwd_bwd():
            qg, kg, vg = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
            o = fa.flash_attention_varlen(qg, kg, vg, cuq, cuk, max(lens), max(klens), causal=causal)
            o.backward(do)
            return o.detach(), qg.grad, kg.grad, vg.grad

        r1, r2 = _both(fwd_bwd)
        what = f"case {case}: D={D} Hq={Hq} Hkv={Hkv} lens={lens} klens={klens} causal={causal} {dt}"
        for a, b, name in zip(r1, r2, ("out", "dq", "dk", "dv")):
            assert not bool(torch.isnan(a.float()).any()), f"{what} {name}"
            assert _rel(a, b) <= TOL, f"{what} {name}"
    assert fa.kernel_status() == 0
