"""ALiBi (per-head linear position bias) against the CPU oracle: forward for f16 / bf16 / f32, GQA, cross lengths,
with causal masks and softcap, and the backward through float64 autograd of the oracle
(mlx_mfa/attention.py:77-81, 1774-1822, 1883-1928; csrc/mfa_steel_fwd.cpp:951-970; the reference's own checks
compare the kernel with _alibi_sdpa_ref)."""
import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from oracle import sdpa_oracle as orc

from .util import LSE_TOL, assert_close, assert_close_grad, randn

pytestmark = pytest.mark.gpu


def _slopes(H):
    return torch.tensor([2.0 ** (-8.0 * (i + 1) / H) for i in range(H)], dtype=torch.float32)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("Hq,Hkv,N,S,D,causal", [(4, 4, 200, 200, 128, True), (8, 2, 130, 130, 64, True),
                                                  (4, 2, 64, 300, 128, False), (4, 1, 1, 257, 128, True)])
def test_alibi_forward(dev, dtype, Hq, Hkv, N, S, D, causal):
    q, k, v = randn((2, Hq, N, D), dtype, 900), randn((2, Hkv, S, D), dtype, 901), randn((2, Hkv, S, D), dtype, 902)
    sl = _slopes(Hq)
    out, lse = fa.flash_attention(q.to(dev), k.to(dev), v.to(dev), causal=causal, alibi_slopes=sl.to(dev), return_lse=True)
    O, L, _ = orc.sdpa(q, k, v, causal=causal, alibi_slopes=sl)
    assert_close(out, O, dtype)
    assert_close(lse, L, dtype, "lse", LSE_TOL[dtype])
    # the bias matters: without it the result differs
    plain = fa.flash_attention(q.to(dev), k.to(dev), v.to(dev), causal=causal)
    if S > 1:
        assert float((plain.float() - out.float()).abs().max()) > 1e-3


def test_alibi_with_softcap_and_window(dev):
    q, k, v = (randn((1, 4, 150, 128), torch.bfloat16, 910 + i) for i in range(3))
    sl = _slopes(4)
    out = fa.flash_attention(q.to(dev), k.to(dev), v.to(dev), causal=True, softcap=30.0, window_size=(40, 0), alibi_slopes=sl.to(dev))
    O, _, _ = orc.sdpa(q, k, v, causal=True, softcap=30.0, window_left=40, alibi_slopes=sl)
    assert_close(out, O, torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,N,S,D", [(4, 4, 100, 100, 64), (4, 2, 70, 150, 128)])
def test_alibi_backward(dev, dtype, Hq, Hkv, N, S, D):
    q, k, v, do = (randn(shape, dtype, 920 + i) for i, shape in enumerate(((1, Hq, N, D), (1, Hkv, S, D), (1, Hkv, S, D), (1, Hq, N, D))))
    sl = _slopes(Hq)
    qg, kg, vg = (x.to(dev).requires_grad_(True) for x in (q, k, v))
    fa.flash_attention(qg, kg, vg, causal=True, alibi_slopes=sl.to(dev)).backward(do.to(dev))
    qr, kr, vr = (x.double().requires_grad_(True) for x in (q, k, v))
    O, _, _ = orc.sdpa(qr, kr, vr, causal=True, alibi_slopes=sl)
    O.backward(do.double())
    assert_close_grad(qg.grad, qr.grad, dtype, "dQ")
    assert_close_grad(kg.grad, kr.grad, dtype, "dK")
    assert_close_grad(vg.grad, vr.grad, dtype, "dV")


def test_alibi_argument_rules(dev):
    q = randn((1, 4, 16, 64), torch.float16, 930).to(dev)
    with pytest.raises(ValueError):
        fa.flash_attention(q, q, q, alibi_slopes=torch.ones(3, device=dev))
    with pytest.raises(RuntimeError):
        fa.flash_attention(q, q, q, alibi_slopes=torch.ones(4))              # slopes on the host
    out = fa.flash_attention_kvcache(q, q, q, alibi_slopes=_slopes(4).to(dev))  # dense cache route forwards them
    O, _, _ = orc.sdpa(q.cpu(), q.cpu(), q.cpu(), causal=True, alibi_slopes=_slopes(4))
    assert_close(out, O, torch.float16)
