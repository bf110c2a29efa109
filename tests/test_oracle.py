"""CPU tests of the oracle itself: analytic known answers, the behaviours the
reference's tests state (tests/test_attention.py in the reference, cited per case),
the C gather against the numpy gather, and the committed golden vectors."""
import ctypes
import math
import os

import numpy as np
import pytest
import torch

from oracle import sdpa_oracle as orc

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def test_uniform_scores_give_mean_of_visible_values():
    # q = 0 -> all scores 0 -> O = mean of the visible V rows, L = log2(count)
    B, H, N, S, D = 1, 2, 5, 7, 8
    q = torch.zeros(B, H, N, D)
    k = torch.randn(B, H, S, D)
    v = torch.randn(B, H, S, D)
    O, L1, L2 = orc.sdpa(q, k, v, causal=True)
    for i in range(N):
        cnt = i + (S - N) + 1
        ref = v[0, :, :cnt].double().mean(dim=1)
        assert torch.allclose(O[0, :, i], ref, atol=1e-12)
        assert torch.allclose(L1[0, :, i], torch.full((H,), math.log2(cnt), dtype=torch.float64), atol=1e-12)
        assert torch.allclose(L2[0, :, i], torch.full((H,), math.log2(cnt), dtype=torch.float64), atol=1e-12)


def test_single_key_returns_its_value():
    q = torch.randn(1, 1, 3, 4)
    k = torch.randn(1, 1, 1, 4)
    v = torch.randn(1, 1, 1, 4)
    O, L1, _ = orc.sdpa(q, k, v)
    assert torch.allclose(O, v.double().expand(1, 1, 3, 4), atol=1e-12)
    s = (q.double() @ k.double().transpose(-1, -2)).squeeze(-1) * 0.5
    assert torch.allclose(L1, s * orc.LOG2E, atol=1e-12)


def test_two_lse_conventions_differ_by_the_documented_factor():
    # kernel convention: log2(e)*logsumexp(s); fallback: log2(sum 2^s)
    s = torch.tensor([0.3, -1.2, 2.0], dtype=torch.float64)
    q = torch.ones(1, 1, 1, 1)
    k = s.view(1, 1, 3, 1).float()
    v = torch.zeros(1, 1, 3, 1)
    _, L1, L2 = orc.sdpa(q, k, v, scale=1.0)
    sf = k.double().view(-1)
    assert abs(float(L1) - math.log2(math.e) * float(torch.logsumexp(sf, 0))) < 1e-12
    assert abs(float(L2) - float(torch.log2(torch.exp2(sf).sum()))) < 1e-12


def test_causal_matches_triu_mask_definition():
    # tests/test_attention.py:32-39 (reference_sdpa): triu(-inf, k = S - N + 1)
    torch.manual_seed(0)
    N, S, D = 6, 9, 16
    q, k, v = torch.randn(1, 2, N, D), torch.randn(1, 2, S, D), torch.randn(1, 2, S, D)
    mask = torch.triu(torch.full((N, S), float("-inf"), dtype=torch.float64), diagonal=S - N + 1)
    s = q.double() @ k.double().transpose(-1, -2) / math.sqrt(D) + mask
    ref = torch.softmax(s, -1) @ v.double()
    O, _, _ = orc.sdpa(q, k, v, causal=True)
    assert torch.allclose(O, ref, atol=1e-12)


def test_softcap_zero_is_identity_and_formula():
    # tests/test_attention.py:2855-2886 (softcap reference; softcap=0 identical)
    torch.manual_seed(1)
    q, k, v = torch.randn(1, 2, 5, 8), torch.randn(1, 2, 5, 8), torch.randn(1, 2, 5, 8)
    O0, _, _ = orc.sdpa(q, k, v, causal=True, softcap=0.0)
    O1, _, _ = orc.sdpa(q, k, v, causal=True)
    assert torch.equal(O0, O1)
    cap = 5.0
    s = q.double() @ k.double().transpose(-1, -2) / math.sqrt(8)
    s = torch.tanh(s / cap) * cap
    s = s + torch.triu(torch.full((5, 5), float("-inf"), dtype=torch.float64), diagonal=1)
    ref = torch.softmax(s, -1) @ v.double()
    Oc, _, _ = orc.sdpa(q, k, v, causal=True, softcap=cap)
    assert torch.allclose(Oc, ref, atol=1e-12)


def test_window_left_only_and_none_is_identity():
    # tests/test_attention.py:4829-4886: in_win = k >= q - left (and k <= q iff causal)
    torch.manual_seed(2)
    N = S = 12
    q, k, v = torch.randn(1, 1, N, 8), torch.randn(1, 1, S, 8), torch.randn(1, 1, S, 8)
    O_none, _, _ = orc.sdpa(q, k, v, causal=True, window_left=-1)
    O_big, _, _ = orc.sdpa(q, k, v, causal=True, window_left=100)
    assert torch.allclose(O_none, O_big, atol=1e-14)
    left = 3
    qi = torch.arange(N).view(-1, 1)
    kj = torch.arange(S).view(1, -1)
    for causal in (False, True):
        vis = kj >= qi - left
        if causal:
            vis = vis & (kj <= qi)
        s = (q.double() @ k.double().transpose(-1, -2) / math.sqrt(8)).masked_fill(~vis, float("-inf"))
        ref = torch.softmax(s, -1) @ v.double()
        O, _, _ = orc.sdpa(q, k, v, causal=causal, window_left=left)
        assert torch.allclose(O, ref, atol=1e-12)


def test_decode_row_causal_equals_noncausal():
    # tests/test_attention.py:1472-1487: N = 1 sees every key either way
    torch.manual_seed(3)
    q, k, v = torch.randn(2, 4, 1, 16), torch.randn(2, 2, 33, 16), torch.randn(2, 2, 33, 16)
    a, _, _ = orc.sdpa(q, k, v, causal=True)
    b, _, _ = orc.sdpa(q, k, v, causal=False)
    assert torch.allclose(a, b, atol=1e-14)


def test_gqa_equals_repeated_kv():
    # tests/test_attention.py:458-460, 843-845
    torch.manual_seed(4)
    q, k, v = torch.randn(1, 8, 7, 16), torch.randn(1, 2, 7, 16), torch.randn(1, 2, 7, 16)
    a, _, _ = orc.sdpa(q, k, v, causal=True)
    b, _, _ = orc.sdpa(q, k.repeat_interleave(4, 1), v.repeat_interleave(4, 1), causal=True)
    assert torch.allclose(a, b, atol=1e-14)


def test_varlen_is_per_sequence():
    # tests/test_attention.py:2254-2272, lengths [33, 64, 17] (2306-2325)
    torch.manual_seed(5)
    lens = [33, 64, 17]
    cu = [0, 33, 97, 114]
    q, k, v = torch.randn(1, 2, 114, 8), torch.randn(1, 2, 114, 8), torch.randn(1, 2, 114, 8)
    O, _ = orc.varlen(q, k, v, cu, cu, causal=True)
    for i in range(3):
        sl = slice(cu[i], cu[i + 1])
        ref, _, _ = orc.sdpa(q[:, :, sl], k[:, :, sl], v[:, :, sl], causal=True)
        assert torch.equal(O[:, :, sl], ref)


def _c_gather():
    path = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(path):
        import subprocess

        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle")])
    return ctypes.CDLL(path)


def test_gather_contract_and_c_restatement():
    # csrc/mfa_paged_gather.cpp:89-129; two sequences of different length with -1 padding
    rng = np.random.default_rng(0)
    P, bs, H, D = 9, 4, 3, 8
    pool = rng.integers(-30000, 30000, size=(P, bs, H, D), dtype=np.int16)
    table = np.array([[5, 2, 7, -1], [3, -1, 1, -1]], dtype=np.int32)
    lens = np.array([11, 9], dtype=np.int32)
    out = orc.paged_gather(pool, table, lens, 12)
    assert out.shape == (2, H, 12, D)
    assert np.array_equal(out[0, :, 0:4], pool[5].transpose(1, 0, 2))
    assert np.array_equal(out[0, :, 8:11], pool[7, :3].transpose(1, 0, 2))
    assert not out[0, :, 11:].any()
    assert not out[1, :, 4:8].any()            # page entry -1 inside the sequence stays zero
    assert np.array_equal(out[1, :, 8:9], pool[1, :1].transpose(1, 0, 2))
    lib = _c_gather()
    cout = np.empty_like(out)
    lib.oracle_paged_gather(pool.ctypes.data_as(ctypes.c_void_p), table.ctypes.data_as(ctypes.c_void_p),
                            lens.ctypes.data_as(ctypes.c_void_p), 2, H, D, 2, bs, 4, 12,
                            cout.ctypes.data_as(ctypes.c_void_p))
    assert np.array_equal(out, cout)


def test_dequant_rounds_to_query_dtype():
    # mlx_mfa/integrations/mlx_lm.py:97-110: dequantise to q.dtype, then dense attention
    x = torch.tensor([[[[-127, 5, 64, 0]]]], dtype=torch.int8)
    sc = torch.tensor([[[0.0123]]], dtype=torch.float16)
    y = orc.dequant(x, sc, torch.bfloat16)
    ref = (x.float() * sc.float().unsqueeze(-1)).to(torch.bfloat16)
    assert y.dtype == torch.bfloat16 and torch.equal(y, ref)


def test_backward_matches_finite_differences():
    torch.manual_seed(6)
    q, k, v = torch.randn(1, 2, 4, 4), torch.randn(1, 1, 4, 4), torch.randn(1, 1, 4, 4)
    do = torch.randn(1, 2, 4, 4)
    dq, dk, dv = orc.backward(q, k, v, do, causal=True)
    eps = 1e-6

    def f(qq, kk, vv):
        o, _, _ = orc.sdpa(qq, kk, vv, causal=True)
        return float((o * do.double()).sum())

    for t, gt in ((q, dq), (k, dk), (v, dv)):
        idx = (0, 0, 1, 2)
        tp = t.double().clone(); tp[idx] += eps
        tm = t.double().clone(); tm[idx] -= eps
        args_p = [tp if x is t else x.double() for x in (q, k, v)]
        args_m = [tm if x is t else x.double() for x in (q, k, v)]
        fd = (f(*args_p) - f(*args_m)) / (2 * eps)
        assert abs(fd - float(gt[idx])) < 1e-6


def test_golden_vectors():
    """Small committed input/output vectors (tests/golden/make_golden.py) pin the
    oracle against silent changes."""
    path = os.path.join(HERE, "golden", "sdpa_golden.npz")
    z = np.load(path)
    for name in ("dense_causal_gqa", "softcap_window"):
        q, k, v = (torch.from_numpy(z[f"{name}_{t}"]) for t in "qkv")
        kw = {}
        if name == "softcap_window":
            kw = dict(softcap=float(z[f"{name}_softcap"]), window_left=int(z[f"{name}_window_left"]))
        O, L1, _ = orc.sdpa(q, k, v, causal=True, **kw)
        assert np.allclose(O.numpy(), z[f"{name}_o"], atol=1e-12)
        assert np.allclose(L1.numpy(), z[f"{name}_lse"], atol=1e-12)


def test_oracle_agrees_with_an_independent_implementation():
    """The oracle restates the reference's formulas; nothing the reference ships can pin it (its CPU arithmetic lives
    in MLX).  An independent implementation at least catches a typo: torch's own CPU scaled_dot_product_attention in
    float64 (masks built here from the definition j <= i + S - N, j >= i + S - N - left) must give the same outputs,
    and autograd through it the same gradients, for causal, windowed, GQA and cross-length cases."""
    import torch.nn.functional as F

    g = torch.Generator().manual_seed(7)
    for (B, Hq, Hkv, N, S, causal, wl) in ((2, 4, 2, 33, 33, True, -1), (1, 6, 3, 20, 47, True, 9), (1, 2, 2, 40, 25, False, -1),
                                           (2, 8, 1, 17, 64, True, 0)):
        q = torch.randn((B, Hq, N, 32), generator=g, dtype=torch.float64)
        k = torch.randn((B, Hkv, S, 32), generator=g, dtype=torch.float64)
        v = torch.randn((B, Hkv, S, 32), generator=g, dtype=torch.float64)
        do = torch.randn((B, Hq, N, 32), generator=g, dtype=torch.float64)
        i = torch.arange(N).unsqueeze(1) + (S - N)
        j = torch.arange(S).unsqueeze(0)
        vis = torch.ones((N, S), dtype=torch.bool)
        if causal:
            vis &= j <= i
        if wl >= 0:
            vis &= j >= i - wl
        rows_ok = vis.any(dim=1)
        qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
        rep = Hq // Hkv
        ref = F.scaled_dot_product_attention(qg, kg.repeat_interleave(rep, 1), vg.repeat_interleave(rep, 1),
                                             attn_mask=vis | ~rows_ok.unsqueeze(1))
        ref = ref * rows_ok.view(1, 1, N, 1)                 # rows without a visible key: zero by this library's convention
        O, _, _ = orc.sdpa(q, k, v, causal=causal, window_left=wl)
        assert float((O - ref.detach()).abs().max()) < 1e-10
        ref.backward(do)
        dq, dk, dv = orc.backward(q, k, v, do, causal=causal, window_left=wl)
        for a, b in ((dq, qg.grad), (dk, kg.grad), (dv, vg.grad)):
            assert float((a - b).abs().max()) < 1e-9
