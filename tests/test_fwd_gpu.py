"""GPU parity tests of the dense forward against the CPU oracle (2e-2 for f16/bf16,
1e-5 for float32).  Cases follow the reference's own test list
(tests/test_attention.py in the reference: remainders 509-520 and 5632-5651,
cross-attention 522-538, GQA ratios 830-881, softcap 2855-2932, window 4829-4886,
decode rows 1472-1598)."""
import math

import numpy as np
import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from mlx_flashattention_steel_b200 import _lib, attention as fa_attn
from oracle import sdpa_oracle as orc

from .util import LSE_TOL, assert_close, randn

pytestmark = pytest.mark.gpu

DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def _run(dev, dtype, B, Hq, Hkv, N, S, D, seed, **kw):
    q = randn((B, Hq, N, D), dtype, seed)
    k = randn((B, Hkv, S, D), dtype, seed + 1)
    v = randn((B, Hkv, S, D), dtype, seed + 2)
    ws = kw.pop("window_size", None)
    out, lse = fa.flash_attention(q.to(dev), k.to(dev), v.to(dev), return_lse=True, window_size=ws, **kw)
    torch.cuda.synchronize()
    wl = -1 if ws is None else max(ws[0], 0)
    O, L, _ = orc.sdpa(q, k, v, scale=kw.get("scale"), causal=kw.get("causal", False),
                       softcap=kw.get("softcap", 0.0), window_left=wl)
    assert out.dtype == dtype and out.shape == q.shape and lse.dtype == torch.float32
    e = assert_close(out, O, dtype)
    assert_close(lse, L, dtype, "lse", LSE_TOL[dtype])
    return e


@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_basic(dev, dt, D, causal):
    _run(dev, DT[dt], 2, 4, 4, 256, 256, D, 10, causal=causal)


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("N,S", [(37, 40), (1, 257), (4, 300), (5, 256), (129, 129), (200, 77), (64, 1)])
@pytest.mark.parametrize("causal", [False, True])
def test_remainders_and_cross_attention(dev, dt, N, S, causal):
    if causal and N > S:
        pytest.skip("rows without visible keys are covered separately")
    _run(dev, DT[dt], 1, 2, 2, N, S, 128, 20, causal=causal)


@pytest.mark.parametrize("dt", ["f16", "f32"])
@pytest.mark.parametrize("ratio", [2, 4, 8])
def test_gqa(dev, dt, ratio):
    _run(dev, DT[dt], 2, 8, 8 // ratio, 150, 150, 64, 30, causal=True)


def test_mqa(dev):
    _run(dev, torch.bfloat16, 1, 8, 1, 300, 300, 128, 31, causal=True)


@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("cap", [5.0, 50.0])
def test_softcap(dev, dt, cap):
    _run(dev, DT[dt], 1, 4, 2, 200, 200, 128, 40, causal=True, softcap=cap)


@pytest.mark.parametrize("mult", [1.0, 3.0, 6.0, 12.0, 40.0])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_softcap_score_ranges(dev, dt, mult):
    """The tcgen05 kernel evaluates tanh by a polynomial whose degree follows the largest |score/cap| of the
    tile (degree 3, 5, 7, then tanh.approx).  Scaling the scores up walks through every branch, up to
    saturated scores (|score/cap| >> 1)."""
    _run(dev, DT[dt], 1, 4, 2, 384, 512, 128, 45, causal=True, softcap=50.0, scale=mult / math.sqrt(128))
    _run(dev, DT[dt], 1, 2, 2, 256, 256, 64, 46, causal=False, softcap=20.0, scale=mult / math.sqrt(64))


@pytest.mark.parametrize("level", [6.0, 20.0])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_softcap_all_scores_negative(dev, dt, level):
    """Every score of every row sits near -level: the bf16 path takes its reference max from max|score|, an upper
    bound far above the true row max here, and must still produce the same probabilities and lse."""
    dtype = DT[dt]
    g = torch.Generator().manual_seed(47)
    D, N = 128, 256
    u = torch.randn(D, generator=g)
    u = u / u.norm()
    amp = math.sqrt(level * math.sqrt(D))
    q = (amp * u + 0.05 * torch.randn((1, 2, N, D), generator=g)).to(dtype)
    k = (-amp * u + 0.05 * torch.randn((1, 2, N, D), generator=g)).to(dtype)
    v = torch.randn((1, 2, N, D), generator=g).to(dtype)
    out, lse = fa.flash_attention(q.to(dev), k.to(dev), v.to(dev), causal=False, softcap=50.0, return_lse=True)
    O, L, _ = orc.sdpa(q, k, v, causal=False, softcap=50.0)
    assert float(L.max()) < 1.4427 * (math.log(N) - 0.8 * level)      # every score is below -0.8 * level
    assert_close(out, O, dtype)
    assert_close(lse, L, dtype, "lse", LSE_TOL[dtype])


@pytest.mark.parametrize("frac", [0.2, 0.4])
@pytest.mark.parametrize("cap", [100.0, 200.0, 1000.0])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_softcap_large_caps_strongly_negative_rows(dev, dt, cap, frac):
    """Capped scores near -frac * cap with a large cap: the bf16 path's reference max taken from max|score| would sit
    up to 2 * frac * cap * log2(e) binades above the true row max -- beyond the exponent range P is computed in from
    cap ~ 95 -- so the kernel has to fall back to the exact row max there.  A second case mixes rows: half of them
    strongly negative, half near zero, inside the same 64-key tiles."""
    dtype = DT[dt]
    g = torch.Generator().manual_seed(48)
    D, N = 128, 256
    u = torch.randn(D, generator=g)
    u = u / u.norm()
    level = frac * cap                                   # |raw scaled score|; tanh(frac) * cap after the cap
    amp = math.sqrt(level * math.sqrt(D))
    k = (-amp * u + 0.05 * torch.randn((1, 2, N, D), generator=g)).to(dtype)
    v = torch.randn((1, 2, N, D), generator=g).to(dtype)
    q_neg = (amp * u + 0.05 * torch.randn((1, 2, N, D), generator=g)).to(dtype)
    q_mix = q_neg.clone()
    q_mix[:, :, ::2] = (0.05 * torch.randn((1, 2, N // 2, D), generator=g)).to(dtype)     # rows with scores near zero
    for q in (q_neg, q_mix):
        out, lse = fa.flash_attention(q.to(dev), k.to(dev), v.to(dev), causal=False, softcap=cap, return_lse=True)
        O, L, _ = orc.sdpa(q, k, v, causal=False, softcap=cap)
        assert torch.isfinite(L).all() and float(L.min()) < -0.7 * math.tanh(frac) * cap
        assert_close(out, O, dtype)
        assert_close(lse, L, dtype, "lse", LSE_TOL[dtype])


def test_softcap_zero_is_bit_identical(dev):
    # tests/test_attention.py:2869-2886
    q, k, v = (randn((1, 2, 100, 64), torch.float16, 50 + i).to(dev) for i in range(3))
    a = fa.flash_attention(q, k, v, causal=True, softcap=0.0)
    b = fa.flash_attention(q, k, v, causal=True)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dt", ["f16", "f32"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("left", [0, 7, 64, 300])
def test_window(dev, dt, causal, left):
    _run(dev, DT[dt], 1, 2, 2, 333, 333, 128, 60, causal=causal, window_size=(left, 0))


def test_window_cross_lengths(dev):
    _run(dev, torch.bfloat16, 1, 2, 1, 100, 400, 64, 61, causal=True, window_size=(50, -1))


def test_window_none_is_bit_identical(dev):
    # tests/test_attention.py:4870-4886
    q, k, v = (randn((1, 2, 100, 64), torch.bfloat16, 70 + i).to(dev) for i in range(3))
    a = fa.flash_attention(q, k, v, causal=True, window_size=None)
    b = fa.flash_attention(q, k, v, causal=True)
    assert torch.equal(a, b)


def test_decode_row_causal_equals_noncausal(dev):
    # tests/test_attention.py:1472-1487
    q = randn((2, 4, 1, 128), torch.float16, 80).to(dev)
    k = randn((2, 4, 500, 128), torch.float16, 81).to(dev)
    v = randn((2, 4, 500, 128), torch.float16, 82).to(dev)
    assert torch.equal(fa.flash_attention(q, k, v, causal=True), fa.flash_attention(q, k, v, causal=False))


def test_rows_without_visible_keys_are_zero(dev):
    # N > S with causal: the first N - S rows see nothing -> O = 0, L = -inf
    q = randn((1, 2, 40, 64), torch.float16, 90).to(dev)
    k = randn((1, 2, 24, 64), torch.float16, 91).to(dev)
    v = randn((1, 2, 24, 64), torch.float16, 92).to(dev)
    out, lse = fa.flash_attention(q, k, v, causal=True, return_lse=True)
    assert not out[:, :, :16].any()
    assert torch.isinf(lse[:, :, :16]).all() and (lse[:, :, :16] < 0).all()
    O, L, _ = orc.sdpa(q.cpu(), k.cpu(), v.cpu(), causal=True)
    assert_close(out, O, torch.float16)


def test_strided_views_and_scale(dev):
    # head-sliced views (the (batch, kv-head) shards of a larger tensor) run without a copy
    full_q = randn((2, 8, 96, 128), torch.bfloat16, 100)
    full_k = randn((2, 4, 96, 128), torch.bfloat16, 101)
    full_v = randn((2, 4, 96, 128), torch.bfloat16, 102)
    q, k, v = full_q[:, 2:6], full_k[:, 1:3], full_v[:, 1:3]
    out = fa.flash_attention(q.to(dev)[:, :], k.to(dev), v.to(dev), scale=0.05, causal=True)
    gq, gk, gv = full_q.to(dev)[:, 2:6], full_k.to(dev)[:, 1:3], full_v.to(dev)[:, 1:3]
    out2 = fa.flash_attention(gq, gk, gv, scale=0.05, causal=True)
    O, _, _ = orc.sdpa(q, k, v, scale=0.05, causal=True)
    assert_close(out, O, torch.bfloat16)
    assert torch.equal(out, out2)


def test_broadcast_views_match_contiguous(dev):
    """k / v expanded over the batch or the head axis (stride 0) must give what their materialised copies give,
    forward and backward: TMA cannot describe a zero stride, so such views must not reach the tcgen05 kernels
    with a made-up stride."""
    for D in (64, 128):
        q = randn((2, 4, 160, D), torch.bfloat16, 110).to(dev)
        k1 = randn((1, 1, 160, D), torch.bfloat16, 111).to(dev)
        v1 = randn((1, 1, 160, D), torch.bfloat16, 112).to(dev)
        do = randn((2, 4, 160, D), torch.bfloat16, 113).to(dev)
        for shape in ((2, 1, 160, D), (1, 4, 160, D), (2, 4, 160, D), (2, 2, 160, D)):
            res = []
            for contiguous in (False, True):
                qg = q.clone().requires_grad_(True)
                kb, vb = k1.clone().requires_grad_(True), v1.clone().requires_grad_(True)
                qq = qg if shape[0] == 2 else qg[:1]
                ke, ve = kb.expand(shape), vb.expand(shape)
                if contiguous:
                    ke, ve = ke.contiguous(), ve.contiguous()
                out = fa.flash_attention(qq, ke, ve, causal=True)
                out.backward(do[: qq.shape[0]])
                res.append((out.detach().float(), qg.grad.float(), kb.grad.float(), vb.grad.float()))
            for name, a_, b_ in zip(("out", "dq", "dk", "dv"), res[0], res[1]):
                assert float((a_ - b_).abs().max()) <= 2e-2 + 2.0 ** -7 * float(b_.abs().max()), (D, shape, name)
        O, _, _ = orc.sdpa(q.cpu(), k1.expand(2, 4, 160, D).cpu(), v1.expand(2, 4, 160, D).cpu(), causal=True)
        assert_close(fa.flash_attention(q, k1.expand(2, 4, 160, D), v1.expand(2, 4, 160, D), causal=True), O, torch.bfloat16)


def test_golden_vectors(dev):
    import os

    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "sdpa_golden.npz"))
    q, k, v = (torch.from_numpy(z[f"dense_causal_gqa_{t}"]) for t in "qkv")
    out, lse = fa.flash_attention(q.to(dev), k.to(dev), v.to(dev), causal=True, return_lse=True)
    assert_close(out, torch.from_numpy(z["dense_causal_gqa_o"]), torch.float32)
    assert_close(lse, torch.from_numpy(z["dense_causal_gqa_lse"]), torch.float32, "lse", 2e-5)
    q, k, v = (torch.from_numpy(z[f"softcap_window_{t}"]) for t in "qkv")
    for dtype in (torch.float32, torch.bfloat16):
        out = fa.flash_attention(q.to(dev, dtype), k.to(dev, dtype), v.to(dev, dtype), causal=True,
                                 softcap=30.0, window_size=(17, 0))
        if dtype == torch.float32:
            assert_close(out, torch.from_numpy(z["softcap_window_o"]), dtype)
        else:
            O, _, _ = orc.sdpa(q.to(dtype), k.to(dtype), v.to(dtype), causal=True, softcap=30.0, window_left=17)
            assert_close(out, O, dtype)


def test_config1_full_size_fp32(dev):
    """B=1, H=8, N=S=1024, D=128, float32, causal: the reference's CPU-runnable config."""
    _run(dev, torch.float32, 1, 8, 8, 1024, 1024, 128, 1, causal=True)


def test_config2_shaped_slice_bf16(dev):
    """GQA causal bf16 with softcap 50 and lse, one batch and two kv groups of config 2
    at a reduced length the oracle finishes in seconds."""
    _run(dev, torch.bfloat16, 1, 8, 2, 2048, 2048, 128, 2, causal=True, softcap=50.0)


def test_portable_and_tcgen05_kernels_agree(dev):
    """The mma.sync kernel (forced) and the default choice agree within tolerance."""
    q = randn((1, 8, 1024, 128), torch.bfloat16, 110).to(dev)
    k = randn((1, 2, 1024, 128), torch.bfloat16, 111).to(dev)
    v = randn((1, 2, 1024, 128), torch.bfloat16, 112).to(dev)
    a, la = fa.flash_attention(q, k, v, causal=True, return_lse=True)
    old = fa_attn._set_force_flags(_lib.FLAG_FORCE_MMA_SYNC)
    try:
        b, lb = fa.flash_attention(q, k, v, causal=True, return_lse=True)
    finally:
        fa_attn._set_force_flags(old)
    assert float((a.float() - b.float()).abs().max()) <= 2e-2
    assert float((la - lb).abs().max()) <= 2e-2


def test_full_size_linearity_in_v(dev):
    """Size-independent property at config-2 scale (no oracle): attention is linear in V,
    so O(v1 + v2) = O(v1) + O(v2) up to bf16 rounding; and rows of V equal to a constant c
    give O = c exactly up to rounding."""
    B, Hq, Hkv, N, D = 1, 8, 2, 8192, 128
    q = randn((B, Hq, N, D), torch.bfloat16, 120).to(dev)
    k = randn((B, Hkv, N, D), torch.bfloat16, 121).to(dev)
    v1 = randn((B, Hkv, N, D), torch.bfloat16, 122).to(dev)
    v2 = randn((B, Hkv, N, D), torch.bfloat16, 123).to(dev)
    o1 = fa.flash_attention(q, k, v1, causal=True, softcap=50.0).float()
    o2 = fa.flash_attention(q, k, v2, causal=True, softcap=50.0).float()
    o12 = fa.flash_attention(q, k, (v1.float() + v2.float()).to(torch.bfloat16), causal=True, softcap=50.0).float()
    assert float((o12 - (o1 + o2)).abs().max()) <= 4e-2
    ones = torch.full((B, Hkv, N, D), 0.75, dtype=torch.bfloat16, device=dev)
    oc = fa.flash_attention(q, k, ones, causal=True).float()
    assert float((oc - 0.75).abs().max()) <= 1e-2


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("Hq,Hkv,N,S,causal", [(4, 4, 200, 200, True), (4, 2, 70, 333, False), (2, 1, 1, 500, True)])
def test_head_dim_256_forward(dev, dt, Hq, Hkv, N, S, causal):
    """head_dim 256 (the reference's largest kernel size, mlx_mfa/attention.py:30): 16-bit forward (the tcgen05 kernel,
    one CTA per SM); the backward and float32 are refused."""
    _run(dev, DT[dt], 1, Hq, Hkv, N, S, 256, 180, causal=causal)
    _run(dev, DT[dt], 1, Hq, Hkv, N, S, 256, 181, causal=causal, softcap=20.0, window_size=(64, 0))
    q = randn((1, 2, 16, 256), torch.float32, 182).to(dev)
    with pytest.raises(NotImplementedError):
        fa.flash_attention(q, q, q)
    qh = randn((1, 2, 16, 256), DT[dt], 183).to(dev).requires_grad_(True)
    with pytest.raises(NotImplementedError):
        fa.flash_attention(qh, qh, qh).sum().backward()


@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_head_dim_256_long_and_varlen(dev, dt):
    """head_dim 256 over many key tiles (lazy rescale, both S buffers, all four 64-column halves of O), GQA, softcap,
    against the oracle; the tcgen05 kernel against the portable one; packed sequences against per-sequence calls."""
    _run(dev, DT[dt], 2, 4, 2, 700, 700, 256, 184, causal=True)
    _run(dev, DT[dt], 1, 2, 2, 130, 1100, 256, 185, causal=False, softcap=30.0)
    q = randn((1, 4, 900, 256), DT[dt], 186).to(dev)
    k = randn((1, 2, 900, 256), DT[dt], 187).to(dev)
    v = randn((1, 2, 900, 256), DT[dt], 188).to(dev)
    a, la = fa.flash_attention(q, k, v, causal=True, return_lse=True)
    old = fa_attn._set_force_flags(_lib.FLAG_FORCE_MMA_SYNC)
    try:
        b, lb = fa.flash_attention(q, k, v, causal=True, return_lse=True)
    finally:
        fa_attn._set_force_flags(old)
    assert float((a.float() - b.float()).abs().max()) <= 2e-2
    assert float((la - lb).abs().max()) <= 2e-2
    lens = [300, 129, 471]
    cu = torch.tensor([0, 300, 429, 900], dtype=torch.int32, device=dev)
    pv = fa.flash_attention_varlen(q, k, v, cu, cu, max(lens), max(lens), causal=True)
    for i, n in enumerate(lens):
        b0 = int(cu[i])
        ref = fa.flash_attention(q[:, :, b0:b0 + n], k[:, :, b0:b0 + n], v[:, :, b0:b0 + n], causal=True)
        assert float((pv[:, :, b0:b0 + n].float() - ref.float()).abs().max()) <= 2e-2
    assert fa.kernel_status() == 0


@pytest.mark.parametrize("D", [64, 128, 256])
def test_query_tiles_without_any_visible_key(dev, D):
    """Causal with N > S: the first N - S rows see no key and must come out as exact zeros with lse = -inf, in both
    forward kernels.  (The portable kernel reuses its Q tile as the output staging area; a query tile that visits no
    key tile must still wait for every thread's Q copies before it does.)"""
    N, S, Hq, Hkv = 2049, 63, 24, 3
    q = randn((1, Hq, N, D), torch.float16, 190).to(dev)
    k = randn((1, Hkv, S, D), torch.float16, 191).to(dev)
    v = randn((1, Hkv, S, D), torch.float16, 192).to(dev)
    dead = N - S
    for flags in (0, _lib.FLAG_FORCE_MMA_SYNC):
        old = fa_attn._set_force_flags(flags)
        try:
            for _ in range(6):
                o, l = fa.flash_attention(q, k, v, causal=True, return_lse=True)
                assert int((o[:, :, :dead] != 0).sum()) == 0
                assert bool(torch.isinf(l[:, :, :dead]).all()) and bool((l[:, :, :dead] < 0).all())
                assert bool(torch.isfinite(l[:, :, dead:]).all())
        finally:
            fa_attn._set_force_flags(old)
    assert fa.kernel_status() == 0


def test_short_tiles_wait_for_both_pending_accumulations(dev):
    """A query tile with two key tiles can finish its second softmax before the first P.V product has completed;
    the epilogue must then wait for both.  With constant V every output equals that constant whatever the
    probabilities are, so any read of an unfinished accumulator shows.  Many such tiles, mixed with long ones."""
    v_const = 0.75
    for rep in range(8):
        q = randn((1, 8, 8192, 128), torch.bfloat16, 140 + rep).to(dev)
        k = randn((1, 2, 8192, 128), torch.bfloat16, 150 + rep).to(dev)
        v = torch.full((1, 2, 8192, 128), v_const, dtype=torch.bfloat16, device=dev)
        out = fa.flash_attention(q, k, v, causal=True).float()
        assert float((out - v_const).abs().max()) <= 1e-2
        q = randn((16, 8, 128, 128), torch.bfloat16, 160 + rep).to(dev)
        k = randn((16, 2, 128, 128), torch.bfloat16, 170 + rep).to(dev)
        v = torch.full((16, 2, 128, 128), v_const, dtype=torch.bfloat16, device=dev)
        out = fa.flash_attention(q, k, v, causal=True, softcap=30.0).float()
        assert float((out - v_const).abs().max()) <= 1e-2


def test_host_pipeline_overlapping_calls(dev):
    """Calls with join=False follow one another without draining the pipeline; each still returns its own result."""
    gen = torch.Generator().manual_seed(11)
    shapes = ((3, 8, 256, 128), (3, 2, 256, 128))
    reqs = [tuple(torch.randn(sh, generator=gen).to(torch.bfloat16).pin_memory() for sh in (shapes[0], shapes[1], shapes[1]))
            for _ in range(4)]
    outs = [torch.empty(shapes[0], dtype=torch.bfloat16).pin_memory() for _ in reqs]
    lses = [torch.empty(shapes[0][:3], dtype=torch.float32).pin_memory() for _ in reqs]
    pipe = fa.HostPipeline(shapes[0], shapes[1], torch.bfloat16, dev, chunk=1, depth=2, want_lse=True)
    for (q, k, v), o, l in zip(reqs, outs, lses):
        fa.flash_attention_from_host(q, k, v, out=o, lse=l, pipeline=pipe, return_lse=True, causal=True, join=False)
    pipe.join()
    torch.cuda.synchronize()
    for (q, k, v), o, l in zip(reqs, outs, lses):
        ro, rl = fa.flash_attention(q.to(dev), k.to(dev), v.to(dev), causal=True, return_lse=True)
        assert torch.equal(o, ro.cpu())
        assert torch.equal(l, rl.cpu())


def test_host_pipeline_matches_device_call(dev):
    """flash_attention_from_host (chunked, stream-pipelined copies) returns what the device call returns."""
    q = randn((3, 8, 300, 128), torch.bfloat16, 130).pin_memory()
    k = randn((3, 2, 300, 128), torch.bfloat16, 131).pin_memory()
    v = randn((3, 2, 300, 128), torch.bfloat16, 132).pin_memory()
    out, lse = fa.flash_attention_from_host(q, k, v, return_lse=True, causal=True, softcap=30.0, device=dev)
    torch.cuda.synchronize()
    ref, lref = fa.flash_attention(q.to(dev), k.to(dev), v.to(dev), causal=True, softcap=30.0, return_lse=True)
    assert torch.equal(out, ref.cpu()) and torch.equal(lse, lref.cpu())
    with pytest.raises(ValueError):
        fa.flash_attention_from_host(q.to(dev), k, v)


def test_kernel_status_word_stays_clear(dev):
    """The tcgen05 kernels set bit 0 of a device status word only when a bounded wait gives up;
    after a forward and a backward on healthy inputs it reads 0 (and reading clears it)."""
    q = randn((1, 4, 300, 64), torch.bfloat16, 990).to(dev).requires_grad_(True)
    k = randn((1, 2, 300, 64), torch.bfloat16, 991).to(dev).requires_grad_(True)
    v = randn((1, 2, 300, 64), torch.bfloat16, 992).to(dev).requires_grad_(True)
    fa.flash_attention(q, k, v, causal=True).sum().backward()
    assert fa.kernel_status() == 0
    assert fa.kernel_status() == 0
