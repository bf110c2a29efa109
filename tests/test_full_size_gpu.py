"""Oracle parity at the FULL sizes of the five benchmark configurations, on sampled rows.

The kernels run on the whole workload; the CPU oracle is evaluated only on sampled query tiles / sequences, which is
exact because a query row's result depends on its own row of scores alone: for rows [lo, hi) of a causal (and
windowed) problem the keys are cut to [0, hi), which keeps the lower-right alignment (offset = hi - n = lo).
Inputs are generated on the device from a seed (the distributions the configurations name: N(0,1), bf16 / fp16,
int8 pools with f16 scales) and only the sampled slices travel to the host.  Tolerances: 2e-2 max-abs on outputs,
lse and gradients (gradients with the half-ulp allowance of util.grad_bound), float32 1e-5.
"""
import numpy as np
import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from oracle import sdpa_oracle as orc

from .util import LSE_TOL, assert_close, assert_close_grad

pytestmark = pytest.mark.gpu


def _mk(dev, seed):
    gd = torch.Generator(device=dev).manual_seed(seed)
    return lambda shape, dt: torch.randn(shape, generator=gd, device=dev).to(dt)


def _check_rows(out, lse, q, k, v, samples, group, dtype, **kw):
    """samples: (batch, q head, lo, hi).  Oracle on rows [lo, hi) of that head against keys [0, hi + S - N)."""
    off = k.shape[2] - q.shape[2]
    worst = 0.0
    for b, h, lo, hi in samples:
        kvh = h // group
        qs = q[b:b + 1, h:h + 1, lo:hi].cpu()
        ks = k[b:b + 1, kvh:kvh + 1, :hi + off].cpu()
        vs = v[b:b + 1, kvh:kvh + 1, :hi + off].cpu()
        O, L, _ = orc.sdpa(qs, ks, vs, **kw)
        worst = max(worst, assert_close(out[b:b + 1, h:h + 1, lo:hi], O, dtype, f"out[{b},{h},{lo}:{hi}]"))
        assert_close(lse[b:b + 1, h:h + 1, lo:hi], L, dtype, f"lse[{b},{h},{lo}:{hi}]", LSE_TOL[dtype])
    return worst


def test_config2_full_size_sampled_rows(dev):
    """B=4, Hq=32, Hkv=8, N=S=8192, D=128, bf16, causal, softcap 50, lse: first, middle, off-tile-boundary and last
    query tiles of three (batch, head) pairs."""
    mk = _mk(dev, 2)
    q, k, v = mk((4, 32, 8192, 128), torch.bfloat16), mk((4, 8, 8192, 128), torch.bfloat16), mk((4, 8, 8192, 128), torch.bfloat16)
    out, lse = fa.flash_attention(q, k, v, causal=True, softcap=50.0, return_lse=True)
    samples = [(b, h, lo, hi) for (b, h) in ((0, 0), (1, 13), (3, 31))
               for (lo, hi) in ((0, 128), (4000, 4200), (8064, 8192))]
    _check_rows(out, lse, q, k, v, samples, 4, torch.bfloat16, causal=True, softcap=50.0)
    assert fa.kernel_status() == 0


def test_config3_full_size_sampled_rows(dev):
    """B=2, H=16, N=S=32768, D=128, fp16, causal, window (512, 0): rows inside the first window, across the point where
    the window starts to cut, deep inside the sequence and at its end."""
    mk = _mk(dev, 3)
    q, k, v = (mk((2, 16, 32768, 128), torch.float16) for _ in range(3))
    out, lse = fa.flash_attention(q, k, v, causal=True, window_size=(512, 0), return_lse=True)
    samples = [(b, h, lo, hi) for (b, h) in ((0, 0), (1, 7), (1, 15))
               for (lo, hi) in ((0, 128), (448, 704), (16300, 16500), (32640, 32768))]
    _check_rows(out, lse, q, k, v, samples, 1, torch.float16, causal=True, window_left=512)
    assert fa.kernel_status() == 0


def _config5_lens():
    rng = np.random.default_rng(5)
    lens = []
    while sum(lens) < 65536:
        lens.append(int(rng.integers(128, 4097)))
    lens[-1] -= sum(lens) - 65536
    return lens


def test_config5_full_size_forward_and_backward_sampled(dev):
    """65536 packed tokens, lengths ~ U[128, 4096], H=16, D=64, bf16, causal.  Forward: the first and last query tile
    of EVERY sequence (each sequence boundary) for two heads.  Backward: dQ, dK, dV of three whole sequences (the
    longest, the shortest and one in the middle of the pack) for two heads against float64 autograd of the oracle."""
    lens = _config5_lens()
    cu = [0] + list(np.cumsum(lens))
    mk = _mk(dev, 5)
    q, k, v, do = (mk((1, 16, 65536, 64), torch.bfloat16) for _ in range(4))
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
    out = fa.flash_attention_varlen(qg, kg, vg, cu_t, cu_t, max(lens), max(lens), causal=True)
    out.backward(do)
    heads = (0, 11)
    for i, L in enumerate(lens):
        b0 = cu[i]
        for h in heads:
            for lo, hi in ((0, min(128, L)), (max(0, L - 128), L)):
                qs = q[:, h:h + 1, b0 + lo:b0 + hi].cpu()
                ks, vs = k[:, h:h + 1, b0:b0 + hi].cpu(), v[:, h:h + 1, b0:b0 + hi].cpu()
                O, _, _ = orc.sdpa(qs, ks, vs, causal=True)
                assert_close(out[:, h:h + 1, b0 + lo:b0 + hi], O, torch.bfloat16, f"seq {i} head {h} rows {lo}:{hi}")
    order = np.argsort(lens)
    for i in (int(order[-1]), int(order[0]), int(order[len(order) // 2])):
        sl = slice(cu[i], cu[i + 1])
        hs = list(heads)
        dq, dk, dv = orc.backward(q[:, hs, sl].cpu(), k[:, hs, sl].cpu(), v[:, hs, sl].cpu(), do[:, hs, sl].cpu(), causal=True)
        assert_close_grad(qg.grad[:, hs, sl], dq, torch.bfloat16, f"dQ seq {i}")
        assert_close_grad(kg.grad[:, hs, sl], dk, torch.bfloat16, f"dK seq {i}")
        assert_close_grad(vg.grad[:, hs, sl], dv, torch.bfloat16, f"dV seq {i}")
    assert fa.kernel_status() == 0


def test_config4_full_size_sampled_sequences(dev):
    """B=128, Hq=32, Hkv=8, D=128, page 16, seq_lens ~ U[512, 32768], int8 K/V with f16 scales (dequantised values
    ~ N(0,1)), block table = a random permutation of the pool's pages, bf16 q, one query token.  The four longest,
    four shortest and four random sequences are checked against the oracle's gather + dequantise + per-sequence
    attention; their pages are copied out of the device pool into a small pool for the host."""
    rng = np.random.default_rng(4)
    B, Hq, Hkv, D, bs = 128, 32, 8, 128, 16
    lens = rng.integers(512, 32769, size=B).astype(np.int32)
    pages_per = (lens + bs - 1) // bs
    P = int(pages_per.sum()) + 8
    perm = rng.permutation(P)
    table = -np.ones((B, int(pages_per.max())), dtype=np.int32)
    pos = 0
    for b in range(B):
        table[b, :pages_per[b]] = perm[pos:pos + pages_per[b]]
        pos += pages_per[b]
    gd = torch.Generator(device=dev).manual_seed(4)
    pools = {}
    for name in ("k", "v"):
        qx = torch.empty((P, bs, Hkv, D), dtype=torch.int8, device=dev)
        sc = torch.empty((P, bs, Hkv), dtype=torch.float16, device=dev)
        for p0 in range(0, P, 8192):
            x = torch.randn((min(8192, P - p0), bs, Hkv, D), generator=gd, device=dev)
            s = (x.abs().amax(dim=-1) / 127.0).to(torch.float16)
            qx[p0:p0 + x.shape[0]] = (x / s.float().unsqueeze(-1)).round().clamp(-127, 127).to(torch.int8)
            sc[p0:p0 + x.shape[0]] = s
        pools[name] = (qx, sc)
    q = torch.randn((B, Hq, 1, D), generator=gd, device=dev).to(torch.bfloat16)
    tt, lt = torch.from_numpy(table).to(dev), torch.from_numpy(lens).to(dev)
    out, lse = fa.flash_attention_paged(q, pools["k"][0], pools["v"][0], tt, lt, causal=True, k_scale=pools["k"][1],
                                        v_scale=pools["v"][1], max_kv_len=int(lens.max()), return_lse=True)
    order = np.argsort(lens)
    picks = sorted(set(order[-4:].tolist() + order[:4].tolist() + rng.choice(B, 4, replace=False).tolist()))
    for b in picks:
        n = int(pages_per[b])
        pages = torch.from_numpy(table[b, :n].astype(np.int64)).to(dev)
        small = {nm: (pools[nm][0][pages].cpu(), pools[nm][1][pages].cpu()) for nm in ("k", "v")}
        tbl = torch.arange(n, dtype=torch.int32).unsqueeze(0)
        ln = torch.tensor([int(lens[b])], dtype=torch.int32)
        O, L = orc.paged_attention(q[b:b + 1].cpu(), small["k"][0], small["v"][0], tbl, ln, causal=True,
                                   k_scale=small["k"][1], v_scale=small["v"][1])
        assert_close(out[b:b + 1], O, torch.bfloat16, f"sequence {b} (len {int(lens[b])})")
        assert_close(lse[b:b + 1], L, torch.bfloat16, f"lse of sequence {b}")
