"""GPU parity: packed varlen forward against the per-sequence oracle, and the page
gather bit-exact against both the numpy and the plain-C restatement."""
import ctypes
import os

import numpy as np
import pytest
import torch

import mlx_flashattention_steel_b200 as fa
from oracle import sdpa_oracle as orc

from .util import LSE_TOL, assert_close, make_paged, randn

pytestmark = pytest.mark.gpu


def _cu(lens):
    return [0] + list(np.cumsum(lens))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("lens,D", [([33, 64, 17], 64), ([1, 128, 129, 5], 128), ([300], 64)])
def test_varlen_forward(dev, dtype, causal, lens, D):
    cu = _cu(lens)
    T = cu[-1]
    q, k, v = (randn((1, 4, T, D), dtype, 200 + i) for i in range(3))
    k, v = k[:, :2], v[:, :2]
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    out = fa.flash_attention_varlen(q.to(dev), k.to(dev), v.to(dev), cu_t, cu_t, max(lens), max(lens), causal=causal)
    O, _ = orc.varlen(q, k, v, cu, cu, causal=causal)
    assert_close(out, O, dtype)


def test_varlen_different_q_and_k_lengths(dev):
    lens_q, lens_k = [5, 70, 1], [64, 70, 33]
    cu_q, cu_k = _cu(lens_q), _cu(lens_k)
    q = randn((1, 2, cu_q[-1], 128), torch.bfloat16, 210)
    k = randn((1, 2, cu_k[-1], 128), torch.bfloat16, 211)
    v = randn((1, 2, cu_k[-1], 128), torch.bfloat16, 212)
    out = fa.flash_attention_varlen(q.to(dev), k.to(dev), v.to(dev), torch.tensor(cu_q, dtype=torch.int32, device=dev),
                                    torch.tensor(cu_k, dtype=torch.int32, device=dev), max(lens_q), max(lens_k), causal=True)
    O, _ = orc.varlen(q, k, v, cu_q, cu_k, causal=True)
    assert_close(out, O, torch.bfloat16)


def test_varlen_config5_shaped(dev):
    """Config-5 shape at reduced total: lengths ~ U{128..4096}, H=16 -> 4, D=64, bf16, causal."""
    rng = np.random.default_rng(5)
    lens = []
    while sum(lens) < 8192:
        lens.append(int(rng.integers(128, 2049)))
    lens[-1] -= sum(lens) - 8192
    cu = _cu(lens)
    q, k, v = (randn((1, 4, 8192, 64), torch.bfloat16, 220 + i) for i in range(3))
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    out = fa.flash_attention_varlen(q.to(dev), k.to(dev), v.to(dev), cu_t, cu_t, max(lens), max(lens), causal=True)
    O, _ = orc.varlen(q, k, v, cu, cu, causal=True)
    assert_close(out, O, torch.bfloat16)


@pytest.mark.parametrize("dtype,D,H", [(torch.float16, 128, 2), (torch.bfloat16, 64, 3), (torch.int8, 128, 8), (torch.float32, 64, 1)])
def test_gather_bit_exact(dev, dtype, D, H):
    lens = [48, 32, 1, 0, 77]
    pg = make_paged(len(lens), H, D, 16, lens, torch.float16, 300)
    if dtype == torch.int8:
        pool = torch.randint(-128, 128, pg["k"].shape, dtype=torch.int8)
    else:
        pool = pg["k"].to(dtype)
    table = pg["block_table"].clone()
    table[4, 2] = -1                        # a hole inside a sequence stays zero
    max_len = 80
    out = fa.paged_kv_gather(pool.to(dev), table.to(dev), pg["seq_lens"].to(dev), max_len)
    torch.cuda.synchronize()
    view = {1: torch.int8, 2: torch.int16, 4: torch.int32}[pool.element_size()]
    ref = orc.paged_gather(pool.view(view).numpy(), table.numpy(), pg["seq_lens"].numpy(), max_len)
    got = out.cpu().view(view).numpy()
    assert np.array_equal(got, ref)
    lib = ctypes.CDLL(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "liboracle.so"))
    cref = np.empty_like(ref)
    p = np.ascontiguousarray(pool.view(view).numpy())
    t = np.ascontiguousarray(table.numpy())
    l = np.ascontiguousarray(pg["seq_lens"].numpy())
    lib.oracle_paged_gather(p.ctypes.data_as(ctypes.c_void_p), t.ctypes.data_as(ctypes.c_void_p),
                            l.ctypes.data_as(ctypes.c_void_p), len(lens), H, D, pool.element_size(), 16,
                            table.shape[1], max_len, cref.ctypes.data_as(ctypes.c_void_p))
    assert np.array_equal(got, cref)


def test_gather_large_offsets(dev):
    """Pool beyond 2^31 bytes: offsets are 64-bit (the reference indexes with int)."""
    P, bs, H, D = 70000, 16, 8, 128            # 1.15e9 int16 elements = 2.3 GB
    pool = torch.empty((P, bs, H, D), dtype=torch.int16, device=dev)
    pool.view(-1)[:] = torch.arange(pool.numel(), device=dev, dtype=torch.int64).to(torch.int16)
    table = torch.tensor([[P - 1, 3], [P - 2, -1]], dtype=torch.int32, device=dev)
    lens = torch.tensor([20, 16], dtype=torch.int32, device=dev)
    out = fa.paged_kv_gather(pool, table, lens, 32)
    assert torch.equal(out[0, :, :16], pool[P - 1].permute(1, 0, 2))
    assert torch.equal(out[0, :, 16:20], pool[3, :4].permute(1, 0, 2))
    assert torch.equal(out[1, :, :16], pool[P - 2].permute(1, 0, 2))
    assert not out[0, :, 20:].any() and not out[1, :, 16:].any()


@pytest.mark.parametrize("D", [64, 128])
def test_varlen_tcgen05_and_portable_kernels_agree(dev, D):
    """Packed varlen through the default (tcgen05) kernel and through the forced mma.sync kernel."""
    from mlx_flashattention_steel_b200 import _lib, attention as A

    lens = [700, 129, 1, 64, 1300, 257]
    cu = _cu(lens)
    q, k, v = (randn((1, 8, cu[-1], D), torch.bfloat16, 230 + i).to(dev) for i in range(3))
    k, v = k[:, :2].contiguous(), v[:, :2].contiguous()
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    a = fa.flash_attention_varlen(q, k, v, cu_t, cu_t, max(lens), max(lens), causal=True)
    old = A._set_force_flags(_lib.FLAG_FORCE_MMA_SYNC)
    try:
        b = fa.flash_attention_varlen(q, k, v, cu_t, cu_t, max(lens), max(lens), causal=True)
    finally:
        A._set_force_flags(old)
    assert float((a.float() - b.float()).abs().max()) <= 2e-2
    O, _ = orc.varlen(q.cpu(), k.cpu(), v.cpu(), cu, cu, causal=True)
    assert_close(a, O, torch.bfloat16)
