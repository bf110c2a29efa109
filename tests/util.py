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


def grad_bound(ref, dtype):
    """Element-wise bound for a 16-bit gradient: 2e-2 absolute, widened only where one rounding of the result to its
    storage type is itself a sizeable part of that (half a unit in the last place at the reference value, plus 1.5e-2
    for the arithmetic): gradients summed over a GQA group reach |x| >= 8, where bf16's half-ulp alone is 0.03."""
    return torch.clamp(0.5 * ULP[dtype] * ref.abs() + 1.5e-2, min=TOL[dtype])


def assert_close_grad(got, ref, dtype, what):
    a = got.detach().double().cpu()
    b = ref.detach().double().cpu()
    err = (a - b).abs()
    excess = float((err - grad_bound(b, dtype)).max())
    beyond = float((err > TOL[dtype]).double().mean())
    assert excess <= 0, (f"{what}: exceeds max(2e-2, 0.5 ulp + 1.5e-2) by {excess:.3e}; plain max-abs {float(err.max()):.3e}, "
                         f"share of elements beyond 2e-2: {beyond:.2e}, max |ref| {float(b.abs().max()):.2f}")
    return float(err.max()), beyond


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


def free_port():
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def run_ranks(worker, world, args, timeout=300):
    """Spawns `world` processes running worker(rank, world, port, *args, ret) and returns what rank 0 puts on `ret`.
    A rank that dies before reporting fails the test at once (its exit code is polled while waiting), and no child
    outlives the call: whatever is still alive at the end is terminated, then killed, so that a surviving rank cannot
    stay blocked in a collective on its device."""
    import queue
    import time

    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, *args, ret)) for r in range(world)]
    try:
        for p in procs:
            p.start()
        deadline = time.time() + timeout
        result = None
        while result is None:
            try:
                result = ret.get(timeout=1.0)
            except queue.Empty:
                dead = [p.exitcode for p in procs if p.exitcode not in (None, 0)]
                assert not dead, f"a rank exited with code {dead} before reporting"
                assert time.time() < deadline, f"no result from the ranks within {timeout} s"
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0, f"rank exit code {p.exitcode}"
        return result
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
