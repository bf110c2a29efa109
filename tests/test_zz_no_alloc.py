"""The allocation-free decode entry point, b200fa_decode_paged_static, through the C-ABI.

Some callers of this library cannot hand an operator scratch memory: an inference
server that gave every spare byte of HBM to its KV page pool when it started, or a
foreign-language binding that only forwards the input and output buffers.  For them
the library keeps a fixed 16 MiB scratch array inside its own device image.  This test
drives that entry point with ctypes exactly as such a caller would (raw pointers, no
workspace argument) and checks, on two calls in a row that reuse the shared scratch,
that the result equals the one from the workspace-taking entry point.

Collected last (file name) so that a run stopping at the first failure has already
been through every other test; it also passes when run alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from mlx_flashattention_steel_b200 import _lib

from .util import make_paged, randn

pytestmark = pytest.mark.gpu


def _call(lib, static, d, q, pg, table, lens, max_len, out, lse, ws=None):
    p = lambda t: None if t is None else C.c_void_p(t.data_ptr())
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    common = (C.byref(d), p(q), p(pg["k"]), p(pg["v"]), p(pg["k_scale"]), p(pg["v_scale"]), p(table), p(lens),
              pg["k"].shape[0], 16, table.shape[1], max_len, p(out), p(lse))
    if static:
        return lib.b200fa_decode_paged_static(*common, stream)
    return lib.b200fa_decode_paged(*common, p(ws), ws.numel(), stream)


@pytest.mark.parametrize("quant,qdtype", [("int8", torch.bfloat16), (None, torch.float16)])
def test_static_scratch_matches_workspace_entry(dev, quant, qdtype):
    lib = _lib.load()
    B, Hq, Hkv, D = 6, 32, 8, 128
    out_prev = None
    for call, seed in enumerate((900, 901)):          # two calls in a row share the scratch
        lens_list = [700, 33, 0, 4000, 16, 129] if call == 0 else [64, 2500, 17, 1, 900, 300]
        pg = make_paged(B, Hkv, D, 16, lens_list, qdtype, seed, quant=quant)
        pg = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in pg.items()}
        table, lens = pg["block_table"].contiguous(), pg["seq_lens"].contiguous()
        q = randn((B, Hq, 1, D), qdtype, seed + 50).to(dev)
        d = _lib.Desc()
        d.dtype = _lib.BF16 if qdtype == torch.bfloat16 else _lib.F16
        d.kv_dtype = _lib.I8 if quant == "int8" else d.dtype
        d.B, d.Hq, d.Hkv, d.N, d.S, d.D = B, Hq, Hkv, 1, 0, D
        d.scale, d.softcap, d.causal, d.window_left = D ** -0.5, 0.0, 1, -1
        max_len = max(lens_list)
        need = lib.b200fa_decode_paged_workspace_bytes(C.byref(d), max_len)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        o_ref = torch.empty_like(q)
        l_ref = torch.empty((B, Hq, 1), dtype=torch.float32, device=dev)
        o_new = torch.full_like(q, float("nan"))
        l_new = torch.full_like(l_ref, float("nan"))
        assert _call(lib, False, d, q, pg, table, lens, max_len, o_ref, l_ref, ws) == _lib.OK, _lib.last_error()
        assert _call(lib, True, d, q, pg, table, lens, max_len, o_new, l_new) == _lib.OK, _lib.last_error()
        torch.cuda.synchronize()
        # a caller of the static entry has no workspace pointer to read the kernel's error word from: it asks for it
        word = C.c_int32(-1)
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert lib.b200fa_decode_paged_static_status(stream, C.byref(word)) == _lib.OK, _lib.last_error()
        assert word.value == 0
        assert float((o_new.float() - o_ref.float()).abs().max()) <= 2e-2
        fin = torch.isfinite(l_ref)
        assert torch.equal(torch.isfinite(l_new), fin)
        assert float((l_new[fin] - l_ref[fin]).abs().max()) <= 2e-2
        assert not torch.isnan(o_new).any()
        if out_prev is not None:
            assert not torch.equal(o_new, out_prev)      # the second call really recomputed
        out_prev = o_new.clone()


def test_static_scratch_rejects_oversized_problems(dev):
    lib = _lib.load()
    d = _lib.Desc()
    d.dtype = d.kv_dtype = _lib.BF16
    d.B, d.Hq, d.Hkv, d.N, d.S, d.D = 4096, 64, 8, 1, 0, 128     # partials far beyond 16 MiB
    d.scale, d.window_left, d.causal = 0.1, -1, 1
    p = C.c_void_p(256)          # never dereferenced: the size check comes first
    st = lib.b200fa_decode_paged_static(C.byref(d), p, p, p, None, None, p, p, 10, 16, 4, 64, p, None, None)
    assert st == _lib.ERR_WORKSPACE
    assert "scratch" in _lib.last_error()


def test_static_scratch_reports_a_table_entry_beyond_the_pool(dev):
    """A block_table entry >= num_pages is not followed (the kernel treats it as a hole: K = V = 0 for that page) and
    sets bit 1 of the error word, which the static entry's status call must be able to show."""
    lib = _lib.load()
    B, Hq, Hkv, D = 2, 8, 2, 128
    pg = make_paged(B, Hkv, D, 16, [40, 100], torch.bfloat16, 910)
    pg = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in pg.items()}
    table, lens = pg["block_table"].clone().contiguous(), pg["seq_lens"].contiguous()
    table[1, 2] = pg["k"].shape[0] + 5                  # beyond the pool
    q = randn((B, Hq, 1, D), torch.bfloat16, 911).to(dev)
    d = _lib.Desc()
    d.dtype = d.kv_dtype = _lib.BF16
    d.B, d.Hq, d.Hkv, d.N, d.S, d.D = B, Hq, Hkv, 1, 0, D
    d.scale, d.softcap, d.causal, d.window_left = D ** -0.5, 0.0, 1, -1
    out = torch.empty_like(q)
    assert _call(lib, True, d, q, pg, table, lens, 100, out, None) == _lib.OK, _lib.last_error()
    word = C.c_int32(-1)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.b200fa_decode_paged_static_status(stream, C.byref(word)) == _lib.OK, _lib.last_error()
    assert word.value == 2
    assert torch.isfinite(out.float()).all()
    # the next valid call clears the word again
    table[1, 2] = pg["block_table"][1, 2]
    assert _call(lib, True, d, q, pg, table, lens, 100, out, None) == _lib.OK, _lib.last_error()
    assert lib.b200fa_decode_paged_static_status(stream, C.byref(word)) == _lib.OK
    assert word.value == 0
