"""CPU tests of the C-ABI boundary: the library loads, exports every symbol that
include/b200fa.h declares, and rejects bad arguments on the host before any launch."""
import ctypes as C
import os
import re

import pytest

from mlx_flashattention_steel_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    txt = open(os.path.join(ROOT, "include", "b200fa.h")).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b(b200fa_[a-z0-9_]+)\s*\(", txt)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), f"{n} declared in b200fa.h but not exported"
    assert sorted(_lib.SIGNATURES) == [n for n in names if n in _lib.SIGNATURES]
    missing = [n for n in names if n not in _lib.SIGNATURES]
    assert not missing, f"no ctypes prototype for {missing}"
    assert b"b200fa" in lib.b200fa_version()


def _desc(**kw):
    d = _lib.Desc()
    d.dtype = d.kv_dtype = _lib.BF16
    d.B, d.Hq, d.Hkv, d.N, d.S, d.D = 1, 4, 2, 16, 16, 128
    d.scale = 0.1
    d.window_left = -1
    for k, v in kw.items():
        setattr(d, k, v)
    return d


@pytest.mark.parametrize(
    "kw,code",
    [
        (dict(D=96), _lib.ERR_UNSUPPORTED),
        (dict(dtype=7), _lib.ERR_UNSUPPORTED),
        (dict(Hq=5), _lib.ERR_INVALID_ARG),
        (dict(N=-1), _lib.ERR_INVALID_ARG),
        (dict(softcap=-1.0), _lib.ERR_INVALID_ARG),
        (dict(window_left=-5), _lib.ERR_INVALID_ARG),
    ],
)
def test_forward_rejects_bad_descriptors(kw, code):
    lib = _lib.load()
    d = _desc(**kw)
    buf = C.c_void_p(256)  # never dereferenced: validation fails first
    st = lib.b200fa_fwd(C.byref(d), buf, buf, buf, buf, None, None, 0, None)
    assert st == code
    assert _lib.last_error()


def test_forward_rejects_null_and_misaligned_pointers():
    lib = _lib.load()
    d = _desc()
    st = lib.b200fa_fwd(C.byref(d), None, None, None, None, None, None, 0, None)
    assert st == _lib.ERR_INVALID_ARG
    st = lib.b200fa_fwd(C.byref(d), C.c_void_p(8), C.c_void_p(256), C.c_void_p(256), C.c_void_p(256), None, None, 0, None)
    assert st == _lib.ERR_INVALID_ARG and "aligned" in _lib.last_error()
    st = lib.b200fa_fwd(None, None, None, None, None, None, None, 0, None)
    assert st == _lib.ERR_INVALID_ARG


def test_empty_problem_is_a_no_op():
    lib = _lib.load()
    d = _desc(N=0)
    assert lib.b200fa_fwd(C.byref(d), None, None, None, None, None, None, 0, None) == _lib.OK
    d = _desc(B=0)
    assert lib.b200fa_fwd(C.byref(d), None, None, None, None, None, None, 0, None) == _lib.OK


def test_backward_needs_workspace_and_16bit():
    lib = _lib.load()
    d = _desc()
    need = lib.b200fa_bwd_workspace_bytes(C.byref(d))
    assert need > 0
    p = C.c_void_p(256)
    st = lib.b200fa_bwd(C.byref(d), p, p, p, p, p, p, p, p, p, None, 0, None)
    assert st == _lib.ERR_WORKSPACE
    d32 = _desc(dtype=_lib.F32, kv_dtype=_lib.F32)
    st = lib.b200fa_bwd(C.byref(d32), p, p, p, p, p, p, p, p, p, p, 1 << 30, None)
    assert st == _lib.ERR_UNSUPPORTED


def test_gather_rejects_bad_arguments():
    lib = _lib.load()
    p = C.c_void_p(256)
    assert lib.b200fa_paged_kv_gather(p, p, p, 1, 2, 12, 2, 16, 4, 32, p, None) == _lib.ERR_INVALID_ARG  # D*eb % 16
    assert lib.b200fa_paged_kv_gather(p, p, p, 1, 2, 64, 3, 16, 4, 32, p, None) == _lib.ERR_INVALID_ARG  # elem_bytes
    assert lib.b200fa_paged_kv_gather(p, p, p, 1, 2, 64, 2, 16, 1, 32, p, None) == _lib.ERR_INVALID_ARG  # max_kv_len
    assert lib.b200fa_paged_kv_gather(None, p, p, 1, 2, 64, 2, 16, 4, 32, p, None) == _lib.ERR_INVALID_ARG
    assert lib.b200fa_paged_kv_gather(None, None, None, 0, 2, 64, 2, 16, 4, 32, None, None) == _lib.OK


def test_decode_rejects_bad_arguments():
    lib = _lib.load()
    p = C.c_void_p(256)
    d = _desc(N=1, Hq=32, Hkv=8, kv_dtype=_lib.I8)
    # quantized pools without scales
    st = lib.b200fa_decode_paged(C.byref(d), p, p, p, None, None, p, p, 10, 16, 4, 64, p, None, p, 1 << 30, None)
    assert st == _lib.ERR_INVALID_ARG
    d = _desc(N=4, Hq=32, Hkv=8)   # 16 query rows per kv head
    st = lib.b200fa_decode_paged(C.byref(d), p, p, p, None, None, p, p, 10, 16, 4, 64, p, None, p, 1 << 30, None)
    assert st == _lib.ERR_UNSUPPORTED
    d = _desc(N=1, Hq=32, Hkv=8)
    st = lib.b200fa_decode_paged(C.byref(d), p, p, p, None, None, p, p, 10, 16, 4, 64, p, None, None, 0, None)
    assert st == _lib.ERR_WORKSPACE


def test_decode_shapes_and_page_sizes_are_validated():
    lib = _lib.load()
    p = C.c_void_p(256)
    d = _desc(N=1, Hq=32, Hkv=8)
    # pages must hold a multiple of 16 tokens
    st = lib.b200fa_decode_paged(C.byref(d), p, p, p, None, None, p, p, 10, 24, 4, 64, p, None, p, 1 << 30, None)
    assert st == _lib.ERR_UNSUPPORTED and "multiple of 16" in _lib.last_error()
    # head_dim 64 takes 16-bit pools only
    d = _desc(N=1, Hq=32, Hkv=8, D=64, kv_dtype=_lib.I8)
    st = lib.b200fa_decode_paged(C.byref(d), p, p, p, p, p, p, p, 10, 16, 4, 64, p, None, p, 1 << 30, None)
    assert st == _lib.ERR_UNSUPPORTED and "head_dim 64" in _lib.last_error()


def test_dense_decode_route_asks_for_a_workspace_only_where_it_applies():
    lib = _lib.load()
    # N <= 4 and S >= 256 (the reference's flash-decode threshold), at most 8 query rows per kv head
    assert lib.b200fa_fwd_workspace_bytes(C.byref(_desc(N=1, S=4096, Hq=32, Hkv=8))) > 0
    assert lib.b200fa_fwd_workspace_bytes(C.byref(_desc(N=4, S=256, Hq=4, Hkv=2))) > 0
    assert lib.b200fa_fwd_workspace_bytes(C.byref(_desc(N=5, S=4096, Hq=4, Hkv=4))) == 0
    assert lib.b200fa_fwd_workspace_bytes(C.byref(_desc(N=1, S=255, Hq=4, Hkv=4))) == 0
    assert lib.b200fa_fwd_workspace_bytes(C.byref(_desc(N=4, S=4096, Hq=32, Hkv=8))) == 0          # 16 rows per kv head
    assert lib.b200fa_fwd_workspace_bytes(C.byref(_desc(N=1, S=4096, Hq=4, Hkv=4, window_left=64))) == 0
    assert lib.b200fa_fwd_workspace_bytes(C.byref(_desc(N=1, S=4096, Hq=4, Hkv=4, dtype=_lib.F32))) == 0


def test_paged_forward_and_helpers_reject_bad_arguments():
    lib = _lib.load()
    p = C.c_void_p(256)
    d = _desc(N=64, Hq=8, Hkv=2)
    call = lambda dd, bs=16, pages=10, mb=8, ml=100: lib.b200fa_fwd_paged(C.byref(dd), p, p, p, p, p, pages, bs, mb, ml, p, None, None)
    assert call(d, bs=24) == _lib.ERR_UNSUPPORTED                       # pages of a multiple of 16 tokens
    assert call(_desc(N=64, Hq=8, Hkv=2, kv_dtype=_lib.I8)) == _lib.ERR_UNSUPPORTED and "gather_dequant" in _lib.last_error()
    assert call(d, mb=2, ml=100) == _lib.ERR_INVALID_ARG                # max_kv_len beyond max_blocks * block_size
    assert call(_desc(N=64, Hq=8, Hkv=2, D=256)) == _lib.ERR_UNSUPPORTED
    assert lib.b200fa_fwd_paged(C.byref(d), p, None, p, p, p, 10, 16, 8, 100, p, None, None) == _lib.ERR_INVALID_ARG
    # gather + dequantise
    gd = lib.b200fa_paged_kv_gather_dequant
    assert gd(p, p, p, p, 1, 2, 128, _lib.BF16, _lib.BF16, 16, 4, 32, p, None) == _lib.ERR_UNSUPPORTED    # pool must be 8-bit
    assert gd(p, p, p, p, 1, 2, 128, _lib.I8, _lib.F32, 16, 4, 32, p, None) == _lib.ERR_UNSUPPORTED
    assert gd(p, p, p, p, 1, 2, 72, _lib.I8, _lib.BF16, 16, 4, 32, p, None) == _lib.ERR_INVALID_ARG       # D % 16
    assert gd(p, None, p, p, 1, 2, 128, _lib.I8, _lib.BF16, 16, 4, 32, p, None) == _lib.ERR_INVALID_ARG
    assert gd(None, None, None, None, 0, 2, 128, _lib.I8, _lib.BF16, 16, 4, 32, None, None) == _lib.OK
    # combine of partials
    cp = lib.b200fa_combine_partials
    assert cp(p, 2, 8, 130, _lib.BF16, p, None, None) == _lib.ERR_INVALID_ARG                            # D % 4, D <= 128
    assert cp(p, 2, 8, 128, _lib.F32, p, None, None) == _lib.ERR_UNSUPPORTED
    assert cp(None, 2, 8, 128, _lib.BF16, p, None, None) == _lib.ERR_INVALID_ARG
    assert cp(None, 0, 8, 128, _lib.BF16, None, None, None) == _lib.OK
    # the static decode entry's status reader
    assert lib.b200fa_decode_paged_static_status(None, None) == _lib.ERR_INVALID_ARG


def test_kv_lens_is_refused_where_no_kernel_honours_it():
    lib = _lib.load()
    p = C.c_void_p(256)
    d = _desc(dtype=_lib.F32, kv_dtype=_lib.F32)
    d.kv_lens = 256
    assert lib.b200fa_fwd(C.byref(d), p, p, p, p, None, None, 0, None) == _lib.ERR_UNSUPPORTED
    d = _desc()
    d.kv_lens = 256
    assert lib.b200fa_bwd(C.byref(d), p, p, p, p, p, p, p, p, p, p, 1 << 30, None) == _lib.ERR_UNSUPPORTED
    dv = _desc(B=1)
    dv.kv_lens = 256
    assert lib.b200fa_fwd_varlen(C.byref(dv), p, p, p, p, p, 1, 16, 16, p, None, None, 0, None) == _lib.ERR_UNSUPPORTED
