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
