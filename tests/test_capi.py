"""The C-ABI library loads, exports every symbol include/nckv.h declares, and rejects bad
arguments on the host before touching a device (no compute happens in this file)."""
import ctypes
import os
import re

from nanochat_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "nckv.h")).read()
    return sorted(set(re.findall(r"NCKV_API[^;(]*?\b(nckv_\w+)\s*\(", text)))


def test_header_and_library_agree():
    declared = _declared_symbols()
    assert len(declared) >= 11
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/nckv.h but not exported"
    assert set(_lib.SIGNATURES) == set(declared), "ctypes table and header drifted apart"
    assert _lib.lib.nckv_arch() == b"sm_100a"
    assert _lib.lib.nckv_version() >= 100


def test_host_side_rejections():
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)  # never dereferenced: every call below is rejected during validation
    rc = _lib.lib.nckv_decode_attn(null, null, null, null, null, null, null, 1, 1, 1, 128, 16, 0, 128, 1, -1, 0, 0,
                                   null, 0, null)
    assert rc == -1 and b"null" in _lib.lib.nckv_last_error()
    rc = _lib.lib.nckv_decode_attn(one, one, one, one, one, null, null, 1, 2, 2, 64, 16, 0, 128, 1, -1, 0, 0, one, 0,
                                   null)
    assert rc == -2 and b"head_dim" in _lib.lib.nckv_last_error()
    rc = _lib.lib.nckv_decode_attn(one, one, one, one, one, null, null, 1, 3, 2, 128, 16, 0, 256, 1, -1, 0, 0, one, 0,
                                   null)
    assert rc == -2  # Hq not a multiple of Hkv
    rc = _lib.lib.nckv_append(one, one, one, one, one, 1, 4, 1, 128, 2, 256, 128, one, null)
    assert rc == -3 and b"capacity" in _lib.lib.nckv_last_error()
    rc = _lib.lib.nckv_prefill_broadcast(one, one, one, one, null, 1, 2, 9, 1, 128, 8, 16, null)
    assert rc == -3
    rc = _lib.lib.nckv_lse_combine(one, one, 0, 4, 128, 512, 4, one, null, null)
    assert rc == -1
    assert _lib.lib.nckv_workspace_bytes(1, 3, 2, 128) == 0
    try:
        _lib.call("nckv_lse_combine", one, one, 2, 4, 64, 256, 4, one, null, null)
    except _lib.NckvError as e:
        assert e.code == -2 and "head_dim" in str(e)
    else:
        raise AssertionError("expected NckvError")
