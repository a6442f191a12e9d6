"""The shared library loads on a machine without a GPU and exports every function include/sqattn_b200.h
declares; argument errors are reported through status codes without touching the device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "sqattn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sqattn_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    from longcontext_sqattn_paddle_b200 import _lib as L
    names = _declared()
    assert len(names) >= 18
    bound = {n for n, _, _ in L.SYMBOLS}
    for n in names:
        assert hasattr(L.lib, n), f"{n} is declared in the header but not exported"
        assert n in bound, f"{n} has no ctypes prototype in _lib.SYMBOLS"
    assert L.lib.sqattn_version() >= 100


def test_argument_errors_are_status_codes():
    from longcontext_sqattn_paddle_b200 import _lib as L
    a = L.PrefillArgs()
    a.head_dim = 256
    assert L.lib.sqattn_prefill(C.byref(a), None) == L.ERR_UNSUPPORTED
    assert b"head_dim" in L.lib.sqattn_last_error_string()
    a.head_dim, a.batch, a.num_q_heads, a.num_kv_heads, a.qo_len, a.kv_len = 128, 1, 4, 3, 128, 128
    assert L.lib.sqattn_prefill(C.byref(a), None) == L.ERR_INVALID_ARG
    d = L.DecodeArgs()
    d.head_dim, d.batch, d.num_q_heads, d.num_kv_heads, d.kv_len = 128, 1, 34, 2, 100
    assert L.lib.sqattn_decode(C.byref(d), None) == L.ERR_UNSUPPORTED   # 17 query heads per KV head
    assert L.lib.sqattn_decode_workspace_bytes(C.byref(d)) == 0
    assert L.lib.sqattn_kmeans_assign(None, None, 0, 1, 10, 33, 128, None, None, None, None, 0, None) == L.ERR_INVALID_ARG
    with pytest.raises(ValueError):
        L.check(L.ERR_INVALID_ARG)


def test_struct_layout_matches_header():
    """Field offsets that the C side relies on (a mismatch would scramble arguments silently)."""
    from longcontext_sqattn_paddle_b200 import _lib as L
    assert C.sizeof(L.Tensor) == 32
    assert L.PrefillArgs.lse.offset == 6 * 32
    assert L.PrefillArgs.win8_ratios.offset == 6 * 32 + 8 + 12 * 4
    assert L.DecodeArgs.kv_lens.offset == 4 * 32 + 8 + 6 * 4
