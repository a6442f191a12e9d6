"""ctypes binding of libsqattn_b200.so (the C ABI declared in include/sqattn_b200.h).

The library is the product: there is no fallback.  Importing this module when
the shared object has not been built raises at once.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# SQATTN_B200_LIB selects another build of the same library (e.g. the one with the debug exports)
LIB_PATH = os.environ.get("SQATTN_B200_LIB") or os.path.join(_HERE, "libsqattn_b200.so")

F16, BF16 = 0, 1
MODE_DENSE_CAUSAL, MODE_RELATIVE_WINDOW, MODE_ABSOLUTE_WINDOW = 0, 1, 2
P_FP8_OFF, P_FP8_ALL, P_FP8_STAGE2 = 0, 1, 2
QTYPE = {"int": 0, "e4m3": 1, "e5m2": 2}

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE, ERR_DEVICE_TIMEOUT = range(6)


class SqattnError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"sqattn_b200 error {code}: {msg}")
        self.code = code


class Tensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_n", C.c_int64)]


class PrefillArgs(C.Structure):
    _fields_ = [
        ("q_int8", Tensor), ("k_int8", Tensor), ("q_int4", Tensor), ("k_int4", Tensor), ("v", Tensor), ("o", Tensor),
        ("lse", C.c_void_p),
        ("batch", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("qo_len", C.c_int32),
        ("kv_len", C.c_int32), ("head_dim", C.c_int32),
        ("qk_dtype", C.c_int32), ("v_dtype", C.c_int32), ("o_dtype", C.c_int32),
        ("mode", C.c_int32), ("sink_size", C.c_int32),
        ("win8_ratios", C.POINTER(C.c_float)), ("win4_ratios", C.POINTER(C.c_float)),
        ("win8_sizes", C.POINTER(C.c_int32)), ("win4_sizes", C.POINTER(C.c_int32)),
        ("p_fp8_mode", C.c_int32), ("q_is_scaled", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("q_row_offset", C.c_int32), ("q_split_rows", C.c_int32), ("q_row_offset2", C.c_int32),
        ("q_fake_quant", C.c_int32), ("q_round_half_even", C.c_int32), ("head_dim_og", C.c_int32),
    ]


class PrepArgs(C.Structure):
    _fields_ = [
        ("q", Tensor), ("k", Tensor), ("v", Tensor),
        ("q_bit8", C.c_void_p), ("q_bit4", C.c_void_p), ("k_bit8", C.c_void_p), ("k_bit4", C.c_void_p),
        ("v_bit8", C.c_void_p),
        ("batch", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("seq_len", C.c_int32),
        ("head_dim", C.c_int32), ("dtype", C.c_int32), ("qk_qtype", C.c_int32), ("v_qtype", C.c_int32),
        ("round_half_even", C.c_int32), ("skip_bit4", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("k_mean", C.c_void_p), ("kv_out_nhd", C.c_int32), ("parts", C.c_int32),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", Tensor), ("k", Tensor), ("v", Tensor), ("o", Tensor), ("lse", C.c_void_p),
        ("batch", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("kv_len", C.c_int32), ("kv_lens", C.POINTER(C.c_int32)),
        ("dtype", C.c_int32), ("o_dtype", C.c_int32), ("p_fp8", C.c_int32), ("q_is_scaled", C.c_int32),
        ("num_splits", C.c_int32), ("reference_tail", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("partial_o", C.c_void_p), ("partial_lse", C.c_void_p), ("kv_lens_device", C.c_void_p), ("peer", C.c_void_p),
        ("head_dim_og", C.c_int32), ("gather", C.c_void_p),
    ]


class DecodeGather(C.Structure):
    _fields_ = [("idx", C.c_void_p), ("cap", C.c_int32), ("k_rows", C.c_void_p), ("v_rows", C.c_void_p),
                ("row_stride", C.c_int64)]


# every symbol include/sqattn_b200.h declares: (name, restype, argtypes)
class RetrieveItem(C.Structure):
    _fields_ = [("q", C.c_void_p), ("centroids", C.c_void_p), ("cluster_size", C.c_void_p), ("clusters", C.c_void_p),
                ("num_clusters", C.c_int32), ("max_cluster_size", C.c_int32), ("num_tokens", C.c_int32),
                ("out_idx", C.c_void_p), ("out_count", C.c_void_p), ("k_src", C.c_void_p), ("v_src", C.c_void_p),
                ("src_group_stride", C.c_int64), ("src_row_stride", C.c_int64), ("k_dst", C.c_void_p), ("v_dst", C.c_void_p),
                ("tail_start", C.c_int32), ("split_row", C.c_int32), ("k_src2", C.c_void_p), ("v_src2", C.c_void_p),
                ("src2_group_stride", C.c_int64)]


class PeerMergeArgs(C.Structure):
    _fields_ = [("peer_data", C.c_void_p * 16), ("peer_flags", C.c_void_p * 16), ("rank", C.c_int32), ("world", C.c_int32),
                ("rows", C.c_int32), ("rows_cap", C.c_int32), ("head_dim", C.c_int32), ("epoch", C.c_void_p),
                ("part_o", C.c_void_p), ("part_lse", C.c_void_p), ("out", C.c_void_p), ("o_dtype", C.c_int32),
                ("lse", C.c_void_p)]


SYMBOLS = [
    ("sqattn_prefill_workspace_bytes", C.c_size_t, [C.POINTER(PrefillArgs)]),
    ("sqattn_prefill", C.c_int, [C.POINTER(PrefillArgs), C.c_void_p]),
    ("sqattn_prep_workspace_bytes", C.c_size_t, [C.POINTER(PrepArgs)]),
    ("sqattn_prep_qkv", C.c_int, [C.POINTER(PrepArgs), C.c_void_p]),
    ("sqattn_k_column_sums", C.c_int, [C.POINTER(Tensor), C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    ("sqattn_decode_workspace_bytes", C.c_size_t, [C.POINTER(DecodeArgs)]),
    ("sqattn_decode", C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    ("sqattn_decode_static_scratch", C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    ("sqattn_decode_merge", C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_void_p, C.c_int32,
                                      C.c_void_p, C.c_void_p]),
    ("sqattn_kmeans_workspace_bytes", C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    ("sqattn_kmeans_assign", C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    ("sqattn_kmeans_update", C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_int32, C.c_void_p]),
    ("sqattn_kmeans_reverse_index", C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    ("sqattn_kmeans_index_add", C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    ("sqattn_kmeans_max_count", C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    ("sqattn_retrieve_select", C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                         C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                         C.c_int32, C.c_int32, C.c_void_p]),
    ("sqattn_gather_rows", C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                     C.c_int32, C.c_void_p, C.c_void_p]),
    ("sqattn_retrieve_batch", C.c_int, [C.POINTER(RetrieveItem), C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                        C.c_int32, C.c_int32, C.c_void_p]),
    ("sqattn_window_histogram", C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                          C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    ("sqattn_peer_merge_data_bytes", C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    ("sqattn_peer_merge_flag_bytes", C.c_size_t, [C.c_int32, C.c_int32]),
    ("sqattn_decode_peer_merge", C.c_int, [C.POINTER(PeerMergeArgs), C.c_void_p]),
    ("sqattn_rmsnorm", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int64, C.c_int64, C.c_float,
                                 C.c_int32, C.c_void_p]),
    ("sqattn_rope_qk", C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int64,
                                 C.c_int64, C.c_int32, C.c_void_p]),
    ("sqattn_rope_qk_devpos", C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                        C.c_int64, C.c_int64, C.c_void_p, C.c_int32, C.c_void_p]),
    ("sqattn_silu_mul", C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p]),
    ("sqattn_cache_copy_rows", C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int32,
                                         C.c_void_p]),
    ("sqattn_cache_append", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                      C.c_int64, C.c_int32, C.c_int32, C.c_int64, C.c_void_p]),
    ("sqattn_check_device_status", C.c_int, [C.c_void_p]),
    ("sqattn_set_status_mirror", C.c_int, [C.c_void_p]),
    ("sqattn_last_error_string", C.c_char_p, []),
    ("sqattn_version", C.c_int, []),
]

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()' or "
        "python longcontext_sqattn_paddle_b200/build.py). There is no CPU or PyTorch fallback.")

lib = C.CDLL(LIB_PATH)
for _name, _res, _args in SYMBOLS:
    try:
        _fn = getattr(lib, _name)
    except AttributeError as exc:
        raise ImportError(f"{LIB_PATH} is stale (no symbol {_name}): rebuild it with "
                          "python longcontext_sqattn_paddle_b200/build.py --force") from exc
    _fn.restype = _res
    _fn.argtypes = _args


def check(code: int):
    """Raise for a non-zero status, mapping argument errors to ValueError like the reference does."""
    if code == OK:
        return
    msg = lib.sqattn_last_error_string().decode()
    if code in (ERR_INVALID_ARG, ERR_UNSUPPORTED):
        raise ValueError(msg)
    raise SqattnError(code, msg)
