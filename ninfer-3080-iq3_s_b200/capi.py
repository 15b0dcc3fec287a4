"""ctypes binding of the C ABI declared in include/kvarn_b200.h.

The library is the product: there is no CPU fallback.  `load()` raises if libkvarn_b200.so is missing,
and every wrapper raises `KvarnError` on a non-zero status with the library's own error text.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("KVB_LIBRARY", os.path.join(_HERE, "libkvarn_b200.so"))

KVB_OK, KVB_EINVAL, KVB_ECUDA, KVB_ERANGE, KVB_ETIMEOUT = range(5)
DTYPE_F16, DTYPE_BF16 = 0, 1
ERR_PAGE_RANGE, ERR_TABLE_RANGE, ERR_WAIT_TIMEOUT, ERR_POSITIONS, ERR_GEOMETRY = 1, 2, 4, 8, 16


class KvarnError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"kvarn_b200 status {status}: {text}")
        self.status = status


class kvb_layer(C.Structure):
    _fields_ = [
        ("k_code", C.c_void_p), ("k_scale", C.c_void_p), ("v_code", C.c_void_p), ("v_scale", C.c_void_p),
        ("stage", C.c_void_p), ("table_direct", C.c_void_p), ("tables", C.c_void_p), ("table_rows", C.c_void_p),
        ("table_stride", C.c_int32), ("table_len", C.c_int32), ("pages", C.c_int32), ("kv_heads", C.c_int32),
        ("q_heads", C.c_int32), ("head_dim", C.c_int32), ("dtype", C.c_int32), ("sinkhorn_iters", C.c_int32),
        ("error_word", C.c_void_p),
    ]


class kvb_peer_ring(C.Structure):
    _fields_ = [("peer_bufs", C.POINTER(C.c_void_p)), ("local_buf", C.c_void_p), ("state", C.c_void_p), ("rank", C.c_int32),
                ("world", C.c_int32), ("max_spins", C.c_uint32), ("rows", C.c_uint32)]


# name -> (restype, argtypes); every symbol the header declares
SYMBOLS = {
    "kvb_last_error_string": (C.c_char_p, []),
    "kvb_version": (C.c_int, []),
    "kvb_stage_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "kvb_plane_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "kvb_append": (C.c_int, [C.POINTER(kvb_layer), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "kvb_decode_tile": (C.c_int, [C.POINTER(kvb_layer), C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "kvb_record_bytes": (C.c_size_t, [C.c_int]),
    "kvb_records_encode": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "kvb_records_decode": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "kvb_split_capacity": (C.c_int, [C.c_int] * 5),
    "kvb_workspace_bytes": (C.c_size_t, [C.c_int] * 6),
    "kvb_attn_decode": (C.c_int, [C.POINTER(kvb_layer), C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p,
                                  C.c_void_p, C.c_void_p]),
    "kvb_static_scratch_bytes": (C.c_size_t, []),
    "kvb_attn_decode_static": (C.c_int, [C.POINTER(kvb_layer), C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p, C.c_void_p]),
    "kvb_attn_decode_partial": (C.c_int, [C.POINTER(kvb_layer), C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int,
                                          C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "kvb_merge_partials": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_void_p, C.c_void_p]),
    "kvb_merge_partials_packed": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "kvb_batch_workspace_bytes": (C.c_size_t, [C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int, C.c_int]),
    "kvb_attn_decode_batch": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_float,
                                        C.POINTER(C.c_int32), C.c_void_p, C.c_void_p, C.c_void_p]),
    "kvb_peer_ring_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "kvb_attn_decode_sharded": (C.c_int, [C.POINTER(kvb_layer), C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p,
                                          C.POINTER(kvb_peer_ring), C.c_void_p, C.c_void_p]),
    "kvb_attn_rows_sharded": (C.c_int, [C.POINTER(kvb_layer), C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_void_p,
                                        C.POINTER(kvb_peer_ring), C.c_void_p, C.c_void_p]),
    "kvb_append_decode": (C.c_int, [C.POINTER(kvb_layer), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p,
                                    C.POINTER(kvb_peer_ring), C.c_void_p, C.c_void_p]),
    "kvb_attn_verify": (C.c_int, [C.POINTER(kvb_layer), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                  C.c_float, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "kvb_attn_rows": (C.c_int, [C.POINTER(kvb_layer), C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_float, C.c_int, C.c_void_p,
                                C.c_void_p, C.c_void_p]),
    "kvb_attn_prefill": (C.c_int, [C.POINTER(kvb_layer), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                   C.c_float, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "kvb_prefill_workspace_bytes": (C.c_size_t, [C.c_int] * 5),
    "kvb_attn_chunk_partial": (C.c_int, [C.POINTER(kvb_layer), C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(f"{LIB_PATH} is missing: build it with `python {_HERE}/build.py` (needs nvcc)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status != KVB_OK:
        raise KvarnError(status, load().kvb_last_error_string().decode(errors="replace"))
