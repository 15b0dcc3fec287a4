"""ctypes/numpy front end of the CPU oracle (oracle/kvarn_oracle.c) and of the compiled reference
oracle (oracle/_ref/libbee_ref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's
CPU-baseline leg.  The product path (the CUDA library and its bindings) never imports this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

TILE, PAGE, SLICE = 128, 64, 128


def build(quiet: bool = True) -> None:
    """Compile the C restatement (and the reference oracle when its sources are present)."""
    subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL if quiet else None)


def _p(a, t=C.c_void_p):
    return None if a is None else a.ctypes.data_as(t)


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libkvarn_oracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.kvo_f32_to_f16.restype = C.c_uint16
        L.kvo_f32_to_f16.argtypes = [C.c_float]
        L.kvo_f16_to_f32.restype = C.c_float
        L.kvo_f16_to_f32.argtypes = [C.c_uint16]
        L.kvo_plane_offset.restype = C.c_int64
        L.kvo_plane_offset.argtypes = [C.c_int] * 6
        L.kvo_record_bytes.restype = C.c_size_t
        L.kvo_record_bytes.argtypes = [C.c_int] * 3
        _LIB = L
    return _LIB


def ref():
    """The reference's own oracle (None when it was not built, e.g. on a box without its sources)."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libbee_ref.so")
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        R.bee_ref_f32_to_f16.restype = C.c_uint16
        R.bee_ref_f32_to_f16.argtypes = [C.c_float]
        R.bee_ref_f16_to_f32.restype = C.c_float
        R.bee_ref_f16_to_f32.argtypes = [C.c_uint16]
        R.bee_ref_quant_tile.restype = C.c_int
        _REF = R
    return _REF


# --------------------------------------------------------------------------- codec primitives
def hadamard(x: np.ndarray) -> np.ndarray:
    """Normalised Hadamard of the last axis (128 or 256), fp32, in the oracle's butterfly order."""
    y = np.ascontiguousarray(x, dtype=np.float32).copy()
    flat = y.reshape(-1, y.shape[-1])
    for r in flat:
        lib().kvo_hadamard(_p(r), C.c_int(r.shape[0]))
    return y


def quantize_tile(tile: np.ndarray, bits: int = 4, iters: int = 0):
    """-> (record bytes, codes[rows, cols], best_col, best_row)."""
    tile = np.ascontiguousarray(tile, dtype=np.float32)
    rows, cols = tile.shape
    rec = np.zeros(lib().kvo_record_bytes(rows, cols, bits), np.uint8)
    q = np.zeros((rows, cols), np.uint8)
    bc, br = np.zeros(cols, np.float32), np.zeros(rows, np.float32)
    lib().kvo_quantize_tile(_p(tile), rows, cols, bits, iters, _p(rec), _p(q), _p(bc), _p(br))
    return rec, q, bc, br


def dequant_tile(record: np.ndarray, rows: int, cols: int, bits: int = 4) -> np.ndarray:
    out = np.zeros((rows, cols), np.float32)
    lib().kvo_dequant_tile(_p(np.ascontiguousarray(record)), rows, cols, bits, _p(out))
    return out


def ref_quantize_tile(tile: np.ndarray, bits: int = 4, iters: int = 0, cpu_order: bool = False):
    R = ref()
    tile = np.ascontiguousarray(tile, dtype=np.float32)
    rows, cols = tile.shape
    rec = np.zeros(rows * cols * bits // 8 + (2 * rows + cols) * 2, np.uint8)
    bc, br = np.zeros(cols, np.float32), np.zeros(rows, np.float32)
    bi = C.c_int(0)
    R.bee_ref_quant_tile(_p(tile), rows, cols, bits, iters, int(cpu_order), _p(rec), _p(bc), _p(br), C.byref(bi))
    return rec, bc, br, bi.value


def ref_dequant_tile(record: np.ndarray, rows: int, cols: int, bits: int = 4) -> np.ndarray:
    out = np.zeros((rows, cols), np.float32)
    ref().bee_ref_dequant_tile(_p(np.ascontiguousarray(record)), rows, cols, bits, _p(out))
    return out


def scale_slot(head_dim: int, is_value: bool, item: int, slice_: int, index: int):
    r, c = C.c_int(0), C.c_int(0)
    lib().kvo_scale_slot(head_dim, int(is_value), item, slice_, index, C.byref(r), C.byref(c))
    return r.value, c.value


# --------------------------------------------------------------------------- cache of one layer
class CpuLayer:
    """Planes, stage and page table of one layer in host memory, same layout as the CUDA library's."""

    def __init__(self, head_dim: int, kv_heads: int, pages: int, table: np.ndarray, iters: int = 0):
        S = head_dim // SLICE
        self.head_dim, self.kv_heads, self.pages, self.iters = head_dim, kv_heads, pages, iters
        self.k_code = np.zeros((pages, kv_heads, PAGE, head_dim // 2), np.uint8)
        self.v_code = np.zeros((pages, kv_heads, PAGE, head_dim // 2), np.uint8)
        self.k_scale = np.zeros((pages, kv_heads, PAGE, 5 * S), np.uint16)
        self.v_scale = np.zeros((pages, kv_heads, PAGE, 4 * S), np.uint16)
        self.stage = np.zeros((2, 2, kv_heads, TILE, head_dim), np.uint16)
        self.table = np.ascontiguousarray(table, dtype=np.int32)
        self.kv_total = 0

    def append(self, k: np.ndarray, v: np.ndarray, pos0: int, dtype: int = 0) -> None:
        """k, v: [tokens, kv_heads, head_dim] raw 16-bit patterns (uint16 view of fp16/bf16)."""
        k = np.ascontiguousarray(k).view(np.uint16)
        v = np.ascontiguousarray(v).view(np.uint16)
        tokens = k.shape[0]
        lib().kvo_append(_p(self.k_code), _p(self.k_scale), _p(self.v_code), _p(self.v_scale), _p(self.stage),
                         _p(self.table), self.head_dim, self.kv_heads, self.iters, _p(k), _p(v), dtype,
                         int(pos0), int(tokens))
        self.kv_total = pos0 + tokens

    def decode_tile(self, tile: int, head: int):
        ok = np.zeros((TILE, self.head_dim), np.uint16)
        ov = np.zeros((TILE, self.head_dim), np.uint16)
        lib().kvo_decode_tile(_p(self.k_code), _p(self.k_scale), _p(self.v_code), _p(self.v_scale), _p(self.table),
                              self.head_dim, self.kv_heads, tile, head, _p(ok), _p(ov))
        return ok.view(np.float16), ov.view(np.float16)

    def attention(self, q: np.ndarray, q_pos, scale: float, q_heads: int, dtype: int = 0, threads: int = 1,
                  key_begin: int = 0, key_end: int | None = None, kv_total: int | None = None,
                  want_partials: bool = False):
        """q: [T, q_heads, head_dim] 16-bit patterns; q_pos: [T] absolute positions.
        -> out fp32 [T, q_heads, head_dim] (and the (m, l, o_rot) partials when asked)."""
        q = np.ascontiguousarray(q).view(np.uint16)
        T = q.shape[0]
        q_pos = np.ascontiguousarray(q_pos, dtype=np.int32)
        kv_total = self.kv_total if kv_total is None else kv_total
        key_end = kv_total if key_end is None else key_end
        out = np.zeros((T, q_heads, self.head_dim), np.float32)
        pm = np.zeros((T, q_heads), np.float32) if want_partials else None
        pl = np.zeros((T, q_heads), np.float32) if want_partials else None
        po = np.zeros((T, q_heads, self.head_dim), np.float32) if want_partials else None
        lib().kvo_attention(_p(self.k_code), _p(self.k_scale), _p(self.v_code), _p(self.v_scale), _p(self.stage),
                            _p(self.table), self.head_dim, self.kv_heads, q_heads, _p(q), dtype, _p(q_pos), T,
                            int(kv_total), int(key_begin), int(key_end), C.c_float(scale), int(threads), _p(out),
                            _p(pm), _p(pl), _p(po))
        return (out, pm, pl, po) if want_partials else out


def merge_partials(pm: np.ndarray, pl: np.ndarray, po: np.ndarray) -> np.ndarray:
    """pm, pl: [R, rows]; po: [R, rows, D] -> fp32 [rows, D] (normalised, un-rotated)."""
    R, rows, D = po.shape
    out = np.zeros((rows, D), np.float32)
    lib().kvo_merge_partials(_p(np.ascontiguousarray(pm, np.float32)), _p(np.ascontiguousarray(pl, np.float32)),
                             _p(np.ascontiguousarray(po, np.float32)), R, rows, D, _p(out))
    return out


# --------------------------------------------------------------------------- synthetic inputs
OUTLIER_CHANNELS = (3, 17, 64, 101)


def synth_kv(seed: int, tokens: int, heads: int, head_dim: int, stream: int = 0) -> np.ndarray:
    """fp16 [tokens, heads, head_dim] ~ N(0,1) with channels {3,17,64,101} of each head row x20."""
    rng = np.random.default_rng([seed, stream])
    x = rng.standard_normal((tokens, heads, head_dim), dtype=np.float32)
    x[..., list(OUTLIER_CHANNELS)] *= 20.0
    return x.astype(np.float16)


def synth_q(seed: int, tokens: int, q_heads: int, head_dim: int, stream: int = 7) -> np.ndarray:
    rng = np.random.default_rng([seed, stream])
    return rng.standard_normal((tokens, q_heads, head_dim), dtype=np.float32).astype(np.float16)


def shuffled_table(seed: int, logical_pages: int, physical_pages: int | None = None) -> np.ndarray:
    physical_pages = logical_pages if physical_pages is None else physical_pages
    rng = np.random.default_rng([seed, 99])
    return rng.permutation(physical_pages)[:logical_pages].astype(np.int32)


def attention_fp32_dense(k_rot: np.ndarray, v_rot: np.ndarray, q: np.ndarray, q_pos, scale: float) -> np.ndarray:
    """Independent check of CpuLayer.attention: plain numpy softmax attention (float64) on fully
    materialised rotated-domain K/V [kv, H, D]; q fp16 [T, QH, D]."""
    T, QH, D = q.shape
    H = k_rot.shape[1]
    G = QH // H
    qr = hadamard(q.astype(np.float32)).astype(np.float64)
    out = np.zeros((T, QH, D), np.float32)
    for t in range(T):
        n = int(q_pos[t]) + 1
        for h in range(H):
            K = k_rot[:n, h].astype(np.float64)
            V = v_rot[:n, h].astype(np.float64)
            for g in range(G):
                s = K @ qr[t, h * G + g] * scale
                p = np.exp(s - s.max())
                o = (p @ V) / p.sum()
                out[t, h * G + g] = hadamard(o.astype(np.float32))
    return out
