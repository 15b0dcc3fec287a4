"""Host-side objects over the C ABI: a paged KVarN cache layer in device memory and the operator calls
on it.  torch is used for device memory and streams only; every computation is a call into
libkvarn_b200.so.  Names follow the reference operators (kvarn-port/engine/src/ops/kv_cache/append/
kvarn128_launch.h:40-58 and the attention launchers of patches/0003, lines 2362, 3508, 3612).
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import capi

TILE, PAGE = 128, 64


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class KvarnLayer:
    """Planes, stage, block table and error word of one attention layer of one sequence."""

    def __init__(self, head_dim: int, kv_heads: int, q_heads: int, pages: int, table: torch.Tensor,
                 dtype: torch.dtype = torch.float16, sinkhorn_iters: int = 0, device: str = "cuda"):
        lib = capi.load()
        self.head_dim, self.kv_heads, self.q_heads, self.pages = head_dim, kv_heads, q_heads, pages
        self.dtype = dtype
        self.device = torch.device(device)
        S = head_dim // 128
        kw = dict(device=self.device)
        self.k_code = torch.zeros((pages, kv_heads, PAGE, head_dim // 2), dtype=torch.uint8, **kw)
        self.v_code = torch.zeros((pages, kv_heads, PAGE, head_dim // 2), dtype=torch.uint8, **kw)
        self.k_scale = torch.zeros((pages, kv_heads, PAGE, 5 * S), dtype=torch.float16, **kw)
        self.v_scale = torch.zeros((pages, kv_heads, PAGE, 4 * S), dtype=torch.float16, **kw)
        assert self.k_code.numel() == lib.kvb_plane_bytes(0, head_dim, kv_heads, pages)
        assert self.k_scale.numel() * 2 == lib.kvb_plane_bytes(1, head_dim, kv_heads, pages)
        self.stage = torch.zeros(lib.kvb_stage_bytes(head_dim, kv_heads) // 2, dtype=torch.float16, **kw)
        self.table = table.to(device=self.device, dtype=torch.int32).contiguous()
        self.error_word = torch.zeros(1, dtype=torch.int32, **kw)
        self.c = capi.kvb_layer(
            k_code=self.k_code.data_ptr(), k_scale=self.k_scale.data_ptr(), v_code=self.v_code.data_ptr(),
            v_scale=self.v_scale.data_ptr(), stage=self.stage.data_ptr(), table_direct=self.table.data_ptr(),
            tables=None, table_rows=None, table_stride=0, table_len=self.table.numel(), pages=pages,
            kv_heads=kv_heads, q_heads=q_heads, head_dim=head_dim,
            dtype=capi.DTYPE_BF16 if dtype == torch.bfloat16 else capi.DTYPE_F16, sinkhorn_iters=sinkhorn_iters,
            error_word=self.error_word.data_ptr())
        self._ws = None
        self._pws = None

    # ---- kv_cache_append_kvarn128_launch
    def append(self, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor) -> None:
        """k, v: [tokens, kv_heads, head_dim]; positions: int32 [tokens] on the device, contiguous."""
        capi.check(capi.load().kvb_append(C.byref(self.c), _ptr(k), _ptr(v), _ptr(positions), int(k.shape[0]), _stream()))

    # ---- kvarn128_decode_tile
    def decode_tile(self, tile: int, head: int):
        ok = torch.empty((TILE, self.head_dim), dtype=torch.float16, device=self.device)
        ov = torch.empty_like(ok)
        capi.check(capi.load().kvb_decode_tile(C.byref(self.c), tile, head, _ptr(ok), _ptr(ov), _stream()))
        return ok, ov

    def workspace(self, kv_len_max: int, rows: int) -> torch.Tensor:
        """Scratch for attention calls of up to `rows` query tokens at up to `kv_len_max` keys.  One buffer per
        layer that only ever grows: a CUDA graph that captured its address stays valid as long as the first call
        (made before the capture) asked for the largest shape the graph uses."""
        n = capi.load().kvb_workspace_bytes(kv_len_max, self.kv_heads, self.q_heads, self.head_dim, rows, 1)
        if self._ws is None or self._ws.numel() * 4 < n:
            self._ws = torch.empty((n + 3) // 4, dtype=torch.float32, device=self.device)
        return self._ws

    def prefill_workspace(self, kv_len_max: int, tokens: int) -> torch.Tensor:
        n = capi.load().kvb_prefill_workspace_bytes(kv_len_max, self.kv_heads, self.q_heads, self.head_dim, tokens)
        if self._pws is None or self._pws.numel() * 4 < n:
            self._pws = torch.empty((n + 3) // 4, dtype=torch.float32, device=self.device)
        return self._pws

    # ---- causal_attention_cached_small_t_launch
    def attn_decode(self, q: torch.Tensor, pos: torch.Tensor, scale: float, kv_len_max: int, out=None) -> torch.Tensor:
        out = torch.empty_like(q) if out is None else out
        capi.check(capi.load().kvb_attn_decode(C.byref(self.c), _ptr(q), _ptr(pos), scale, kv_len_max,
                                               _ptr(self.workspace(kv_len_max, 1)), _ptr(out), _stream()))
        return out

    # ---- one decode step: kv_cache_append_launch + causal_attention_cached_small_t_launch as one call
    def append_decode(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos: torch.Tensor, scale: float, kv_len_max: int,
                      out=None, ring=None) -> torch.Tensor:
        """k, v: [1, kv_heads, head_dim] (or [kv_heads, head_dim]); pos: int32 [1] on the device.  `ring`: a
        sharded.PeerRing when this cache is the last tile range of a range-sharded sequence."""
        out = torch.empty_like(q) if out is None else out
        capi.check(capi.load().kvb_append_decode(C.byref(self.c), _ptr(q), _ptr(k), _ptr(v), _ptr(pos), scale, kv_len_max,
                                                 _ptr(self.workspace(kv_len_max, 1)), None if ring is None else C.byref(ring.c),
                                                 _ptr(out), _stream()))
        return out

    def attn_decode_partial(self, q, pos, scale, kv_len_max, key_begin=0, key_end=2**31 - 1):
        m = torch.empty(self.q_heads, dtype=torch.float32, device=self.device)
        l = torch.empty_like(m)
        o = torch.empty((self.q_heads, self.head_dim), dtype=torch.float32, device=self.device)
        capi.check(capi.load().kvb_attn_decode_partial(C.byref(self.c), _ptr(q), _ptr(pos), scale, kv_len_max, key_begin,
                                                       key_end, _ptr(self.workspace(kv_len_max, 1)), _ptr(m), _ptr(l),
                                                       _ptr(o), _stream()))
        return m, l, o

    def attn_decode_partial_packed(self, q, pos, scale, kv_len_max, packed):
        """Partial into one caller buffer laid out m[QH] | l[QH] | o[QH, D] (fp32, QH * (D + 2) floats)."""
        qh, d = self.q_heads, self.head_dim
        base = packed.data_ptr()
        capi.check(capi.load().kvb_attn_decode_partial(C.byref(self.c), _ptr(q), _ptr(pos), scale, kv_len_max, 0, 2**31 - 1,
                                                       _ptr(self.workspace(kv_len_max, 1)), C.c_void_p(base),
                                                       C.c_void_p(base + 4 * qh), C.c_void_p(base + 8 * qh), _stream()))
        return packed

    # ---- causal_attention_small_t_launch (append + causal attention of 1..8 rows)
    def attn_verify(self, q, k, v, positions, scale, kv_len_max, out=None):
        out = torch.empty_like(q) if out is None else out
        w = int(q.shape[0])
        capi.check(capi.load().kvb_attn_verify(C.byref(self.c), _ptr(q), _ptr(k), _ptr(v), _ptr(positions), w, scale,
                                               kv_len_max, _ptr(self.workspace(kv_len_max, w)), _ptr(out), _stream()))
        return out

    # ---- causal_attention_prompt_launch (quantise-append a chunk + causal chunk attention)
    def attn_prefill(self, q, k, v, positions, scale, kv_len_max, out=None):
        out = torch.empty_like(q) if out is None else out
        ws = self.prefill_workspace(kv_len_max, int(q.shape[0]))
        capi.check(capi.load().kvb_attn_prefill(C.byref(self.c), _ptr(q), _ptr(k), _ptr(v), _ptr(positions),
                                                int(q.shape[0]), scale, kv_len_max, _ptr(ws), _ptr(out), _stream()))
        return out

    # ---- this cache's share of a verify step / prefill chunk over a range-sharded sequence
    def attn_chunk_partial_packed(self, q, positions, scale, kv_len_max, packed):
        """q: [tokens, q_heads, head_dim]; positions: int32 [tokens] in this cache's coordinates.  Writes the partials
        of the tokens * q_heads rows into `packed`, laid out m[rows] | l[rows] | o[rows, D] (fp32, rows * (D + 2) floats)."""
        tokens = int(q.shape[0])
        rows, d = tokens * self.q_heads, self.head_dim
        ws = self.workspace(kv_len_max, tokens) if tokens <= 8 else self.prefill_workspace(kv_len_max, tokens)
        base = packed.data_ptr()
        capi.check(capi.load().kvb_attn_chunk_partial(C.byref(self.c), _ptr(q), _ptr(positions), tokens, scale, kv_len_max, _ptr(ws),
                                                      C.c_void_p(base), C.c_void_p(base + 4 * rows), C.c_void_p(base + 8 * rows), _stream()))
        return packed

    def errors(self) -> int:
        return int(self.error_word.item())


class DecodeBatch:
    """kvb_attn_decode_batch over a fixed set of sequences (up to 64): the layer descriptors are uploaded once, the
    grid is shaped by the host's bounds of the lengths (`kv_len_max`, fixed for the life of the object)."""

    def __init__(self, layers, kv_len_max):
        lib = capi.load()
        first = layers[0]
        assert all((L.head_dim, L.kv_heads, L.q_heads, L.dtype) == (first.head_dim, first.kv_heads, first.q_heads, first.dtype) for L in layers)
        self.layers, self.n = list(layers), len(layers)
        self.geo = (first.kv_heads, first.q_heads, first.head_dim, capi.DTYPE_BF16 if first.dtype == torch.bfloat16 else capi.DTYPE_F16)
        raw = b"".join(bytes(L.c) for L in layers)
        self.descriptors = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(first.device)
        self.bounds = (C.c_int32 * self.n)(*[int(x) for x in kv_len_max])
        nbytes = lib.kvb_batch_workspace_bytes(self.bounds, self.n, first.kv_heads, first.q_heads, first.head_dim)
        if nbytes == 0:
            raise ValueError("kvb_batch_workspace_bytes refused the batch: " + lib.kvb_last_error_string().decode())
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=first.device)

    def attn_decode(self, q: torch.Tensor, pos: torch.Tensor, scale: float, out=None) -> torch.Tensor:
        """q: [n, q_heads, head_dim]; pos: int32 [n] on the device -> out [n, q_heads, head_dim]."""
        out = torch.empty_like(q) if out is None else out
        kv_heads, q_heads, head_dim, dtype = self.geo
        capi.check(capi.load().kvb_attn_decode_batch(_ptr(self.descriptors), self.n, kv_heads, q_heads, head_dim, dtype, _ptr(q), _ptr(pos),
                                                     scale, self.bounds, _ptr(self.workspace), _ptr(out), _stream()))
        return out


def merge_partials(m: torch.Tensor, l: torch.Tensor, o: torch.Tensor, dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """m, l: [parts, q_heads]; o: [parts, q_heads, head_dim] -> [q_heads, head_dim]."""
    parts, qh, d = o.shape
    out = torch.empty((qh, d), dtype=dtype, device=o.device)
    capi.check(capi.load().kvb_merge_partials(_ptr(m.contiguous()), _ptr(l.contiguous()), _ptr(o.contiguous()), parts, qh, d,
                                              capi.DTYPE_BF16 if dtype == torch.bfloat16 else capi.DTYPE_F16, _ptr(out),
                                              _stream()))
    return out


def merge_partials_packed(packed: torch.Tensor, parts: int, q_heads: int, head_dim: int, out: torch.Tensor) -> torch.Tensor:
    """packed: parts blocks of m[QH] | l[QH] | o[QH, D] -> out [q_heads, head_dim]."""
    capi.check(capi.load().kvb_merge_partials_packed(_ptr(packed), parts, q_heads, head_dim,
                                                     capi.DTYPE_BF16 if out.dtype == torch.bfloat16 else capi.DTYPE_F16,
                                                     _ptr(out), _stream()))
    return out


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
