"""KV dump files of the reference: KVD1 (quantised records taken from the planes) and KVO1 (what the engine
de-quantised from them), which its host verifier reads (kvarn-evidence/verify-g128/README.md:45-135; the engine writes
the same two files under KVARN128_DUMP_DIR, kvarn-port/patches/0004-*.patch, kvarn128_launch.cu:680-718), and GVK2, the
record dump its byte-for-byte quantiser gate compares (kvarn-evidence/gate2-kvarn-quant/dump_oracle.cpp:725-729).

Host-side, numpy only: the planes are copied off the device by the caller.  A *record* is one 128 x 128 slice of
one (tile, head, K | V): K has row = dim, col = token; V has row = token, col = dim.  Its code bytes are the
row-major string of 4-bit codes, low nibble first; its scale block is scale_axis[rows] | zp_axis[rows] |
other_axis[cols] as fp16 bit patterns.  Everything little-endian, no padding.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

TILE, PAGE, SLICE = 128, 64, 128
KVD1_MAGIC, KVO1_MAGIC = 0x3144564B, 0x314F564B  # 'KVD1', 'KVO1'
GVK2_MAGIC = b"GVK2"


@dataclass
class Record:
    name: str
    kind: int                 # 0 = K (row = dim, col = token), 1 = V (row = token, col = dim)
    codes: np.ndarray         # uint8 [128 rows][128 cols], values 0..15
    scale_axis: np.ndarray    # uint16 [128] fp16 patterns, per row
    zp_axis: np.ndarray       # uint16 [128], per row
    other_axis: np.ndarray    # uint16 [128], per column
    tokens: int = TILE
    head_slices: int = 2
    bits: int = 4
    orig: Optional[np.ndarray] = None  # float32 [128][128] values before quantisation (rotated domain), row-major


@dataclass
class DecodedHead:
    name: str
    kind: int
    data: np.ndarray  # float32 [tokens][width]
    domain: int = 0   # 0 = rotated domain (what attention consumes), 1 = inverse rotation applied


def tile_records(k_code, k_scale, v_code, v_scale, table, tile: int, head: int, name: str = "",
                 stage_k=None, stage_v=None) -> List[Record]:
    """The 2 * S records of one sealed tile of one KV head, K slices first, read from planes shaped
    [pages][kv_heads][64][...] (codes uint8 [.., D/2]; scales fp16 or uint16 [.., 5S] and [.., 4S]).
    stage_k / stage_v: optional [128][D] fp16 rows of the tile before quantisation (-> the `orig` block)."""
    k_code, v_code = np.asarray(k_code), np.asarray(v_code)
    k_scale = np.asarray(k_scale).view(np.uint16)
    v_scale = np.asarray(v_scale).view(np.uint16)
    D = k_code.shape[-1] * 2
    S = D // SLICE
    c = 2 * S  # dim-axis entries per scale row
    pages = [int(table[2 * tile]), int(table[2 * tile + 1])]
    out: List[Record] = []
    for kind, code, scale in ((0, k_code, k_scale), (1, v_code, v_scale)):
        rows = np.concatenate([code[p, head] for p in pages], axis=0)            # [128 tok][D/2]
        nib = np.empty((TILE, D), np.uint8)                                       # [tok][dim]
        nib[:, 0::2] = rows & 15
        nib[:, 1::2] = rows >> 4
        sc = [scale[p, head] for p in pages]                                      # 2 x [64][5S | 4S]
        tok_axis = np.concatenate(sc, axis=0)                                     # [128 tok][cols]
        dim_block = sc[0]                                                         # dim-axis entries: same in both pages
        for s in range(S):
            dims = np.arange(s * SLICE, (s + 1) * SLICE)
            if kind == 0:
                codes = nib[:, dims].T.copy()                                     # [dim][tok]
                scale_axis = dim_block[dims // c, dims % c]
                zp_axis = dim_block[dims // c, c + dims % c]
                other_axis = tok_axis[:, 2 * c + s]
                stage = stage_k
            else:
                codes = nib[:, dims].copy()                                       # [tok][dim]
                other_axis = dim_block[dims // c, dims % c]
                scale_axis = tok_axis[:, c + s]
                zp_axis = tok_axis[:, c + S + s]
                stage = stage_v
            orig = None
            if stage is not None:
                x = np.asarray(stage).view(np.float16).reshape(TILE, D)[:, dims].astype(np.float32)
                orig = x.T.copy() if kind == 0 else x.copy()
            out.append(Record(f"{name}{'KV'[kind]}_t{tile}_h{head}_s{s}", kind, codes, scale_axis.astype(np.uint16),
                              zp_axis.astype(np.uint16), other_axis.astype(np.uint16), TILE, S, 4, orig))
    return out


def decoded_heads(decoded_k, decoded_v, tile: int, head: int, name: str = "") -> List[DecodedHead]:
    """KVO1 heads for one tile from the output of kvb_decode_tile ([128][D] fp16 each, rotated domain)."""
    k = np.asarray(decoded_k).view(np.float16).astype(np.float32)
    v = np.asarray(decoded_v).view(np.float16).astype(np.float32)
    return [DecodedHead(f"{name}K_t{tile}_h{head}", 0, k, 0), DecodedHead(f"{name}V_t{tile}_h{head}", 1, v, 0)]


def _pack_codes(codes: np.ndarray) -> bytes:
    flat = np.ascontiguousarray(codes, dtype=np.uint8).reshape(-1)
    return (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8).tobytes()


def write_kvd1(path: str, records: Sequence[Record]) -> None:
    with open(path, "wb") as f:
        f.write(struct.pack("<III", KVD1_MAGIC, 1, len(records)))
        for r in records:
            name = r.name.encode("utf-8")
            rows, cols = r.codes.shape
            f.write(struct.pack("<I", len(name)) + name)
            f.write(struct.pack("<7i", r.kind, r.bits, rows, cols, r.tokens, max(1, (r.tokens + PAGE - 1) // PAGE), r.head_slices))
            f.write(struct.pack("<I", 1 if r.orig is not None else 0))
            code = _pack_codes(r.codes)
            f.write(struct.pack("<I", len(code)) + code)
            scale = np.concatenate([r.scale_axis, r.zp_axis, r.other_axis]).astype("<u2")
            f.write(struct.pack("<I", scale.size) + scale.tobytes())
            if r.orig is not None:
                o = np.ascontiguousarray(r.orig, dtype="<f4")
                f.write(struct.pack("<I", o.size) + o.tobytes())


def read_kvd1(path: str) -> List[Record]:
    buf = open(path, "rb").read()
    magic, version, n = struct.unpack_from("<III", buf, 0)
    if magic != KVD1_MAGIC or version != 1:
        raise ValueError("not a KVD1 version 1 file")
    off, out = 12, []
    for _ in range(n):
        (nl,) = struct.unpack_from("<I", buf, off); off += 4
        name = buf[off:off + nl].decode("utf-8"); off += nl
        kind, bits, rows, cols, tokens, _pages, slices = struct.unpack_from("<7i", buf, off); off += 28
        (flags,) = struct.unpack_from("<I", buf, off); off += 4
        (cb,) = struct.unpack_from("<I", buf, off); off += 4
        if bits != 4 or cb != rows * cols // 2:
            raise ValueError("only 4-bit records are handled here")
        packed = np.frombuffer(buf, np.uint8, cb, off); off += cb
        codes = np.empty(rows * cols, np.uint8)
        codes[0::2], codes[1::2] = packed & 15, packed >> 4
        (sh,) = struct.unpack_from("<I", buf, off); off += 4
        scale = np.frombuffer(buf, "<u2", sh, off).astype(np.uint16); off += 2 * sh
        orig = None
        if flags & 1:
            (nf,) = struct.unpack_from("<I", buf, off); off += 4
            orig = np.frombuffer(buf, "<f4", nf, off).reshape(rows, cols).copy(); off += 4 * nf
        out.append(Record(name, kind, codes.reshape(rows, cols), scale[:rows], scale[rows:2 * rows], scale[2 * rows:], tokens, slices,
                          bits, orig))
    return out


def write_kvo1(path: str, heads: Sequence[DecodedHead]) -> None:
    with open(path, "wb") as f:
        f.write(struct.pack("<III", KVO1_MAGIC, 1, len(heads)))
        for h in heads:
            name = h.name.encode("utf-8")
            data = np.ascontiguousarray(h.data, dtype="<f4")
            tokens, width = data.shape
            f.write(struct.pack("<I", len(name)) + name)
            f.write(struct.pack("<4i", h.kind, tokens, width, h.domain))
            f.write(struct.pack("<I", data.size) + data.tobytes())


def read_kvo1(path: str) -> List[DecodedHead]:
    buf = open(path, "rb").read()
    magic, version, n = struct.unpack_from("<III", buf, 0)
    if magic != KVO1_MAGIC or version != 1:
        raise ValueError("not a KVO1 version 1 file")
    off, out = 12, []
    for _ in range(n):
        (nl,) = struct.unpack_from("<I", buf, off); off += 4
        name = buf[off:off + nl].decode("utf-8"); off += nl
        kind, tokens, width, domain = struct.unpack_from("<4i", buf, off); off += 16
        (nf,) = struct.unpack_from("<I", buf, off); off += 4
        data = np.frombuffer(buf, "<f4", nf, off).reshape(tokens, width).copy(); off += 4 * nf
        out.append(DecodedHead(name, kind, data, domain))
    return out


def dequantise(record: Record) -> np.ndarray:
    """(q * scale_axis[r] + zp_axis[r]) * other_axis[c] in fp32 with separate roundings, [rows][cols]."""
    q = record.codes.astype(np.float32)
    s = record.scale_axis.view(np.float16).astype(np.float32)[:, None]
    z = record.zp_axis.view(np.float16).astype(np.float32)[:, None]
    o = record.other_axis.view(np.float16).astype(np.float32)[None, :]
    return ((q * s).astype(np.float32) + z).astype(np.float32) * o


# ---------------------------------------------------------------------------------------------------------------
# GVK2: per record the quantiser's input tile (fp32, already fp16-exact), the balancing factors it settled on and
# the full record bytes = code payload | scale_axis | zp_axis | other_axis (fp16), the layout of the reference
# oracle's record (bee_oracle.cpp:309-314).
@dataclass
class Gvk2Entry:
    name: str
    bits: int
    iters: int
    best_iter: int
    best_imbalance: float
    s_col: np.ndarray   # float32 [cols]
    s_row: np.ndarray   # float32 [rows]
    tile: np.ndarray    # float32 [rows][cols]
    record: np.ndarray  # uint8 [rows * cols * bits / 8 + 2 * (2 * rows + cols)]


def record_bytes(record: Record) -> np.ndarray:
    """The reference's record byte string of a 4-bit plane record: row-major codes, low nibble first, then the three
    fp16 axes."""
    if record.bits != 4:
        raise ValueError("plane records are 4-bit")
    axes = np.concatenate([record.scale_axis, record.zp_axis, record.other_axis]).astype("<u2")
    return np.concatenate([np.frombuffer(_pack_codes(record.codes), np.uint8), axes.view(np.uint8)])


def gvk2_entry(record: Record, iters: int = 0, s_col=None, s_row=None, best_iter: int = 0, best_imbalance: float = 0.0) -> Gvk2Entry:
    """A GVK2 entry from a plane record that carries its un-quantised values (`orig`, from the stage rows).  With
    iters = 0 the balancing factors are all ones, as in the reference's iters-0 dumps."""
    if record.orig is None:
        raise ValueError("the record has no `orig` block: pass stage_k / stage_v to tile_records")
    rows, cols = record.codes.shape
    s_col = np.ones(cols, np.float32) if s_col is None else np.asarray(s_col, np.float32)
    s_row = np.ones(rows, np.float32) if s_row is None else np.asarray(s_row, np.float32)
    return Gvk2Entry(record.name, record.bits, iters, best_iter, best_imbalance, s_col, s_row,
                     np.ascontiguousarray(record.orig, np.float32), record_bytes(record))


def write_gvk2(path: str, entries: Sequence[Gvk2Entry]) -> None:
    with open(path, "wb") as f:
        f.write(GVK2_MAGIC + struct.pack("<II", 2, len(entries)))
        for e in entries:
            name = e.name.encode("utf-8")
            rows, cols = e.tile.shape
            f.write(struct.pack("<I", len(name)) + name)
            f.write(struct.pack("<5i", rows, cols, e.bits, e.iters, e.best_iter))
            f.write(struct.pack("<f", e.best_imbalance))
            f.write(np.ascontiguousarray(e.s_col, "<f4").tobytes())
            f.write(np.ascontiguousarray(e.s_row, "<f4").tobytes())
            f.write(np.ascontiguousarray(e.tile, "<f4").tobytes())
            rec = np.ascontiguousarray(e.record, np.uint8)
            f.write(struct.pack("<I", rec.size) + rec.tobytes())


def read_gvk2(path: str) -> List[Gvk2Entry]:
    b = open(path, "rb").read()
    if b[:4] != GVK2_MAGIC or struct.unpack_from("<I", b, 4)[0] != 2:
        raise ValueError("not a GVK2 version 2 file")
    (n,) = struct.unpack_from("<I", b, 8)
    o, out = 12, []
    for _ in range(n):
        (nl,) = struct.unpack_from("<I", b, o); o += 4
        name = b[o:o + nl].decode("utf-8"); o += nl
        rows, cols, bits, iters, best_iter = struct.unpack_from("<5i", b, o); o += 20
        (imb,) = struct.unpack_from("<f", b, o); o += 4
        s_col = np.frombuffer(b, "<f4", cols, o).copy(); o += 4 * cols
        s_row = np.frombuffer(b, "<f4", rows, o).copy(); o += 4 * rows
        tile = np.frombuffer(b, "<f4", rows * cols, o).reshape(rows, cols).copy(); o += 4 * rows * cols
        (rl,) = struct.unpack_from("<I", b, o); o += 4
        rec = np.frombuffer(b, np.uint8, rl, o).copy(); o += rl
        out.append(Gvk2Entry(name, bits, iters, best_iter, imb, s_col, s_row, tile, rec))
    if o != len(b):
        raise ValueError("trailing bytes after the last GVK2 record")
    return out
