"""CPU tests of the boundary: the library loads, exports every symbol the header declares, and rejects bad
arguments on the host before any launch (no GPU needed for these paths)."""
import ctypes as C
import os
import re

import pytest

from helpers import ROOT, pkg


def test_library_exports_every_declared_symbol():
    p = pkg()
    p.build()
    lib = p.capi.load()
    header = open(os.path.join(ROOT, "include", "kvarn_b200.h")).read()
    declared = set(re.findall(r"\b(kvb_[a-z_0-9]+)\s*\(", header))
    declared -= {"kvb_status", "kvb_layer"}
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(p.capi.SYMBOLS) == declared


def test_sizes():
    lib = pkg().capi.load()
    assert lib.kvb_stage_bytes(128, 4) == 2 * 2 * 4 * 128 * 128 * 2
    assert lib.kvb_stage_bytes(256, 4) == 1 << 20
    assert [lib.kvb_plane_bytes(w, 128, 4, 2) for w in range(4)] == [4096 * 8, 640 * 8, 4096 * 8, 512 * 8]
    assert [lib.kvb_plane_bytes(w, 256, 1, 1) for w in range(4)] == [8192, 1280, 8192, 1024]
    assert [lib.kvb_record_bytes(b) for b in (2, 3, 4, 5, 6, 8)] == [2048 * b + 768 for b in (2, 3, 4, 5, 6, 8)]
    assert lib.kvb_record_bytes(1) == 0 and lib.kvb_record_bytes(7) == 0
    assert lib.kvb_records_encode(None, 0, 4, None, None) == 0  # nothing to do: no launch
    assert lib.kvb_records_encode(None, 1, 4, None, None) == pkg().capi.KVB_EINVAL
    assert lib.kvb_records_decode(None, 0, 7, None, None) == pkg().capi.KVB_EINVAL
    assert lib.kvb_split_capacity(32768, 4, 24, 1, 1) >= 2
    assert lib.kvb_workspace_bytes(32768, 4, 24, 128, 1, 1) > 0


@pytest.mark.parametrize("kv_heads,q_heads,kv_len_max", [(4, 12, 4608), (3, 9, 6144), (7, 21, 2560), (4, 24, 32768), (2, 16, 9000),
                                                         (1, 7, 12000), (8, 8, 5000), (4, 24, 378944)])
def test_workspace_covers_every_narrower_call(kv_heads, q_heads, kv_len_max):
    """A workspace sized for `rows` query tokens must hold every call of 1..rows tokens: the number of splits (hence of
    partials) is not monotonic in the width, so the size query takes the maximum over the widths."""
    lib = pkg().capi.load()
    sizes = [lib.kvb_workspace_bytes(kv_len_max, kv_heads, q_heads, 128, r, 1) for r in range(1, 9)]
    assert all(a <= b for a, b in zip(sizes, sizes[1:])), sizes
    G = q_heads // kv_heads
    for r in range(1, 9):
        zblocks = (r * G + 15) // 16
        parts = lib.kvb_split_capacity(kv_len_max, kv_heads, q_heads, r, 1)
        assert sizes[r - 1] >= kv_heads * zblocks * parts * 16 * (128 + 2) * 4, (r, parts)


def _layer(capi, **over):
    L = capi.kvb_layer(k_code=16, k_scale=16, v_code=16, v_scale=16, stage=16, table_direct=16, tables=None,
                       table_rows=None, table_stride=0, table_len=4, pages=4, kv_heads=4, q_heads=24, head_dim=128,
                       dtype=0, sinkhorn_iters=0, error_word=None)
    for k, v in over.items():
        setattr(L, k, v)
    return L


@pytest.mark.parametrize("over", [dict(kv_heads=0), dict(kv_heads=9), dict(head_dim=64), dict(q_heads=25), dict(dtype=3),
                                  dict(k_code=None), dict(table_direct=None), dict(pages=0), dict(sinkhorn_iters=-1)])
def test_bad_layer_is_rejected_on_the_host(over, capfd):
    capi = pkg().capi
    lib = capi.load()
    L = _layer(capi, **over)
    st = lib.kvb_append(C.byref(L), 16, 16, 16, 1, None)
    assert st == capi.KVB_EINVAL
    assert lib.kvb_last_error_string()
    assert "kvarn_b200:" in capfd.readouterr().err  # loud failure, like the reference's fprintf before it throws


def test_null_arguments_and_ranges():
    capi = pkg().capi
    lib = capi.load()
    L = _layer(capi)
    assert lib.kvb_append(C.byref(L), None, 16, 16, 1, None) == capi.KVB_EINVAL
    assert lib.kvb_append(C.byref(L), 16, 16, 16, 0, None) == capi.KVB_OK  # empty append: silent no-op
    assert lib.kvb_append(C.byref(L), 16, 16, 16, -1, None) == capi.KVB_EINVAL
    assert lib.kvb_decode_tile(C.byref(L), 5, 0, 16, 16, None) == capi.KVB_EINVAL
    assert lib.kvb_attn_decode(C.byref(L), None, 16, 0.1, 128, 16, 16, None) == capi.KVB_EINVAL
    assert lib.kvb_attn_verify(C.byref(L), 16, 16, 16, 16, 9, 0.1, 128, 16, 16, None) == capi.KVB_ERANGE
    assert lib.kvb_merge_partials(None, 16, 16, 2, 24, 128, 0, 16, None) == capi.KVB_EINVAL
    with pytest.raises(capi.KvarnError):
        capi.check(capi.KVB_EINVAL)
