"""CPU tests: the C restatement of the codec against the reference's golden records, slot map and
(when it was compiled here) the reference's own oracle."""
import csv
import os

import numpy as np
import pytest

from conftest import GOLDEN


def test_fp16_conversion_matches_numpy(oracle):
    rng = np.random.default_rng(1)
    xs = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1, 100, 7e4)])
    xs = np.concatenate([xs, np.array([0.0, -0.0, 65504.0, 65520.0, 65519.99, 6.1e-5, 5.96e-8, 2.98e-8, 2.9802322e-8,
                                       np.inf, -np.inf], np.float32)])
    want = xs.astype(np.float16).view(np.uint16)
    got = np.array([oracle.lib().kvo_f32_to_f16(float(x)) for x in xs], np.uint16)
    assert np.array_equal(got, want)
    hs = np.arange(0, 65536, 7, dtype=np.uint16)
    back = np.array([oracle.lib().kvo_f16_to_f32(int(h)) for h in hs], np.float32)
    ref = hs.view(np.float16).astype(np.float32)
    assert np.array_equal(back[~np.isnan(ref)], ref[~np.isnan(ref)])


def test_golden_records_iters0_bit_exact(oracle):
    g = np.load(os.path.join(GOLDEN, "gvk2_it0.npz"))
    for name, tile, rec in zip(g["names"], g["tiles"], g["records"]):
        got, q, bc, br = oracle.quantize_tile(tile.astype(np.float32), 4, 0)
        assert np.array_equal(got, rec), name
        assert np.all(bc == 1.0) and np.all(br == 1.0)
        # payload nibble order: element (r, c) at bit 4*(r*128+c)
        flat = q.reshape(-1)
        assert np.array_equal(flat[0::2] | (flat[1::2] << 4), rec[:8192])


def test_golden_records_iters16(oracle):
    g = np.load(os.path.join(GOLDEN, "gvk2_it16.npz"))
    for name, tile, rec, sc, sr in zip(g["names"], g["tiles"], g["records"], g["s_col"], g["s_row"]):
        got, q, bc, br = oracle.quantize_tile(tile.astype(np.float32), 4, 16)
        # same host arithmetic as the reference oracle: identical factors and bytes
        assert np.array_equal(bc, sc) and np.array_equal(br, sr), name
        assert np.array_equal(got, rec), name


def test_golden_two_bit_records(oracle):
    """The reference's K4V2 tier: 2-bit V records (bit string, four codes per byte, low bits first), 16 iterations."""
    g = np.load(os.path.join(GOLDEN, "gvk2_v2.npz"))
    for name, tile, rec, iters in zip(g["names"], g["tiles"], g["records"], g["iters"]):
        got, q, _, _ = oracle.quantize_tile(tile.astype(np.float32), 2, int(iters))
        assert got.size == 128 * 128 * 2 // 8 + 384 * 2
        assert np.array_equal(got, rec), name
        flat = q.reshape(-1)
        assert flat.max() <= 3
        assert np.array_equal(flat[0::4] | (flat[1::4] << 2) | (flat[2::4] << 4) | (flat[3::4] << 6), rec[:4096])


def test_dequant_roundtrip_quality(oracle):
    g = np.load(os.path.join(GOLDEN, "gvk2_it0.npz"))
    tile = g["tiles"][0].astype(np.float32)
    rec, q, _, _ = oracle.quantize_tile(tile, 4, 0)
    deq = oracle.dequant_tile(rec, 128, 128, 4)
    cos = float((deq * tile).sum() / np.sqrt((deq * deq).sum() * (tile * tile).sum()))
    assert cos > 0.995
    # per-row affine code: error below half a step (+ fp16 rounding of the axes)
    step = (tile.max(1) - tile.min(1)) / 15
    assert np.all(np.abs(deq - tile).max(1) <= 0.5 * step * 1.01 + 2e-3 * np.abs(tile).max(1))


def test_slot_map_matches_reference_table(oracle):
    item_id = {"scale_axis": 0, "zp_axis": 1, "other_axis": 2}
    n = 0
    with open(os.path.join(GOLDEN, "p1_slot_map_k4v4.csv")) as f:
        for row in csv.DictReader(f):
            is_v = row["plane"].startswith("v_")
            item = item_id[row["item"][2:]]
            s, idx = int(row["slice"]), int(row["index"])
            dim_axis = (item != 2) if not is_v else (item == 2)
            index = s * 128 + idx if dim_axis else idx
            assert oracle.scale_slot(256, is_v, item, s, index) == (int(row["page_row"]), int(row["col"])), row
            n += 1
    assert n == 640 + 512


def test_byte_table(oracle):
    with open(os.path.join(GOLDEN, "byte_table.csv")) as f:
        for row in csv.DictReader(f):
            kb, vb = int(row["kb"]), int(row["vb"])
            rec = 2 * (oracle.lib().kvo_record_bytes(128, 128, kb) + oracle.lib().kvo_record_bytes(128, 128, vb)) // 128
            assert rec == int(row["record_b_per_token"])
            assert rec + 12 == int(row["p1_b_per_token"])


def test_hadamard_properties(oracle):
    rng = np.random.default_rng(3)
    for D in (128, 256):
        x = rng.standard_normal((5, D)).astype(np.float32)
        y = oracle.hadamard(x)
        assert np.allclose(oracle.hadamard(y), x, atol=2e-6)
        assert np.allclose((y * y).sum(1), (x * x).sum(1), rtol=1e-5)
        e = np.zeros((1, D), np.float32)
        e[0, 5] = 1.0
        h = oracle.hadamard(e)[0]
        sign = np.array([(-1) ** bin(5 & j).count("1") for j in range(D)], np.float32)
        norm = np.float32(0.0625) if D == 256 else np.float32(0.08838834764831845)
        assert np.array_equal(h, sign * norm)


@pytest.mark.skipif(not os.path.exists(os.path.join(os.path.dirname(GOLDEN), "..", "oracle", "_ref", "libbee_ref.so")),
                    reason="reference oracle not compiled on this box")
def test_port_equals_compiled_reference(oracle):
    rng = np.random.default_rng(11)
    for case in range(6):
        t = rng.standard_normal((128, 128)).astype(np.float32)
        if case % 2:
            t[[0, 7, 63]] *= 20.0
        t = t.astype(np.float16).astype(np.float32)
        for iters in (0, 3, 16):
            rec, q, bc, br = oracle.quantize_tile(t, 4, iters)
            rrec, rbc, rbr, _ = oracle.ref_quantize_tile(t, 4, iters)
            assert np.array_equal(rec, rrec) and np.array_equal(bc, rbc) and np.array_equal(br, rbr)
            assert np.array_equal(oracle.dequant_tile(rec, 128, 128), oracle.ref_dequant_tile(rrec, 128, 128))
    # the other widths of the reference's tier table (bit-string packing across byte boundaries for 3, 5, 6)
    t = rng.standard_normal((128, 128)).astype(np.float16).astype(np.float32)
    for bits in (2, 3, 5, 6, 8):
        for iters in (0, 16):
            rec, q, bc, br = oracle.quantize_tile(t, bits, iters)
            rrec, rbc, rbr, _ = oracle.ref_quantize_tile(t, bits, iters)
            assert rec.size == 128 * 128 * bits // 8 + 768 and np.array_equal(rec, rrec), (bits, iters)
            assert q.max() <= (1 << bits) - 1
            assert np.array_equal(oracle.dequant_tile(rec, 128, 128, bits), oracle.ref_dequant_tile(rrec, 128, 128, bits))
    xs = rng.standard_normal(5000).astype(np.float32) * 1e-6
    for x in xs:
        assert oracle.lib().kvo_f32_to_f16(float(x)) == oracle.ref().bee_ref_f32_to_f16(float(x))
