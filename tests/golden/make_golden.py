#!/usr/bin/env python3
"""Regenerates the golden fixtures in this directory from the reference repository.

Run where a checkout of the reference is available:  python tests/golden/make_golden.py REFERENCE_ROOT

Fixtures written (all derived from data files of the reference, no source code):
  gvk2_it0.npz    8 of the 32 GVK2 records of kvarn-evidence/verify-g128/data/real_k4v4_it0.bin
                  (Sinkhorn iterations 0): input tile (already fp16-exact, stored as fp16) and the
                  full record bytes the reference oracle produced for it.
  gvk2_it16.npz   4 records of .../real_k4v4.bin (16 iterations) with the reference's s_col/s_row.
  gvk2_v2.npz     4 two-bit V records of .../real_k4v2.bin (16 iterations): the bit-string packing at a width
                  other than 4.
  p1_slot_map_k4v4.csv   the K4V4 rows of kvarn-evidence/offsets-g128/out/p1_slot_map_g128.csv
                  (plane, page_row, col, item, slice, index): the slot of every axis entry in a
                  scale page at head_dim 256.
  byte_table.csv  per-token byte accounting of the 36 bit tiers (offsets_p1_g128.csv, 5 columns).
"""
import csv
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def read_gvk2(path):
    b = open(path, "rb").read()
    magic, ver, n = struct.unpack_from("<4sII", b, 0)
    assert magic == b"GVK2" and ver == 2
    o, out = 12, []
    for _ in range(n):
        (nl,) = struct.unpack_from("<I", b, o); o += 4
        name = b[o:o + nl].decode(); o += nl
        rows, cols, bits, iters, best_iter = struct.unpack_from("<5i", b, o); o += 20
        (imb,) = struct.unpack_from("<f", b, o); o += 4
        s_col = np.frombuffer(b, "<f4", cols, o).copy(); o += 4 * cols
        s_row = np.frombuffer(b, "<f4", rows, o).copy(); o += 4 * rows
        tile = np.frombuffer(b, "<f4", rows * cols, o).reshape(rows, cols).copy(); o += 4 * rows * cols
        (rl,) = struct.unpack_from("<I", b, o); o += 4
        rec = np.frombuffer(b, np.uint8, rl, o).copy(); o += rl
        out.append(dict(name=name, rows=rows, cols=cols, bits=bits, iters=iters, best_iter=best_iter, imb=imb,
                        s_col=s_col, s_row=s_row, tile=tile, rec=rec))
    assert o == len(b)
    return out


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("KVB_REFERENCE_ROOT", "")
    if not os.path.isdir(os.path.join(root, "kvarn-evidence")):
        sys.exit("reference sources absent: pass the reference checkout as the first argument or set KVB_REFERENCE_ROOT")
    ev = os.path.join(root, "kvarn-evidence")
    it0 = read_gvk2(os.path.join(ev, "verify-g128/data/real_k4v4_it0.bin"))
    pick = [r for r in it0 if r["name"] in (
        "L35_k_h0_s0_g0", "L35_k_h1_s1_g0", "L63_k_h2_s0_g0", "L63_k_h3_s1_g0",
        "L35_v_h0_s0_g0", "L35_v_h1_s1_g0", "L63_v_h2_s0_g0", "L63_v_h3_s1_g0")]
    assert len(pick) == 8
    for r in pick:
        assert np.array_equal(r["tile"].astype(np.float16).astype(np.float32), r["tile"])
    np.savez_compressed(os.path.join(HERE, "gvk2_it0.npz"), names=np.array([r["name"] for r in pick]),
                        tiles=np.stack([r["tile"].astype(np.float16) for r in pick]),
                        records=np.stack([r["rec"] for r in pick]))
    it16 = read_gvk2(os.path.join(ev, "verify-g128/data/real_k4v4.bin"))
    pick = [r for r in it16 if r["name"] in ("L35_k_h0_s0_g0", "L63_k_h3_s1_g0", "L35_v_h0_s0_g0", "L63_v_h3_s1_g0")]
    assert len(pick) == 4 and all(r["iters"] == 16 for r in pick)
    np.savez_compressed(os.path.join(HERE, "gvk2_it16.npz"), names=np.array([r["name"] for r in pick]),
                        tiles=np.stack([r["tile"].astype(np.float16) for r in pick]),
                        records=np.stack([r["rec"] for r in pick]),
                        s_col=np.stack([r["s_col"] for r in pick]), s_row=np.stack([r["s_row"] for r in pick]),
                        best_iter=np.array([r["best_iter"] for r in pick]))
    v2 = read_gvk2(os.path.join(ev, "verify-g128/data/real_k4v2.bin"))
    pick = [r for r in v2 if r["name"] in ("L35_v_h0_s0_g0", "L35_v_h3_s1_g0", "L63_v_h1_s0_g0", "L63_v_h2_s1_g0")]
    assert len(pick) == 4 and all(r["bits"] == 2 for r in pick)
    np.savez_compressed(os.path.join(HERE, "gvk2_v2.npz"), names=np.array([r["name"] for r in pick]),
                        tiles=np.stack([r["tile"].astype(np.float16) for r in pick]),
                        records=np.stack([r["rec"] for r in pick]), iters=np.array([r["iters"] for r in pick]))
    with open(os.path.join(ev, "offsets-g128/out/p1_slot_map_g128.csv")) as f, \
            open(os.path.join(HERE, "p1_slot_map_k4v4.csv"), "w", newline="") as g:
        w = csv.writer(g)
        w.writerow(["plane", "page_row", "col", "item", "slice", "index"])
        for row in csv.DictReader(f):
            if row["tier"] == "K4V4" and row["plane"].endswith("scale_pages"):
                w.writerow([row["plane"], row["page_row"], row["col"], row["item"], row["slice"], row["index"]])
    with open(os.path.join(ev, "offsets-g128/out/offsets_p1_g128.csv")) as f, \
            open(os.path.join(HERE, "byte_table.csv"), "w", newline="") as g:
        w = csv.writer(g)
        w.writerow(["kb", "vb", "p1_b_per_token", "record_b_per_token"])
        for row in csv.DictReader(f):
            w.writerow([row["kb"], row["vb"], row["p1_b_per_token"], row["record_b_per_token"]])


if __name__ == "__main__":
    main()
