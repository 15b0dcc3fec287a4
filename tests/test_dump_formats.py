"""KV dump files (KVD1 records from the planes, KVO1 de-quantised tiles, GVK2 quantiser records): round trip through the reader, equality
with the oracle's tile decode, and -- when the reference's own host verifier has been built into oracle/_ref --
its verdict on files written from these planes (it must say PASS, and must say FAIL for a poisoned decode, the
reference's own negative control, kvarn-evidence/verify-g128/README.md:170-172)."""
import os
import subprocess

import numpy as np
import pytest

from helpers import ROOT, pkg
from oracle import kvarn_oracle as orc

VERIFY = os.path.join(ROOT, "oracle", "_ref", "kvarn_g128_verify")


def _filled_cpu_layer(D, H, iters=0, seed=21):
    pages = 4
    cpu = orc.CpuLayer(D, H, pages, orc.shuffled_table(seed, pages, pages), iters=iters)
    k, v = orc.synth_kv(seed + 1, 128, H, D, 1), orc.synth_kv(seed + 1, 128, H, D, 2)
    cpu.append(k, v, 0)
    return cpu


def _files_from(layer_like, decode_tile, D, H, tmp_path, stage=None, poison=False):
    dump = pkg().dump
    recs, heads = [], []
    for h in range(H):
        sk = None if stage is None else stage[0, 0, h]
        sv = None if stage is None else stage[1, 0, h]
        recs += dump.tile_records(layer_like.k_code, layer_like.k_scale, layer_like.v_code, layer_like.v_scale, layer_like.table, 0, h,
                                  stage_k=sk, stage_v=sv)
        dk, dv = decode_tile(0, h)
        heads += dump.decoded_heads(dk, dv, 0, h)
    # the verifier pairs records and heads in file order: all records of a head's K, then of its V
    if poison:
        heads[0].data[7] = -heads[0].data[7]
    a, b = str(tmp_path / "planes.kvd"), str(tmp_path / "decoded.kvo")
    dump.write_kvd1(a, recs)
    dump.write_kvo1(b, heads)
    return a, b, recs, heads


@pytest.mark.parametrize("D", [128, 256])
def test_records_round_trip_and_equal_the_tile_decode(tmp_path, D):
    dump = pkg().dump
    cpu = _filled_cpu_layer(D, 2)
    a, b, recs, heads = _files_from(cpu, cpu.decode_tile, D, 2, tmp_path, stage=cpu.stage)
    back = dump.read_kvd1(a)
    assert len(back) == len(recs) == 2 * 2 * (D // 128)
    for r0, r1 in zip(recs, back):
        assert r0.name == r1.name and r0.kind == r1.kind and r0.head_slices == r1.head_slices
        assert np.array_equal(r0.codes, r1.codes) and np.array_equal(r0.scale_axis, r1.scale_axis)
        assert np.array_equal(r0.zp_axis, r1.zp_axis) and np.array_equal(r0.other_axis, r1.other_axis)
        assert np.array_equal(r0.orig, r1.orig)
    hb = dump.read_kvo1(b)
    assert all(np.array_equal(x.data, y.data) and x.name == y.name for x, y in zip(heads, hb))
    # de-quantising the records reproduces the oracle's tile decode exactly (fp16 rounding of the result)
    S = D // 128
    per_head = 2 * S
    for h in range(2):
        dk, dv = cpu.decode_tile(0, h)
        for s in range(S):
            rk, rv = recs[h * per_head + s], recs[h * per_head + S + s]
            assert np.array_equal(dump.dequantise(rk).T.astype(np.float16), dk[:, s * 128:(s + 1) * 128])
            assert np.array_equal(dump.dequantise(rv).astype(np.float16), dv[:, s * 128:(s + 1) * 128])


@pytest.mark.skipif(not os.path.exists(VERIFY), reason="the reference's verifier has not been built into oracle/_ref")
@pytest.mark.parametrize("iters", [0, 16])
def test_reference_verifier_accepts_the_dump_and_rejects_a_poisoned_decode(tmp_path, iters):
    cpu = _filled_cpu_layer(256, 2, iters=iters)
    a, b, _, _ = _files_from(cpu, cpu.decode_tile, 256, 2, tmp_path, stage=cpu.stage)
    r = subprocess.run([VERIFY, "--from-dump", a, "--decoded", b], capture_output=True, text=True)
    assert r.returncode == 0 and "PASS" in r.stdout.splitlines()[-1], r.stdout[-2000:]
    a, b, _, _ = _files_from(cpu, cpu.decode_tile, 256, 2, tmp_path, stage=cpu.stage, poison=True)
    r = subprocess.run([VERIFY, "--from-dump", a, "--decoded", b], capture_output=True, text=True)
    assert r.returncode != 0, r.stdout[-2000:]


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(VERIFY), reason="the reference's verifier has not been built into oracle/_ref")
@pytest.mark.parametrize("iters", [0, 16])
def test_reference_verifier_accepts_planes_written_by_the_gpu(tmp_path, iters):
    """Planes written by kvb_append and the tile decoded by kvb_decode_tile, judged by the reference's verifier."""
    import torch

    from helpers import Twin

    D, H = 256, 2
    tw = Twin(D=D, H=H, QH=4, capacity_tokens=128, seed=31, iters=iters)
    tw.append(orc.synth_kv(32, 128, H, D, 1), orc.synth_kv(32, 128, H, D, 2))
    torch.cuda.synchronize()
    g = tw.gpu

    class Host:
        k_code, v_code = g.k_code.cpu().numpy(), g.v_code.cpu().numpy()
        k_scale, v_scale = g.k_scale.cpu().numpy().view(np.uint16), g.v_scale.cpu().numpy().view(np.uint16)
        table = g.table.cpu().numpy()

    stage = g.stage.cpu().numpy().view(np.uint16).reshape(2, 2, H, 128, D)

    def decode(tile, head):
        k, v = g.decode_tile(tile, head)
        return k.cpu().numpy(), v.cpu().numpy()

    a, b, _, _ = _files_from(Host, decode, D, H, tmp_path, stage=stage)
    r = subprocess.run([VERIFY, "--from-dump", a, "--decoded", b], capture_output=True, text=True)
    assert r.returncode == 0 and "PASS" in r.stdout.splitlines()[-1], r.stdout[-2000:]
    assert g.errors() == 0


# --------------------------------------------------------------------------------------------------------------
# GVK2: the record dump of the reference's byte-for-byte quantiser gate.
GOLDEN = os.path.join(ROOT, "tests", "golden")
from conftest import REFERENCE_ROOT  # noqa: E402

REF_GVK2 = os.path.join(REFERENCE_ROOT, "kvarn-evidence", "verify-g128", "data", "real_k4v4_it0.bin")


def _stage_from_golden():
    """Stage rows [K|V][slot][head][token][dim] of one head_dim-256 tile of two heads built from the golden slices."""
    g = np.load(os.path.join(GOLDEN, "gvk2_it0.npz"))
    tiles = {n: t for n, t in zip(g["names"], g["tiles"])}
    recs = {n: r for n, r in zip(g["names"], g["records"])}
    kn = ["L35_k_h0_s0_g0", "L35_k_h1_s1_g0", "L63_k_h2_s0_g0", "L63_k_h3_s1_g0"]  # [dim][tok]
    vn = ["L35_v_h0_s0_g0", "L35_v_h1_s1_g0", "L63_v_h2_s0_g0", "L63_v_h3_s1_g0"]  # [tok][dim]
    stage = np.zeros((2, 2, 2, 128, 256), np.float16)
    for h in range(2):
        for s in range(2):
            stage[0, 0, h, :, s * 128:(s + 1) * 128] = tiles[kn[2 * h + s]].T
            stage[1, 0, h, :, s * 128:(s + 1) * 128] = tiles[vn[2 * h + s]]
    return stage, tiles, recs, kn, vn


def test_gvk2_records_cut_from_planes_equal_the_golden_bytes(tmp_path):
    """Planes written by the oracle's append from the golden tiles (rotation skipped: the golden slices are already
    rotated, they go straight into the stage and the oracle seals the tile), cut into records, written as GVK2 and
    read back: every record equals the reference's golden record byte for byte."""
    import ctypes as C

    dump = pkg().dump
    stage, tiles, recs, kn, vn = _stage_from_golden()
    cpu = orc.CpuLayer(256, 2, 4, orc.shuffled_table(5, 4, 4))
    cpu.stage[:] = stage.view(np.uint16)
    lib = orc.lib()
    if not hasattr(lib, "kvo_seal_tile"):
        pytest.skip("the oracle library has no stand-alone seal entry point")
    lib.kvo_seal_tile(cpu.k_code.ctypes.data_as(C.c_void_p), cpu.k_scale.ctypes.data_as(C.c_void_p),
                      cpu.v_code.ctypes.data_as(C.c_void_p), cpu.v_scale.ctypes.data_as(C.c_void_p),
                      cpu.stage.ctypes.data_as(C.c_void_p), cpu.table.ctypes.data_as(C.c_void_p), 256, 2, 0, 0)
    entries = []
    for h in range(2):
        for r in dump.tile_records(cpu.k_code, cpu.k_scale, cpu.v_code, cpu.v_scale, cpu.table, 0, h,
                                   stage_k=cpu.stage[0, 0, h], stage_v=cpu.stage[1, 0, h]):
            entries.append(dump.gvk2_entry(r, iters=0))
    path = str(tmp_path / "records.gvk2")
    dump.write_gvk2(path, entries)
    back = dump.read_gvk2(path)
    assert len(back) == 8
    order = [kn[0], kn[1], vn[0], vn[1], kn[2], kn[3], vn[2], vn[3]]  # per head: K slices, then V slices
    for e, name in zip(back, order):
        assert e.bits == 4 and e.iters == 0 and e.tile.shape == (128, 128)
        assert np.array_equal(e.tile, tiles[name].astype(np.float32)), name
        assert np.array_equal(e.record, recs[name]), name
        assert np.all(e.s_col == 1.0) and np.all(e.s_row == 1.0)


@pytest.mark.skipif(not os.path.exists(REF_GVK2), reason="reference sources absent (set KVB_REFERENCE_ROOT)")
def test_gvk2_reader_and_writer_reproduce_the_reference_file(tmp_path):
    dump = pkg().dump
    entries = dump.read_gvk2(REF_GVK2)
    assert len(entries) == 32
    out = str(tmp_path / "copy.bin")
    dump.write_gvk2(out, entries)
    assert open(out, "rb").read() == open(REF_GVK2, "rb").read()


@pytest.mark.gpu
def test_gvk2_records_written_from_gpu_planes_equal_the_oracle_quantiser(tmp_path):
    """The golden slices with one zero row appended through kvb_append (the rotation of zeros is exact) so that the GPU
    seals the tile; records cut from the GPU's planes and written as GVK2 equal, byte for byte, what the oracle's
    quantiser (pinned to the reference's golden records in the CPU tests) makes of the same tiles."""
    import torch

    from helpers import Twin

    dump = pkg().dump
    stage, _, _, _, _ = _stage_from_golden()
    stage[:, 0, :, 127] = 0
    tw = Twin(D=256, H=2, QH=4, capacity_tokens=128, seed=8)
    tw.cpu.stage[:] = stage.view(np.uint16)
    tw.gpu.stage.copy_(torch.from_numpy(stage.reshape(-1)).to(tw.dev))
    tw.len = 127
    zero = np.zeros((1, 2, 256), np.float16)
    tw.append(zero, zero)
    torch.cuda.synchronize()
    g = tw.gpu
    k_code, v_code = g.k_code.cpu().numpy(), g.v_code.cpu().numpy()
    k_scale, v_scale = g.k_scale.cpu().numpy().view(np.uint16), g.v_scale.cpu().numpy().view(np.uint16)
    entries = []
    for h in range(2):
        for r in dump.tile_records(k_code, k_scale, v_code, v_scale, g.table.cpu().numpy(), 0, h, stage_k=stage[0, 0, h], stage_v=stage[1, 0, h]):
            entries.append(dump.gvk2_entry(r, iters=0))
    path = str(tmp_path / "gpu.gvk2")
    dump.write_gvk2(path, entries)
    for e in dump.read_gvk2(path):
        want, _, _, _ = orc.quantize_tile(e.tile, 4, 0)
        assert np.array_equal(e.record, want), e.name
    assert g.errors() == 0
