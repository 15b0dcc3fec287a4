"""KV dump files (KVD1 records from the planes, KVO1 de-quantised tiles): round trip through the reader, equality
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
