"""GPU parity of the quantise-append path and the tile decode, through the C ABI, against the CPU oracle:
codes, fp16 scales and page placement bit-exact (Sinkhorn iterations = 0)."""
import os

import numpy as np
import pytest

from conftest import GOLDEN
from helpers import Twin, orc

pytestmark = pytest.mark.gpu


def _check_planes(tw):
    eq = tw.planes_equal()
    assert all(eq.values()), eq
    assert tw.live_stage_equal()
    assert tw.gpu.errors() == 0


def test_config0_round_trip_4096_tokens():
    """4 KV heads x 128, 4096 tokens, outlier channels, seed 0, shuffled 64-token pages."""
    tw = Twin(D=128, H=4, capacity_tokens=4096, seed=0)
    k, v = orc.synth_kv(0, 4096, 4, 128, 1), orc.synth_kv(0, 4096, 4, 128, 2)
    tw.append(k, v)
    _check_planes(tw)


@pytest.mark.parametrize("D,dtype", [(128, 0), (256, 0), (128, 1), (256, 1)])
def test_ragged_chunks(D, dtype):
    H, T = 2, 777
    tw = Twin(D=D, H=H, QH=2 * H, capacity_tokens=T, seed=3, dtype=dtype)
    k, v = orc.synth_kv(5, T, H, D, 1), orc.synth_kv(5, T, H, D, 2)
    pos = 0
    for n in (1, 50, 13, 64, 1, 127, 128, 129, 257, 7):
        tw.append(k[pos:pos + n], v[pos:pos + n])
        pos += n
        assert tw.live_stage_equal(), (pos, n)
    assert pos == T
    _check_planes(tw)


def test_single_token_steps_across_a_seal():
    tw = Twin(D=128, H=4, capacity_tokens=260, seed=4)
    k, v = orc.synth_kv(6, 260, 4, 128, 1), orc.synth_kv(6, 260, 4, 128, 2)
    tw.append(k[:120], v[:120])
    for p in range(120, 260):
        tw.append(k[p:p + 1], v[p:p + 1])
    _check_planes(tw)


def test_rollback_reseals_from_the_stage():
    tw = Twin(D=128, H=2, QH=4, capacity_tokens=140, seed=5)
    k, v = orc.synth_kv(2, 140, 2, 128, 1), orc.synth_kv(2, 140, 2, 128, 2)
    k2, v2 = orc.synth_kv(3, 140, 2, 128, 1), orc.synth_kv(3, 140, 2, 128, 2)
    tw.append(k[:124], v[:124])
    tw.append(k[124:131], v[124:131])            # drafts seal tile 0
    tw.append(k2[126:140], v2[126:140], pos0=126)  # roll back to 126, re-append
    _check_planes(tw)


def test_decode_tile_matches_oracle():
    tw = Twin(D=256, H=2, QH=4, capacity_tokens=256, seed=6)
    k, v = orc.synth_kv(7, 256, 2, 256, 1), orc.synth_kv(7, 256, 2, 256, 2)
    tw.append(k, v)
    for tile in range(2):
        for h in range(2):
            gk, gv = tw.gpu.decode_tile(tile, h)
            ck, cv = tw.cpu.decode_tile(tile, h)
            assert np.array_equal(gk.cpu().numpy().view(np.uint16), ck.view(np.uint16))
            assert np.array_equal(gv.cpu().numpy().view(np.uint16), cv.view(np.uint16))


def test_real_tiles_from_the_golden_records():
    """Real (already rotated) K/V slices of the reference's golden records, placed in the stage; one zero row is
    appended to complete the tile (the rotation of zeros is exact), then planes are compared byte for byte."""
    import torch

    g = np.load(os.path.join(GOLDEN, "gvk2_it0.npz"))
    tiles = {n: t for n, t in zip(g["names"], g["tiles"])}
    tw = Twin(D=256, H=2, QH=4, capacity_tokens=128, seed=8)
    ks = [tiles["L35_k_h0_s0_g0"], tiles["L35_k_h1_s1_g0"], tiles["L63_k_h2_s0_g0"], tiles["L63_k_h3_s1_g0"]]  # [dim][tok]
    vs = [tiles["L35_v_h0_s0_g0"], tiles["L35_v_h1_s1_g0"], tiles["L63_v_h2_s0_g0"], tiles["L63_v_h3_s1_g0"]]  # [tok][dim]
    stage = np.zeros((2, 2, 2, 128, 256), np.float16)
    for h in range(2):
        for s in range(2):
            stage[0, 0, h, :, s * 128:(s + 1) * 128] = ks[2 * h + s].T
            stage[1, 0, h, :, s * 128:(s + 1) * 128] = vs[2 * h + s]
    stage[:, 0, :, 127] = 0
    tw.cpu.stage[:] = stage.view(np.uint16)
    tw.gpu.stage.copy_(torch.from_numpy(stage.reshape(-1)).to(tw.dev))
    tw.len = 127
    zero = np.zeros((1, 2, 256), np.float16)
    tw.append(zero, zero)
    _check_planes(tw)
    # and the oracle on the untouched golden tile is the reference's own record (pinned in the CPU tests)


def test_sinkhorn_16_iterations_within_tolerance():
    """iters = 16 is not a byte-exact regime even for the reference's own CUDA kernel (device logf/expf differ
    from the host's); it is judged like the reference does: cosine of the de-quantised tile >= 0.999 against the
    oracle's, and factors close."""
    tw = Twin(D=128, H=2, QH=4, capacity_tokens=128, seed=9, iters=16)
    k, v = orc.synth_kv(10, 128, 2, 128, 1), orc.synth_kv(10, 128, 2, 128, 2)
    tw.append(k, v)
    for h in range(2):
        gk, gv = tw.gpu.decode_tile(0, h)
        ck, cv = tw.cpu.decode_tile(0, h)
        for a, b in ((gk, ck), (gv, cv)):
            a = a.float().cpu().numpy().astype(np.float64)
            b = b.astype(np.float64)
            assert np.isfinite(a).all()
            cos = (a * b).sum() / np.sqrt((a * a).sum() * (b * b).sum())
            assert cos >= 0.999, cos
    frac = (tw.gpu.k_code.cpu().numpy() != tw.cpu.k_code).mean()
    assert frac < 0.05, frac


def test_bad_inputs_set_the_error_word_and_do_not_fault():
    import torch

    tw = Twin(D=128, H=2, QH=4, capacity_tokens=256, seed=11)
    k, v = orc.synth_kv(12, 128, 2, 128, 1), orc.synth_kv(12, 128, 2, 128, 2)
    kb, vb = torch.from_numpy(k).to(tw.dev), torch.from_numpy(v).to(tw.dev)
    capi = __import__("helpers").pkg().capi
    # non-contiguous positions
    pos = torch.arange(0, 256, 2, dtype=torch.int32, device=tw.dev)
    tw.gpu.append(kb, vb, pos)
    torch.cuda.synchronize()
    assert tw.gpu.errors() & capi.ERR_POSITIONS
    tw.gpu.error_word.zero_()
    # a page id outside the pool
    tw.gpu.table[0] = 10_000
    tw.gpu.append(kb, vb, torch.arange(128, dtype=torch.int32, device=tw.dev))
    torch.cuda.synchronize()
    assert tw.gpu.errors() & capi.ERR_PAGE_RANGE
    assert not tw.gpu.k_code.any()
