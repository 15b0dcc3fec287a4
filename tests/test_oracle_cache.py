"""CPU tests of the oracle's cache state machine (append / seal / page decode) and attention."""
import numpy as np
import pytest


def _layer(oracle, D, H, tokens, seed=0, iters=0):
    lp = (tokens + 63) // 64 + 2
    lp += lp & 1
    table = oracle.shuffled_table(seed, lp, lp + 3)
    return oracle.CpuLayer(D, H, lp + 3, table, iters)


def _rot_stage(oracle, x):
    return oracle.hadamard(x.astype(np.float32)).astype(np.float16)


@pytest.mark.parametrize("D", [128, 256])
def test_append_seals_into_p1_planes(oracle, D):
    H, T = 2, 300
    k, v = oracle.synth_kv(0, T, H, D, 1), oracle.synth_kv(0, T, H, D, 2)
    L = _layer(oracle, D, H, T)
    L.append(k, v, 0)
    kr, vr = _rot_stage(oracle, k), _rot_stage(oracle, v)
    S = D // 128
    for tile in range(2):
        for h in range(H):
            dk, dv = L.decode_tile(tile, h)
            for s in range(S):
                sl = slice(s * 128, s * 128 + 128)
                tk = kr[tile * 128:(tile + 1) * 128, h, sl].astype(np.float32).T  # row = dim, col = token
                tv = vr[tile * 128:(tile + 1) * 128, h, sl].astype(np.float32)    # row = token, col = dim
                rk, qk, _, _ = oracle.quantize_tile(tk, 4, 0)
                rv, qv, _, _ = oracle.quantize_tile(tv, 4, 0)
                assert np.array_equal(dk[:, sl].astype(np.float32), oracle.dequant_tile(rk, 128, 128).T.astype(np.float16).astype(np.float32))
                assert np.array_equal(dv[:, sl].astype(np.float32), oracle.dequant_tile(rv, 128, 128).astype(np.float16).astype(np.float32))
                # code plane: byte b of a token row = dims 2b | 2b+1 << 4
                for half in range(2):
                    pg = L.table[2 * tile + half]
                    rows = L.k_code[pg, h][:, s * 64:(s + 1) * 64]
                    want = qk[0::2, half * 64:(half + 1) * 64] | (qk[1::2, half * 64:(half + 1) * 64] << 4)
                    assert np.array_equal(rows, want.T)
    # open tile (tokens 256..299) lives un-quantised in stage slot 0
    assert np.array_equal(L.stage[0, 0, :, :44].view(np.float16), kr[256:300].transpose(1, 0, 2))
    assert np.array_equal(L.stage[1, 0, :, :44].view(np.float16), vr[256:300].transpose(1, 0, 2))


def test_chunked_append_equals_one_shot(oracle):
    D, H, T = 128, 4, 517
    k, v = oracle.synth_kv(1, T, H, D, 1), oracle.synth_kv(1, T, H, D, 2)
    A, B = _layer(oracle, D, H, T), _layer(oracle, D, H, T)
    A.append(k, v, 0)
    pos = 0
    for n in (100, 28, 1, 1, 126, 130, 7, 124):
        B.append(k[pos:pos + n], v[pos:pos + n], pos)
        pos += n
    assert pos == T
    for name in ("k_code", "k_scale", "v_code", "v_scale"):
        assert np.array_equal(getattr(A, name), getattr(B, name)), name
    live = T - 512
    assert np.array_equal(A.stage[:, 0, :, :live], B.stage[:, 0, :, :live])


def test_rollback_and_reappend(oracle):
    """A verify step may seal a tile with draft tokens that are rejected afterwards; re-appending from
    the roll-back point must re-seal the tile from the stage (two stage slots keep the rows)."""
    D, H = 128, 2
    k, v = oracle.synth_kv(2, 140, H, D, 1), oracle.synth_kv(2, 140, H, D, 2)
    k2, v2 = oracle.synth_kv(3, 140, H, D, 1), oracle.synth_kv(3, 140, H, D, 2)
    A, B = _layer(oracle, D, H, 140), _layer(oracle, D, H, 140)
    A.append(k[:124], v[:124], 0)
    A.append(k[124:131], v[124:131], 124)          # seals tile 0 with drafts 124..130
    kk, vv = k.copy(), v.copy()
    kk[126:140], vv[126:140] = k2[126:140], v2[126:140]
    A.append(kk[126:140], vv[126:140], 126)         # drafts 126.. rejected, new tokens take their place
    B.append(kk, vv, 0)
    for name in ("k_code", "k_scale", "v_code", "v_scale"):
        assert np.array_equal(getattr(A, name), getattr(B, name)), name
    assert np.array_equal(A.stage[:, 1, :, :12], B.stage[:, 1, :, :12])


@pytest.mark.parametrize("D,T", [(128, 333), (256, 200)])
def test_attention_matches_dense_numpy(oracle, D, T):
    H, QH = 2, 6
    k, v = oracle.synth_kv(4, T, H, D, 1), oracle.synth_kv(4, T, H, D, 2)
    L = _layer(oracle, D, H, T)
    L.append(k, v, 0)
    # materialise what attention must see: sealed tiles de-quantised, open tile from the stage
    kr = np.zeros((T, H, D), np.float32)
    vr = np.zeros((T, H, D), np.float32)
    sealed = T // 128
    q = oracle.synth_q(4, 3, QH, D)
    q_pos = np.array([T - 3, T - 2, T - 1], np.int32)
    scale = 1.0 / np.sqrt(D)
    out1 = L.attention(q, q_pos, scale, QH, threads=1)
    out4, pm, pl, po = L.attention(q, q_pos, scale, QH, threads=4, want_partials=True)
    assert np.allclose(out1, out4, atol=1e-6)
    # split the key range in two, merge the partials: same answer (the multi-GPU combine)
    cut = 128
    _, m0, l0, o0 = L.attention(q, q_pos, scale, QH, key_begin=0, key_end=cut, want_partials=True)
    _, m1, l1, o1 = L.attention(q, q_pos, scale, QH, key_begin=cut, key_end=T, want_partials=True)
    merged = oracle.merge_partials(np.stack([m0, m1]).reshape(2, -1), np.stack([l0, l1]).reshape(2, -1),
                                   np.stack([o0, o1]).reshape(2, -1, D)).reshape(out1.shape)
    assert np.allclose(merged, out1, atol=2e-6)
    # dense check through fp16 page decode (fp16 rounding of K/V: loose tolerance)
    for t in range(sealed):
        for h in range(H):
            dk, dv = L.decode_tile(t, h)
            kr[t * 128:(t + 1) * 128, h], vr[t * 128:(t + 1) * 128, h] = dk, dv
    live = T - sealed * 128
    kr[sealed * 128:] = L.stage[0, sealed & 1, :, :live].view(np.float16).transpose(1, 0, 2)
    vr[sealed * 128:] = L.stage[1, sealed & 1, :, :live].view(np.float16).transpose(1, 0, 2)
    dense = oracle.attention_fp32_dense(kr, vr, q, q_pos, scale)
    assert np.abs(dense - out1).max() <= 4e-3 * np.abs(dense).max()
