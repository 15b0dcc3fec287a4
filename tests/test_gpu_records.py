"""The compact tile record at every code width, written and read on the GPU (kvb_records_encode / _decode), against
the CPU oracle's record codec (bit string of any width, kvarn-evidence/oracle/bee_oracle.cpp:152-172, 309-374): the
bytes of the records are equal, and so are the tiles read back from them.  Inputs: seeded tiles with outlier
columns, a constant row (scale clamps to 1e-10), a row of two values, a tile of zeros."""
import numpy as np
import pytest

from helpers import orc, pkg

pytestmark = pytest.mark.gpu


def _tiles(seed, n):
    rng = np.random.default_rng(seed)
    t = rng.standard_normal((n, 128, 128)).astype(np.float32)
    t[:, :, [3, 17, 64, 101]] *= 20.0
    t[0, 5, :] = 0.75                      # a constant row
    t[0, 6, :] = np.where(np.arange(128) % 2 == 0, -1.0, 3.0)
    if n > 1:
        t[1] = 0.0
    return t


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_records_equal_the_oracle_at_every_width(bits):
    import torch

    rec_mod = pkg().records
    tiles = _tiles(100 + bits, 5)
    got = rec_mod.encode(torch.from_numpy(tiles).cuda(), bits)
    back = rec_mod.decode(got, bits)
    torch.cuda.synchronize()
    got, back = got.cpu().numpy(), back.cpu().numpy()
    assert got.shape == (5, 2048 * bits + 768) == (5, rec_mod.record_bytes(bits))
    for i in range(5):
        want, codes, bc, br = orc.quantize_tile(tiles[i], bits, 0)
        assert np.all(bc == 1.0) and np.all(br == 1.0)
        assert np.array_equal(got[i], want), f"tile {i}: {int((got[i] != want).sum())} record bytes differ"
        assert np.array_equal(back[i], orc.dequant_tile(want, 128, 128, bits)), f"tile {i}: decoded values differ"
    # the decoded tile is within half a step of the input (the quantiser's own bound), widths ordered as expected
    err = np.abs(back - tiles).max()
    span = (tiles.max(axis=2) - tiles.min(axis=2)).max()
    assert err <= 0.5 * span / (2 ** bits - 1) * 1.01 + 1e-3 * span  # + the fp16 rounding of scale and zero point


def test_k4v4_record_is_140_bytes_per_token_and_head():
    rec_mod = pkg().records
    assert 2 * rec_mod.record_bytes(4) == 128 * 140        # a K and a V record per 128 tokens of a head, head_dim 128
    assert rec_mod.record_bytes(4) + rec_mod.record_bytes(2) == 128 * 108   # K4V2
    with pytest.raises(ValueError):
        rec_mod.record_bytes(7)
