"""kvb_attn_decode_static: decode attention for hosts that cannot hand the library a workspace (their device
memory was all given to their own pool at start-up, or their serving thread may not call the allocator).  The
split-K partials then live in a fixed array inside the library.  The entry point must give exactly what
kvb_attn_decode gives with a caller-owned workspace, on repeated calls that reuse the array, and must refuse
shapes whose partials do not fit.  Collected last on purpose (file name)."""
import ctypes as C

import numpy as np
import pytest

from helpers import Twin, attn_close, orc, pkg

pytestmark = pytest.mark.gpu


def _static_decode(tw, q_dev, pos_dev, kv_len_max):
    import torch

    lib = pkg().capi.load()
    out = torch.empty_like(q_dev)
    st = lib.kvb_attn_decode_static(C.byref(tw.gpu.c), C.c_void_p(q_dev.data_ptr()), C.c_void_p(pos_dev.data_ptr()),
                                    1.0 / np.sqrt(tw.D), kv_len_max, C.c_void_p(out.data_ptr()),
                                    C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return st, out


def test_static_scratch_matches_workspace_path_twice():
    import torch

    capi = pkg().capi
    T = 1500
    tw = Twin(D=128, H=4, QH=24, capacity_tokens=T + 8, seed=71)
    k, v = orc.synth_kv(72, T + 1, 4, 128, 1), orc.synth_kv(72, T + 1, 4, 128, 2)
    tw.append(k[:T], v[:T])
    assert capi.load().kvb_static_scratch_bytes() == 2 << 20
    for call in range(2):  # the second call finds the first call's partials in the array
        if call == 1:
            tw.append(k[T:], v[T:])  # one more token: a different position and open-tile length
        n = tw.len
        q = orc.synth_q(73 + call, 1, 24, 128)
        q_dev = torch.from_numpy(q[0]).to(tw.dev)
        pos = torch.tensor([n - 1], dtype=torch.int32, device=tw.dev)
        ref = tw.gpu.attn_decode(q_dev, pos, 1.0 / np.sqrt(128), n)
        st, got = _static_decode(tw, q_dev, pos, n)
        torch.cuda.synchronize()
        assert st == capi.KVB_OK, capi.load().kvb_last_error_string()
        # same kernels, same split: the two paths agree to the last bit; the oracle bounds both
        assert torch.equal(got, ref)
        want = tw.cpu.attention(q, [n - 1], 1.0 / np.sqrt(128), 24, threads=4)
        ok, msg = attn_close(got.float().cpu().numpy(), want[0])
        assert ok, msg
    assert tw.gpu.errors() == 0


def test_every_decode_shape_of_this_gpu_fits_the_array():
    """The refusal (KVB_ERANGE) guards GPUs with more SMs than a B200: with 148 SMs the split count is capped so
    that kv_heads x splits <= 148 partial sets of 8,320 bytes, which is below the 2 MiB the array holds."""
    lib = pkg().capi.load()
    worst = max(lib.kvb_workspace_bytes(400000, h, h * g, 128, 1, 1) for h in range(1, 9) for g in (1, 6, 8))
    assert 0 < worst <= lib.kvb_static_scratch_bytes()
