"""GPU parity of the fused attention kernels (decode, MTP verify, partial + merge, prefill chunk) against the
CPU oracle: softmax attention in double precision over the de-quantised cache.  Tolerance: see helpers."""
import numpy as np
import pytest

from helpers import Twin, attn_close, cpu_twin_of, orc, pkg

pytestmark = pytest.mark.gpu


def _decode(tw, q16, pos):
    import torch

    qd = torch.from_numpy(q16).to(tw.dev)
    p = torch.tensor([pos], dtype=torch.int32, device=tw.dev)
    out = tw.gpu.attn_decode(qd, p, 1.0 / np.sqrt(tw.D), pos + 1)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


def test_config0_decode_at_4096():
    tw = Twin(D=128, H=4, QH=24, capacity_tokens=4096, seed=0)
    k, v = orc.synth_kv(0, 4096, 4, 128, 1), orc.synth_kv(0, 4096, 4, 128, 2)
    tw.append(k, v)
    q = orc.synth_q(0, 1, 24, 128)
    want = tw.cpu.attention(q, [4095], 1.0 / np.sqrt(128), 24, threads=8)
    got = _decode(tw, q[0], 4095)
    ok, msg = attn_close(got, want[0])
    assert ok, msg
    assert tw.gpu.errors() == 0


@pytest.mark.parametrize("T", [1, 15, 16, 51, 64, 127, 128, 129, 191, 192, 300, 1000, 2049])
def test_decode_ragged_lengths(T):
    tw = Twin(D=128, H=4, QH=24, capacity_tokens=T, seed=T)
    k, v = orc.synth_kv(T, T, 4, 128, 1), orc.synth_kv(T, T, 4, 128, 2)
    tw.append(k, v)
    q = orc.synth_q(T, 1, 24, 128)
    want = tw.cpu.attention(q, [T - 1], 1.0 / np.sqrt(128), 24, threads=4)
    got = _decode(tw, q[0], T - 1)
    ok, msg = attn_close(got, want[0])
    assert ok, msg


@pytest.mark.parametrize("H,QH", [(4, 4), (2, 16), (1, 7), (8, 8)])
def test_decode_other_head_shapes(H, QH):
    T = 700
    tw = Twin(D=128, H=H, QH=QH, capacity_tokens=T, seed=21)
    k, v = orc.synth_kv(22, T, H, 128, 1), orc.synth_kv(22, T, H, 128, 2)
    tw.append(k, v)
    q = orc.synth_q(22, 1, QH, 128)
    want = tw.cpu.attention(q, [T - 1], 1.0 / np.sqrt(128), QH, threads=4)
    ok, msg = attn_close(_decode(tw, q[0], T - 1), want[0])
    assert ok, msg


def test_decode_bf16_io():
    import torch

    T = 900
    tw = Twin(D=128, H=4, QH=24, capacity_tokens=T, seed=23, dtype=1)
    k, v = orc.synth_kv(24, T, 4, 128, 1), orc.synth_kv(24, T, 4, 128, 2)
    tw.append(k, v)
    from helpers import from_bits, to_bits
    qb = to_bits(orc.synth_q(24, 1, 24, 128), 1)
    want = tw.cpu.attention(qb, [T - 1], 1.0 / np.sqrt(128), 24, dtype=1, threads=4)
    out = tw.gpu.attn_decode(from_bits(qb[0], 1).to(tw.dev), torch.tensor([T - 1], dtype=torch.int32, device=tw.dev),
                             1.0 / np.sqrt(128), T)
    got = out.float().cpu().numpy()
    err = np.abs(got - want[0]).max()
    assert err <= 2.0 ** -8 * np.abs(want).max(), err  # bf16 output rounding dominates


@pytest.mark.parametrize("prefix,width", [(300, 1), (300, 4), (1000, 8), (125, 6), (120, 8), (127, 2), (0, 5)])
def test_verify_rows_are_causal(prefix, width):
    """Append width new rows then attend; covers verify steps that complete a tile (prefix 125 + 6, 120 + 8)."""
    import torch

    H, QH, D = 4, 24, 128
    T = prefix + width
    tw = Twin(D=D, H=H, QH=QH, capacity_tokens=T, seed=31)
    k, v = orc.synth_kv(32, T, H, D, 1), orc.synth_kv(32, T, H, D, 2)
    if prefix:
        tw.append(k[:prefix], v[:prefix])
    q = orc.synth_q(32, width, QH, D)
    pos = np.arange(prefix, T, dtype=np.int32)
    tw.cpu.append(k[prefix:], v[prefix:], prefix)
    want = tw.cpu.attention(q, pos, 1.0 / np.sqrt(D), QH, threads=4)
    out = tw.gpu.attn_verify(torch.from_numpy(q).to(tw.dev), torch.from_numpy(k[prefix:]).to(tw.dev),
                             torch.from_numpy(v[prefix:]).to(tw.dev), torch.from_numpy(pos).to(tw.dev), 1.0 / np.sqrt(D), T)
    torch.cuda.synchronize()
    tw.len = T
    eq = tw.planes_equal()
    assert all(eq.values()), eq
    # from 32 GQA-merged rows per KV head on (width >= 6 here) the step runs on the tcgen05 chunk kernel, which rounds
    # the de-quantised tiles to fp16; narrower steps run on the warp-level kernel and are held to its tolerance
    from helpers import PREFILL_MAX_ABS, PREFILL_REL_L2
    dense = width * (QH // H) >= 32
    ok, msg = attn_close(out.float().cpu().numpy(), want, PREFILL_MAX_ABS if dense else 2.0 ** -10, PREFILL_REL_L2 if dense else 1e-3)
    assert ok, msg


@pytest.mark.parametrize("H,QH,T", [(4, 12, 4600), (3, 9, 6100), (7, 21, 2550)])
def test_verify_widths_share_one_workspace(H, QH, T):
    """Three query heads per KV head at 2.5K-6K tokens: a narrow verify step is cut into more splits than a wide one.
    One workspace sized for width 8 serves every width, canary words behind it stay intact."""
    import torch

    D = 128
    tw = Twin(D=D, H=H, QH=QH, capacity_tokens=T + 8, seed=57)
    k, v = orc.synth_kv(58, T + 8, H, D, 1), orc.synth_kv(58, T + 8, H, D, 2)
    tw.append(k[:T], v[:T])
    lib = pkg().capi.load()
    nbytes = lib.kvb_workspace_bytes(T + 8, H, QH, D, 8, 1)
    guard = 4096
    buf = torch.full((nbytes // 4 + guard,), float("nan"), dtype=torch.float32, device=tw.dev)
    buf[nbytes // 4:] = 12345.0
    tw.gpu._ws = buf[:nbytes // 4]  # the layer's grow-only workspace: large enough, so it is kept
    scale = 1.0 / np.sqrt(D)
    for width in (1, 2, 5, 8, 3):
        q = orc.synth_q(59 + width, width, QH, D)
        pos = np.arange(T, T + width, dtype=np.int32)
        tw.cpu.append(k[T:T + width], v[T:T + width], T)
        want = tw.cpu.attention(q, pos, scale, QH, threads=4)
        out = tw.gpu.attn_verify(torch.from_numpy(q).to(tw.dev), torch.from_numpy(k[T:T + width]).to(tw.dev),
                                 torch.from_numpy(v[T:T + width]).to(tw.dev), torch.from_numpy(pos).to(tw.dev), scale, T + 8)
        torch.cuda.synchronize()
        assert tw.gpu._ws.data_ptr() == buf.data_ptr()
        assert bool((buf[nbytes // 4:] == 12345.0).all()), f"width {width} wrote past its workspace"
        from helpers import PREFILL_MAX_ABS, PREFILL_REL_L2
        ok, msg = attn_close(out.float().cpu().numpy(), want, PREFILL_MAX_ABS, PREFILL_REL_L2)
        assert ok, (width, msg)
    assert tw.gpu.errors() == 0


@pytest.mark.parametrize("T0", [300, 127, 255, 1000])
def test_append_decode_equals_append_then_decode(T0):
    """kvb_append_decode (the attention chained to the append, only the CTAs that read the stage or a freshly sealed tile
    waiting for it) against kvb_append followed by kvb_attn_decode on a twin cache: same bits, over steps that cross a
    tile boundary (the append seals a tile in the middle of the run)."""
    import torch

    H, QH, D, steps = 4, 24, 128, 6
    k, v = orc.synth_kv(91, T0 + steps, H, D, 1), orc.synth_kv(91, T0 + steps, H, D, 2)
    q = orc.synth_q(91, steps, QH, D)
    a = Twin(D=D, H=H, QH=QH, capacity_tokens=T0 + steps, seed=92)
    b = Twin(D=D, H=H, QH=QH, capacity_tokens=T0 + steps, seed=92)
    a.append(k[:T0], v[:T0])
    b.append(k[:T0], v[:T0])
    scale = 1.0 / np.sqrt(D)
    for s in range(steps):
        p = T0 + s
        pos = torch.tensor([p], dtype=torch.int32, device=a.dev)
        kd, vd, qd = (torch.from_numpy(x).to(a.dev) for x in (k[p:p + 1], v[p:p + 1], q[s]))
        got = a.gpu.append_decode(qd, kd, vd, pos, scale, T0 + steps)
        b.gpu.append(kd, vd, pos)
        want = b.gpu.attn_decode(qd, pos, scale, T0 + steps)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (T0, s)
        a.cpu.append(k[p:p + 1], v[p:p + 1], p)
        ref = a.cpu.attention(q[s:s + 1], [p], scale, QH, threads=4)[0]
        ok, msg = attn_close(got.float().cpu().numpy(), ref)
        assert ok, msg
    a.len = T0 + steps
    assert all(a.planes_equal().values()) and a.gpu.errors() == 0


def test_partials_merge_to_the_full_answer():
    """Key ranges attended separately and merged by log-sum-exp (what the multi-GPU combine does)."""
    import torch

    T = 1500
    tw = Twin(D=128, H=4, QH=24, capacity_tokens=T, seed=41)
    k, v = orc.synth_kv(42, T, 4, 128, 1), orc.synth_kv(42, T, 4, 128, 2)
    tw.append(k, v)
    q = orc.synth_q(42, 1, 24, 128)
    scale = 1.0 / np.sqrt(128)
    want, wm, wl, wo = tw.cpu.attention(q, [T - 1], scale, 24, threads=4, want_partials=True)
    qd = torch.from_numpy(q[0]).to(tw.dev)
    pos = torch.tensor([T - 1], dtype=torch.int32, device=tw.dev)
    cuts = [0, 200, 640, 1283, T]
    ms, ls, os_ = [], [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        m, l, o = tw.gpu.attn_decode_partial(qd, pos, scale, T, a, b)
        ms.append(m); ls.append(l); os_.append(o)
        cm, cl, co = tw.cpu.attention(q, [T - 1], scale, 24, key_begin=a, key_end=b, want_partials=True)[1:]
        # compare normalised partial outputs (m, l individually depend on the split, their combination does not)
        assert np.allclose(m.cpu().numpy() + np.log(l.cpu().numpy()), cm[0] + np.log(cl[0]), atol=2e-3)
    merged = pkg().merge_partials(torch.stack(ms), torch.stack(ls), torch.stack(os_))
    ok, msg = attn_close(merged.float().cpu().numpy(), want[0])
    assert ok, msg
    full = tw.gpu.attn_decode(qd, pos, scale, T)
    ok, msg = attn_close(full.float().cpu().numpy(), want[0])
    assert ok, msg


@pytest.mark.parametrize("prefix,chunk,cut", [(1000, 4, 512), (1000, 8, 640), (700, 300, 384), (2048, 64, 1024), (300, 3, 256)])
def test_chunk_partials_of_two_range_caches_merge_to_the_full_answer(prefix, chunk, cut):
    """A verify step / prefill chunk over a sequence held as two caches (tokens [0, cut) and [cut, ...), the layout of a
    range-sharded sequence on two GPUs, here side by side on one): the new rows are appended to the second cache, each
    cache exports its partials (kvb_attn_chunk_partial), the merge equals the oracle's attention over the whole sequence."""
    import torch

    H, QH, D = 4, 24, 128
    T = prefix + chunk
    k, v = orc.synth_kv(71, T, H, D, 1), orc.synth_kv(71, T, H, D, 2)
    q = orc.synth_q(71, chunk, QH, D)
    scale = 1.0 / np.sqrt(D)
    lp = T // 64 + 6
    cpu = orc.CpuLayer(D, H, lp, orc.shuffled_table(72, lp, lp))
    cpu.append(k, v, 0)
    want = cpu.attention(q, np.arange(prefix, T, dtype=np.int32), scale, QH, threads=4)
    dev = torch.device("cuda:0")

    def cache_of(rows_k, rows_v, seed, room):
        n = rows_k.shape[0]
        pages = (n + room + 63) // 64 + 2
        pages += pages & 1
        L = pkg().KvarnLayer(D, H, QH, pages, torch.from_numpy(orc.shuffled_table(seed, pages, pages)), device="cuda:0")
        L.append(torch.from_numpy(rows_k).to(dev), torch.from_numpy(rows_v).to(dev), torch.arange(n, dtype=torch.int32, device=dev))
        return L

    A = cache_of(k[:cut], v[:cut], 73, 0)
    B = cache_of(k[cut:prefix], v[cut:prefix], 74, chunk)
    qd = torch.from_numpy(q).to(dev)
    pos_b = torch.arange(prefix - cut, T - cut, dtype=torch.int32, device=dev)
    B.append(torch.from_numpy(k[prefix:]).to(dev), torch.from_numpy(v[prefix:]).to(dev), pos_b)  # the owner of the open tile
    pos_a = torch.full((chunk,), cut - 1, dtype=torch.int32, device=dev)
    rows = chunk * QH
    packed = torch.empty((2, rows * (D + 2)), dtype=torch.float32, device=dev)
    A.attn_chunk_partial_packed(qd, pos_a, scale, cut, packed[0])
    B.attn_chunk_partial_packed(qd, pos_b, scale, T - cut, packed[1])
    out = torch.empty((chunk, QH, D), dtype=torch.float16, device=dev)
    pkg().cache.merge_partials_packed(packed.view(-1), 2, rows, D, out.view(rows, D))
    torch.cuda.synchronize()
    assert A.errors() == 0 and B.errors() == 0
    from helpers import PREFILL_MAX_ABS, PREFILL_REL_L2
    dense = chunk > 8 or chunk * (QH // H) >= 32
    ok, msg = attn_close(out.float().cpu().numpy(), want, PREFILL_MAX_ABS if dense else 2.0 ** -10, PREFILL_REL_L2 if dense else 1e-3)
    assert ok, msg


@pytest.mark.parametrize("prefix,chunk", [(333, 100), (0, 128), (1000, 300), (120, 8), (3000, 20), (256, 1024), (77, 1)])
def test_prefill_chunk(prefix, chunk):
    """Quantise-append a chunk, then causal chunk attention over prefix + chunk on the tcgen05 kernel.  Covers a
    chunk that starts the cache, chunks that complete tiles, an open tile left in the stage, a 1,024-token chunk."""
    import torch

    from helpers import PREFILL_MAX_ABS, PREFILL_REL_L2

    H, QH, D = 4, 24, 128
    T = prefix + chunk
    tw = Twin(D=D, H=H, QH=QH, capacity_tokens=T, seed=51)
    k, v = orc.synth_kv(52, T, H, D, 1), orc.synth_kv(52, T, H, D, 2)
    if prefix:
        tw.append(k[:prefix], v[:prefix])
    q = orc.synth_q(52, chunk, QH, D)
    pos = np.arange(prefix, T, dtype=np.int32)
    tw.cpu.append(k[prefix:], v[prefix:], prefix)
    want = tw.cpu.attention(q, pos, 1.0 / np.sqrt(D), QH, threads=8)
    out = tw.gpu.attn_prefill(torch.from_numpy(q).to(tw.dev), torch.from_numpy(k[prefix:]).to(tw.dev),
                              torch.from_numpy(v[prefix:]).to(tw.dev), torch.from_numpy(pos).to(tw.dev), 1.0 / np.sqrt(D), T)
    torch.cuda.synchronize()
    assert tw.gpu.errors() == 0
    tw.len = T
    eq = tw.planes_equal()
    assert all(eq.values()), eq
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    ok, msg = attn_close(got, want, PREFILL_MAX_ABS, PREFILL_REL_L2)
    assert ok, msg


def test_bad_page_id_is_reported_not_faulted():
    import torch

    T = 600
    tw = Twin(D=128, H=4, QH=24, capacity_tokens=T, seed=61)
    k, v = orc.synth_kv(62, T, 4, 128, 1), orc.synth_kv(62, T, 4, 128, 2)
    tw.append(k, v)
    tw.gpu.table[3] = -7
    q = orc.synth_q(62, 1, 24, 128)
    out = _decode(tw, q[0], T - 1)
    assert np.isfinite(out).all()
    assert tw.gpu.errors() & pkg().capi.ERR_PAGE_RANGE


def test_packed_partial_and_merge():
    """The send-buffer layout of the sharded decode: m | l | o in one block per part."""
    import torch

    T = 900
    tw = Twin(D=128, H=4, QH=24, capacity_tokens=T, seed=91)
    k, v = orc.synth_kv(92, T, 4, 128, 1), orc.synth_kv(92, T, 4, 128, 2)
    tw.append(k, v)
    q = orc.synth_q(92, 1, 24, 128)
    qd = torch.from_numpy(q[0]).to(tw.dev)
    pos = torch.tensor([T - 1], dtype=torch.int32, device=tw.dev)
    scale = 1.0 / np.sqrt(128)
    n = 24 * 130
    buf = torch.zeros(2 * n, dtype=torch.float32, device=tw.dev)
    tw.gpu.attn_decode_partial_packed(qd, pos, scale, T, buf[:n])
    buf[n:n + 24] = float("-inf")  # second part: a rank without keys (neutral partial)
    out = torch.empty((24, 128), dtype=torch.float16, device=tw.dev)
    pkg().cache.merge_partials_packed(buf, 2, 24, 128, out)
    full = tw.gpu.attn_decode(qd, pos, scale, T)
    torch.cuda.synchronize()
    assert torch.equal(out, full)


def _sync_cpu_from_gpu(tw):
    """Make the oracle layer hold exactly the bytes the GPU layer holds (needed when the two quantisers may
    differ in a few codes, i.e. with Sinkhorn iterations > 0)."""
    g, c = tw.gpu, tw.cpu
    c.k_code[:] = g.k_code.cpu().numpy(); c.v_code[:] = g.v_code.cpu().numpy()
    c.k_scale[:] = g.k_scale.cpu().numpy().view(np.uint16); c.v_scale[:] = g.v_scale.cpu().numpy().view(np.uint16)
    c.stage[:] = g.stage.cpu().numpy().view(np.uint16).reshape(c.stage.shape)


@pytest.mark.parametrize("D,H,QH,iters,T", [(256, 4, 24, 0, 700), (256, 2, 4, 0, 333), (128, 4, 24, 16, 600), (256, 2, 8, 16, 300)])
def test_general_kernel_head_dim_256_and_sinkhorn(D, H, QH, iters, T):
    """The reference engine's own geometry (head_dim 256, with and without Sinkhorn iterations) runs on the general
    kernel, a balanced head_dim-128 cache on the tuned kernels: decode, a 4-row verify step and a small prefill chunk,
    against the oracle on the same cache bytes."""
    import torch

    tw = Twin(D=D, H=H, QH=QH, capacity_tokens=T + 40, seed=101, iters=iters)
    k, v = orc.synth_kv(102, T + 40, H, D, 1), orc.synth_kv(102, T + 40, H, D, 2)
    tw.append(k[:T], v[:T])
    _sync_cpu_from_gpu(tw)
    scale = 1.0 / np.sqrt(D)
    q = orc.synth_q(102, 1, QH, D)
    want = tw.cpu.attention(q, [T - 1], scale, QH, threads=4)
    ok, msg = attn_close(_decode(tw, q[0], T - 1), want[0])
    assert ok, "decode: " + msg
    # verify step of 4 rows (append inside)
    q4 = orc.synth_q(103, 4, QH, D)
    pos = np.arange(T, T + 4, dtype=np.int32)
    out = tw.gpu.attn_verify(torch.from_numpy(q4).to(tw.dev), torch.from_numpy(k[T:T + 4]).to(tw.dev), torch.from_numpy(v[T:T + 4]).to(tw.dev),
                             torch.from_numpy(pos).to(tw.dev), scale, T + 40)
    torch.cuda.synchronize()
    tw.cpu.append(k[T:T + 4], v[T:T + 4], T)
    _sync_cpu_from_gpu(tw)
    want = tw.cpu.attention(q4, pos, scale, QH, threads=4)
    ok, msg = attn_close(out.float().cpu().numpy(), want)
    assert ok, "verify: " + msg
    # prefill chunk of 36 rows
    qc = orc.synth_q(104, 36, QH, D)
    pos = np.arange(T + 4, T + 40, dtype=np.int32)
    out = tw.gpu.attn_prefill(torch.from_numpy(qc).to(tw.dev), torch.from_numpy(k[T + 4:]).to(tw.dev), torch.from_numpy(v[T + 4:]).to(tw.dev),
                              torch.from_numpy(pos).to(tw.dev), scale, T + 40)
    torch.cuda.synchronize()
    tw.cpu.append(k[T + 4:], v[T + 4:], T + 4)
    _sync_cpu_from_gpu(tw)
    want = tw.cpu.attention(qc, pos, scale, QH, threads=4)
    from helpers import PREFILL_MAX_ABS, PREFILL_REL_L2
    ok, msg = attn_close(out.float().cpu().numpy(), want, *((PREFILL_MAX_ABS, PREFILL_REL_L2) if D == 128 else ()))  # head_dim 128: tcgen05 kernel
    assert ok, "prefill: " + msg
    assert tw.gpu.errors() == 0


@pytest.mark.parametrize("T", [1500, 5003])
def test_balanced_cache_on_the_tuned_kernel(T):
    """A head_dim-128 cache written with 16 Sinkhorn iterations (the engine's default) is read by the int8 decode
    kernel with the per-key factor on the logits and the per-dim factor on the outputs: decode, verify steps of 2, 5
    and 8 rows and a key-range partial, against the oracle over the very bytes the GPU wrote."""
    import torch

    H, QH, D = 4, 24, 128
    tw = Twin(D=D, H=H, QH=QH, capacity_tokens=T + 16, seed=131, iters=16)
    k, v = orc.synth_kv(132, T + 16, H, D, 1), orc.synth_kv(132, T + 16, H, D, 2)
    tw.append(k[:T], v[:T])
    scale = 1.0 / np.sqrt(D)
    cpu = cpu_twin_of(tw.gpu)
    q = orc.synth_q(132, 1, QH, D)
    want = cpu.attention(q, [T - 1], scale, QH, threads=8, kv_total=T)
    ok, msg = attn_close(_decode(tw, q[0], T - 1), want[0])
    assert ok, "decode: " + msg
    # a key range of the same cache as a partial, merged with the rest
    cut = (T // 2) // 128 * 128
    lib, capi = pkg().capi.load(), pkg().capi
    import ctypes as C
    qd = torch.from_numpy(q[0]).to(tw.dev)
    pos = torch.tensor([T - 1], dtype=torch.int32, device=tw.dev)
    pm = torch.empty((2, QH), dtype=torch.float32, device=tw.dev)
    pl = torch.empty((2, QH), dtype=torch.float32, device=tw.dev)
    po = torch.empty((2, QH, D), dtype=torch.float32, device=tw.dev)
    ws = tw.gpu.workspace(T + 16, 1)
    for i, (b, e) in enumerate(((0, cut), (cut, T))):
        capi.check(lib.kvb_attn_decode_partial(C.byref(tw.gpu.c), C.c_void_p(qd.data_ptr()), C.c_void_p(pos.data_ptr()), scale, T + 16, b, e,
                                               C.c_void_p(ws.data_ptr()), C.c_void_p(pm[i].data_ptr()), C.c_void_p(pl[i].data_ptr()),
                                               C.c_void_p(po[i].data_ptr()), None))
    out = pkg().merge_partials(pm, pl, po)
    torch.cuda.synchronize()
    ok, msg = attn_close(out.float().cpu().numpy(), want[0])
    assert ok, "two key ranges merged: " + msg
    # verify steps (appended rows stay in the stage, un-quantised)
    done = T
    for w in (2, 5, 8):
        qw = orc.synth_q(133 + w, w, QH, D)
        p = np.arange(done, done + w, dtype=np.int32)
        out = tw.gpu.attn_verify(torch.from_numpy(qw).to(tw.dev), torch.from_numpy(k[done:done + w]).to(tw.dev),
                                 torch.from_numpy(v[done:done + w]).to(tw.dev), torch.from_numpy(p).to(tw.dev), scale, T + 16)
        torch.cuda.synchronize()
        want_w = cpu_twin_of(tw.gpu).attention(qw, p, scale, QH, threads=8, kv_total=done + w)
        from helpers import PREFILL_MAX_ABS, PREFILL_REL_L2
        dense = w * (QH // H) >= 32  # the tcgen05 kernel rounds the de-quantised K and V to fp16
        ok, msg = attn_close(out.float().cpu().numpy(), want_w, *((PREFILL_MAX_ABS, PREFILL_REL_L2) if dense else ()))
        assert ok, f"verify of {w} rows: " + msg
    # a chunk of 300 rows that completes tiles, on the tcgen05 kernel (factors applied while de-quantising)
    done = T + 8
    n = 300
    k2, v2 = orc.synth_kv(140, n, H, D, 1), orc.synth_kv(140, n, H, D, 2)
    tw2 = Twin(D=D, H=H, QH=QH, capacity_tokens=T + n + 16, seed=133, iters=16)
    tw2.append(k[:T], v[:T])
    qc = orc.synth_q(141, n, QH, D)
    p = np.arange(T, T + n, dtype=np.int32)
    out = tw2.gpu.attn_prefill(torch.from_numpy(qc).to(tw.dev), torch.from_numpy(k2).to(tw.dev), torch.from_numpy(v2).to(tw.dev),
                               torch.from_numpy(p).to(tw.dev), scale, T + n + 16)
    torch.cuda.synchronize()
    want_c = cpu_twin_of(tw2.gpu).attention(qc, p, scale, QH, threads=8, kv_total=T + n)
    ok, msg = attn_close(out.float().cpu().numpy(), want_c, PREFILL_MAX_ABS, PREFILL_REL_L2)
    assert ok, "prefill chunk: " + msg
    assert tw.gpu.errors() == 0 and tw2.gpu.errors() == 0


def test_sharded_verify_ring_loopback():
    """kvb_attn_rows_sharded on one GPU with a one-rank ring: verify steps of 1..8 rows equal kvb_attn_rows of the same
    cache on the warp-level kernel bit for bit (same partials, same merge); a ring sized for one token refuses a
    wider step."""
    import ctypes as C

    import torch

    capi = pkg().capi
    sh = pkg().sharded
    T = 2100
    tw = Twin(D=128, H=4, QH=24, capacity_tokens=T + 16, seed=121)
    k, v = orc.synth_kv(122, T + 8, 4, 128, 1), orc.synth_kv(122, T + 8, 4, 128, 2)
    tw.append(k[:T], v[:T])
    scale = 1.0 / np.sqrt(128)
    ring = sh.PeerRing.loopback(24, 128, tw.dev, tokens=8)
    dec = sh.RingShardedDecode(tw.gpu, ring)
    for w in (1, 3, 5, 8, 2):
        qw = torch.from_numpy(orc.synth_q(123 + w, w, 24, 128)).to(tw.dev)
        pos = torch.arange(T, T + w, dtype=torch.int32, device=tw.dev)
        out = torch.empty_like(qw)
        dec.attn_verify(qw, torch.from_numpy(k[T:T + w]).to(tw.dev), torch.from_numpy(v[T:T + w]).to(tw.dev), pos, scale, T + 16, out,
                        owner=True)
        torch.cuda.synchronize()
        want = cpu_twin_of(tw.gpu).attention(qw.cpu().numpy(), pos.cpu().numpy(), scale, 24, threads=8, kv_total=T + w)
        ok, msg = attn_close(out.float().cpu().numpy(), want)
        assert ok, f"{w} rows: " + msg
    assert tw.gpu.errors() == 0
    small = sh.PeerRing.loopback(24, 128, tw.dev)  # holds one token
    lib = capi.load()
    q2 = torch.zeros((2, 24, 128), dtype=torch.float16, device=tw.dev)
    pos2 = torch.arange(T, T + 2, dtype=torch.int32, device=tw.dev)
    st = lib.kvb_attn_rows_sharded(C.byref(tw.gpu.c), C.c_void_p(q2.data_ptr()), C.c_void_p(pos2.data_ptr()), 2, scale, T + 16,
                                   C.c_void_p(tw.gpu.workspace(T + 16, 2).data_ptr()), C.byref(small.c), C.c_void_p(q2.data_ptr()), None)
    assert st == capi.KVB_ERANGE


def test_sharded_decode_ring_loopback_and_bounded_wait():
    """kvb_attn_decode_sharded on one GPU: with a one-rank ring the result equals kvb_attn_decode on every call (both
    ring slots, advancing call numbers); with a second rank that never sends, the bounded wait runs out, the error
    word reports it, zeros are written and the next call still works -- nothing hangs."""
    import torch

    capi = pkg().capi
    sh = pkg().sharded
    T = 1100
    tw = Twin(D=128, H=4, QH=24, capacity_tokens=T, seed=111)
    k, v = orc.synth_kv(112, T, 4, 128, 1), orc.synth_kv(112, T, 4, 128, 2)
    tw.append(k, v)
    pos = torch.tensor([T - 1], dtype=torch.int32, device=tw.dev)
    scale = 1.0 / np.sqrt(128)
    ring = sh.PeerRing.loopback(24, 128, tw.dev)
    dec = sh.RingShardedDecode(tw.gpu, ring)
    for call in range(5):
        qd = torch.from_numpy(orc.synth_q(113 + call, 1, 24, 128)[0]).to(tw.dev)
        out = torch.empty_like(qd)
        dec.attn_decode(qd, pos, scale, T, out)
        ref = tw.gpu.attn_decode(qd, pos, scale, T)
        torch.cuda.synchronize()
        assert torch.equal(out, ref), call
    assert int(ring.state[0].item()) == 5 and tw.gpu.errors() == 0
    # a rank that never arrives: the wait is bounded
    ring2 = sh.PeerRing.loopback(24, 128, tw.dev, world=2, rank=0, max_spins=2000)
    dec2 = sh.RingShardedDecode(tw.gpu, ring2)
    out = torch.full((24, 128), 7.0, dtype=torch.float16, device=tw.dev)
    dec2.attn_decode(qd, pos, scale, T, out)
    torch.cuda.synchronize()
    assert tw.gpu.errors() & capi.ERR_WAIT_TIMEOUT
    assert not out.any()
    assert int(ring2.state[0].item()) == 1


def test_sharded_decode_ring_merges_arrived_peers_in_rank_order():
    """Receive + merge of kvb_attn_decode_sharded with 4 ranks, checked on one GPU without any waiting: the three
    peers' words (value | call number, the ring's wire format) are placed in this rank's ring buffer before the
    launch, as if they had arrived early.  The result must equal kvb_merge_partials over the four partials in rank
    order bit for bit, for both ring slots, and what this rank sends must show up in every peer's buffer."""
    import torch

    sh = pkg().sharded
    cache = pkg().cache
    QH, D, world, rank = 24, 128, 4, 2
    scale = 1.0 / np.sqrt(D)
    lens = [700, 1100, 900, 333]
    twins = []
    for r in range(world):
        tw = Twin(D=D, H=4, QH=QH, capacity_tokens=lens[r], seed=300 + r)
        tw.append(orc.synth_kv(310 + r, lens[r], 4, D, 1), orc.synth_kv(310 + r, lens[r], 4, D, 2))
        twins.append(tw)
    dev = twins[0].dev
    ring = sh.PeerRing.loopback(QH, D, dev, world=world, rank=rank, max_spins=1000)
    dec = sh.RingShardedDecode(twins[rank].gpu, ring)
    block = QH * (D + 2)
    for call in (1, 2, 3):
        qd = torch.from_numpy(orc.synth_q(320 + call, 1, QH, D)[0]).to(dev)
        ms, ls, os_ = [], [], []
        for r in range(world):
            pos = torch.tensor([lens[r] - 1], dtype=torch.int32, device=dev)
            m, l, o = twins[r].gpu.attn_decode_partial(qd, pos, scale, lens[r])
            ms.append(m.clone()); ls.append(l.clone()); os_.append(o.clone())
        want = cache.merge_partials(torch.stack(ms), torch.stack(ls), torch.stack(os_))
        words = ring.local_buf.view(torch.int32).view(2, world, block, 2)
        for r in range(world):
            if r == rank:
                continue
            vals = torch.cat([torch.stack([ms[r], ls[r]], dim=1).reshape(-1), os_[r].reshape(-1)])
            words[call & 1, r, :, 0] = vals.view(torch.int32)
            words[call & 1, r, :, 1] = call
        out = torch.empty_like(qd)
        pos = torch.tensor([lens[rank] - 1], dtype=torch.int32, device=dev)
        dec.attn_decode(qd, pos, scale, lens[rank], out)
        torch.cuda.synchronize()
        assert twins[rank].gpu.errors() == 0
        assert torch.equal(out, want), call
        mine = torch.cat([torch.stack([ms[rank], ls[rank]], dim=1).reshape(-1), os_[rank].reshape(-1)]).view(torch.int32)
        for r in range(world):
            if r == rank:
                continue
            sent = ring._keep[r].view(torch.int32).view(2, world, block, 2)[call & 1, rank]
            assert torch.equal(sent[:, 0], mine) and bool((sent[:, 1] == call).all()), (call, r)
    assert int(ring.state[0].item()) == 3


def test_batched_decode_equals_one_call_per_sequence():
    """kvb_attn_decode_batch over sequences of very different lengths (shorter than a tile, exactly one tile, long
    ones) against the oracle, sequence by sequence, and against kvb_attn_decode (same kernels, but the keys are cut
    into different splits, so the last bits may differ); bounds larger than the true lengths still work."""
    import torch

    lens = [5, 128, 700, 1100, 64, 3001, 257, 1999]
    twins = []
    for i, n in enumerate(lens):
        tw = Twin(D=128, H=4, QH=24, capacity_tokens=n + 8, seed=400 + i)
        tw.append(orc.synth_kv(410 + i, n, 4, 128, 1), orc.synth_kv(410 + i, n, 4, 128, 2))
        twins.append(tw)
    dev = twins[0].dev
    scale = 1.0 / np.sqrt(128)
    qh = np.stack([orc.synth_q(420 + i, 1, 24, 128)[0] for i in range(len(lens))])
    q = torch.from_numpy(qh).to(dev)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=dev)
    want = torch.stack([tw.gpu.attn_decode(q[i], pos[i:i + 1], scale, lens[i]) for i, tw in enumerate(twins)])
    for slack in (0, 4096):
        batch = pkg().DecodeBatch([tw.gpu for tw in twins], [n + slack for n in lens])
        out = batch.attn_decode(q, pos, scale)
        torch.cuda.synchronize()
        assert (out.float() - want.float()).abs().max().item() <= 2.0 ** -9 * want.float().abs().max().item(), slack
        for i, tw in enumerate(twins):
            ref = tw.cpu.attention(qh[i:i + 1], np.array([lens[i] - 1], np.int32), scale, 24, threads=2)
            ok, msg = attn_close(out[i:i + 1].float().cpu().numpy(), ref)
            assert ok, f"sequence {i} (slack {slack}): {msg}"
            assert tw.gpu.errors() == 0


def test_batched_decode_refuses_bad_arguments():
    import ctypes as C

    capi = pkg().capi
    lib = capi.load()
    bounds = (C.c_int32 * 2)(100, 0)
    assert lib.kvb_batch_workspace_bytes(bounds, 2, 4, 24, 128) == 0          # a bound of zero
    bounds = (C.c_int32 * 2)(100, 100)
    assert lib.kvb_batch_workspace_bytes(bounds, 2, 4, 24, 256) == 0          # head_dim 256: one call per sequence
    assert lib.kvb_batch_workspace_bytes(bounds, 2, 4, 24, 128) > 0
    fake = C.c_void_p(256)
    st = lib.kvb_attn_decode_batch(fake, 65, 4, 24, 128, 0, fake, fake, 0.1, bounds, fake, fake, None)
    assert st == capi.KVB_ERANGE
    st = lib.kvb_attn_decode_batch(fake, 2, 4, 24, 128, 0, fake, fake, 0.1, bounds, None, fake, None)
    assert st == capi.KVB_EINVAL
