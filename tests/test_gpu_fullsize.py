"""Full-size cases (one sequence of 378,944 tokens; a 1,024-token chunk over 262,144 tokens; verify steps over 131,072
tokens; 32 sequences of 16K..131K tokens; 24 / 4 heads, head_dim 128).  Each compares sampled rows with the CPU
oracle run over the very bytes the GPU wrote (the planes are copied into an oracle layer), and keeps the
size-independent properties:
  * the planes do not depend on how the tokens were chunked into appends, nor on where the pages lie: two caches
    with different page tables, filled in chunks of 8,192 and of 4,099 tokens, hold the same bytes page for page;
  * decode attention is bit-identical on the two caches (same logical content, different physical placement);
  * the partials of eight tile-aligned key ranges merge to the full result (log-sum-exp associativity);
  * a looser host bound of the length (kv_len_max) changes the split grid but not the result beyond tolerance.
"""
import numpy as np
import pytest

from helpers import (ATTN_MAX_ABS, ATTN_REL_L2, PREFILL_MAX_ABS, PREFILL_REL_L2, attn_close, cpu_twin_of, host_threads,
                     orc, pkg)

pytestmark = pytest.mark.gpu

T, D, H, QH = 378_944, 128, 4, 24


def _fill(layer, k, v, chunk, dev):
    import torch

    for c0 in range(0, T, chunk):
        n = min(chunk, T - c0)
        layer.append(k[c0:c0 + n], v[c0:c0 + n], torch.arange(c0, c0 + n, dtype=torch.int32, device=dev))


def test_config_4a_properties():
    import torch

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(4242)
    k = torch.randn((T, H, D), generator=gen, device=dev, dtype=torch.float32)
    k[..., [3, 17, 64, 101]] *= 20.0
    k = k.to(torch.float16)
    v = torch.randn((T, H, D), generator=gen, device=dev, dtype=torch.float32).to(torch.float16)
    q = torch.randn((QH, D), generator=gen, device=dev, dtype=torch.float32).to(torch.float16)
    lp = (T + 63) // 64 + 2
    lp += lp & 1
    rng = np.random.default_rng(7)
    tables = [torch.from_numpy(rng.permutation(lp + 5)[:lp].astype(np.int32)) for _ in range(2)]
    A = pkg().KvarnLayer(D, H, QH, lp + 5, tables[0], device="cuda:0")
    B = pkg().KvarnLayer(D, H, QH, lp + 5, tables[1], device="cuda:0")
    _fill(A, k, v, 8192, dev)
    _fill(B, k, v, 4099, dev)
    torch.cuda.synchronize()
    assert A.errors() == 0 and B.errors() == 0
    # same bytes, logical page for logical page
    sealed_pages = 2 * (T // 128)
    ta, tb = tables[0][:sealed_pages].to(dev).long(), tables[1][:sealed_pages].to(dev).long()
    for name in ("k_code", "v_code", "k_scale", "v_scale"):
        assert torch.equal(getattr(A, name)[ta], getattr(B, name)[tb]), name
    # the open tile (64 tokens of tile 2960, stage slot 0) lives in the stage, identically; rows beyond it are stale
    # rows of earlier tiles, whose content depends on the chunking and is never read
    open_tile, live = T // 128, T % 128
    sa, sb = A.stage.view(2, 2, H, 128, D), B.stage.view(2, 2, H, 128, D)
    assert live == 64 and torch.equal(sa[:, open_tile & 1, :, :live], sb[:, open_tile & 1, :, :live])
    pos = torch.tensor([T - 1], dtype=torch.int32, device=dev)
    scale = 1.0 / np.sqrt(D)
    full_a = A.attn_decode(q, pos, scale, T)
    full_b = B.attn_decode(q, pos, scale, T)
    torch.cuda.synchronize()
    assert torch.isfinite(full_a.float()).all()
    assert torch.equal(full_a, full_b)
    # the oracle over the same bytes: the whole decode row at 378,944 tokens, and its partials over eight ranges
    cpu = cpu_twin_of(A)
    qn = q.cpu().numpy()[None]
    want = cpu.attention(qn, [T - 1], scale, QH, threads=host_threads(), kv_total=T)[0]
    ok, msg = attn_close(full_a.float().cpu().numpy(), want, ATTN_MAX_ABS, ATTN_REL_L2)
    assert ok, msg
    # eight tile-aligned key ranges -> partials -> merge
    tiles = (T + 127) // 128
    ms, ls, os_ = [], [], []
    for r in range(8):
        b, e = 128 * (tiles * r // 8), min(T, 128 * (tiles * (r + 1) // 8))
        m, l, o = A.attn_decode_partial(q, pos, scale, T, key_begin=b, key_end=e)
        ms.append(m.clone()); ls.append(l.clone()); os_.append(o.clone())
    merged = pkg().cache.merge_partials(torch.stack(ms), torch.stack(ls), torch.stack(os_))
    ok, msg = attn_close(merged.float().cpu().numpy(), want, ATTN_MAX_ABS, ATTN_REL_L2)
    assert ok, "eight ranges merged vs oracle: " + msg
    ref = full_a.float()
    tol = 2.0 ** -10 * ref.abs().max().item()
    assert (merged.float() - ref).abs().max().item() <= tol
    # a looser bound of the length: other splits, same answer
    loose = A.attn_decode(q, pos, scale, T + 50_000)
    assert (loose.float() - ref).abs().max().item() <= tol
    assert A.errors() == 0


def test_config_3_chunk_rows_equal_single_row_decodes():
    """Full size (a 1,024-token chunk over a 262,144-token prefix): rows 0, 500 and 1,023 against the oracle; and every row of a causal chunk
    attention is the decode attention of that row alone over the keys it may see.  Rows 0, 500 and 1,023 of the
    tensor-core chunk kernel against the warp-level decode kernel on the same cache (two independent kernels),
    within the chunk kernel's tolerance."""
    import torch

    prefix, chunk = 262_144, 1024
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(99)

    def rows(n, heads):
        x = torch.randn((n, heads, D), generator=gen, device=dev, dtype=torch.float32)
        x[..., [3, 17, 64, 101]] *= 20.0
        return x.to(torch.float16)

    lp = (prefix + chunk + 63) // 64 + 2
    lp += lp & 1
    table = torch.from_numpy(np.random.default_rng(3).permutation(lp).astype(np.int32))
    L = pkg().KvarnLayer(D, H, QH, lp, table, device="cuda:0")
    for c0 in range(0, prefix, 8192):
        L.append(rows(8192, H), rows(8192, H), torch.arange(c0, c0 + 8192, dtype=torch.int32, device=dev))
    q, k, v = rows(chunk, QH), rows(chunk, H), rows(chunk, H)
    pos = torch.arange(prefix, prefix + chunk, dtype=torch.int32, device=dev)
    scale = 1.0 / np.sqrt(D)
    out = L.attn_prefill(q, k, v, pos, scale, prefix + chunk)
    torch.cuda.synchronize()
    assert L.errors() == 0 and torch.isfinite(out.float()).all()
    sample = [0, 500, chunk - 1]
    cpu = cpu_twin_of(L)
    want = cpu.attention(q[sample].cpu().numpy(), [prefix + i for i in sample], scale, QH, threads=host_threads(),
                         kv_total=prefix + chunk)
    for j, i in enumerate(sample):
        ok, msg = attn_close(out[i].float().cpu().numpy(), want[j], PREFILL_MAX_ABS, PREFILL_REL_L2)
        assert ok, f"chunk row {i} vs oracle: {msg}"
    for i in (0, 500, chunk - 1):
        ref = L.attn_decode(q[i], pos[i:i + 1], scale, prefix + chunk).float()
        got = out[i].float()
        assert (got - ref).abs().max().item() <= 2.0 ** -8 * ref.abs().max().item(), i
        assert ((got - ref).norm() / ref.norm()).item() <= 5e-3, i
    assert L.errors() == 0


def test_config_2_verify_rows_equal_single_row_decodes():
    """Full size (verify steps of 4 and 8 draft rows over a 131,072-token prefix): every row against the oracle; and row i of a verify step equals the
    decode of row i alone; width 4 runs on the warp-level kernel, width 8 on the tensor-core chunk kernel.  The
    second step re-appends at the same positions (the drafts of the first were rolled back)."""
    import torch

    prefix = 131_072
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)

    def rows(n, heads):
        x = torch.randn((n, heads, D), generator=gen, device=dev, dtype=torch.float32)
        x[..., [3, 17, 64, 101]] *= 20.0
        return x.to(torch.float16)

    lp = (prefix + 8 + 63) // 64 + 2
    lp += lp & 1
    L = pkg().KvarnLayer(D, H, QH, lp, torch.from_numpy(np.random.default_rng(4).permutation(lp).astype(np.int32)), device="cuda:0")
    for c0 in range(0, prefix, 8192):
        L.append(rows(8192, H), rows(8192, H), torch.arange(c0, c0 + 8192, dtype=torch.int32, device=dev))
    scale = 1.0 / np.sqrt(D)
    for width in (4, 8):
        q, k, v = rows(width, QH), rows(width, H), rows(width, H)
        pos = torch.arange(prefix, prefix + width, dtype=torch.int32, device=dev)
        out = L.attn_verify(q, k, v, pos, scale, prefix + 8)
        torch.cuda.synchronize()
        # every row against the oracle over the bytes this step left in the cache (its new rows are in the stage)
        dense = width * (QH // H) >= 32  # the tcgen05 chunk kernel rounds the de-quantised tiles to fp16
        want = cpu_twin_of(L).attention(q.cpu().numpy(), pos.cpu().numpy(), scale, QH, threads=host_threads(),
                                        kv_total=prefix + width)
        ok, msg = attn_close(out.float().cpu().numpy(), want, PREFILL_MAX_ABS if dense else ATTN_MAX_ABS,
                             PREFILL_REL_L2 if dense else ATTN_REL_L2)
        assert ok, f"width {width} vs oracle: {msg}"
        for i in range(width):
            ref = L.attn_decode(q[i], pos[i:i + 1], scale, prefix + 8).float()
            got = out[i].float()
            assert (got - ref).abs().max().item() <= 2.0 ** -8 * ref.abs().max().item(), (width, i)
            assert ((got - ref).norm() / ref.norm()).item() <= 5e-3, (width, i)
    assert L.errors() == 0


def test_config_4b_batched_decode_equals_one_call_per_sequence():
    """Full size (32 sequences of 16,384 .. 131,072 tokens): one kvb_attn_decode_batch call against the oracle on three
    sequences, and against one kvb_attn_decode per sequence (same kernels, different cuts of the keys)."""
    import random

    import torch

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(6)
    rnd = random.Random(0)
    lengths = [rnd.randint(16384, 131072) for _ in range(32)]
    pool_k = torch.randn((131072 + 4096, H, D), generator=gen, device=dev, dtype=torch.float32).to(torch.float16)
    pool_v = torch.randn((131072 + 4096, H, D), generator=gen, device=dev, dtype=torch.float32).to(torch.float16)
    layers = []
    for i, n in enumerate(lengths):
        lp = (n + 63) // 64 + 2
        lp += lp & 1
        L = pkg().KvarnLayer(D, H, QH, lp, torch.from_numpy(np.random.default_rng(100 + i).permutation(lp).astype(np.int32)), device="cuda:0")
        shift = 17 * i  # every sequence reads the pool at its own offset: different content per sequence
        for c0 in range(0, n, 8192):
            m = min(8192, n - c0)
            L.append(pool_k[shift + c0:shift + c0 + m], pool_v[shift + c0:shift + c0 + m], torch.arange(c0, c0 + m, dtype=torch.int32, device=dev))
        layers.append(L)
    q = torch.randn((32, QH, D), generator=gen, device=dev, dtype=torch.float32).to(torch.float16)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=dev)
    scale = 1.0 / np.sqrt(D)
    want = torch.stack([L.attn_decode(q[i], pos[i:i + 1], scale, lengths[i]) for i, L in enumerate(layers)]).float()
    out = pkg().DecodeBatch(layers, lengths).attn_decode(q, pos, scale).float()
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    # The two differ by more than summation order: the weights p * scale_V are rounded to fp16 relative to the running
    # maximum at the time, which depends on where the keys were cut, and that rounding noise is common to all dims of
    # a head (it shows up in dim 0 after the inverse rotation).  An output here is the average of 10^5 random values,
    # about 0.02, so the noise is judged against the scale of V itself: below 2^-13 of the largest |V|.
    vmax = pool_v.float().abs().max().item()
    order = sorted(range(32), key=lambda i: lengths[i])
    for i in (order[0], order[16], order[-1]):  # shortest, a middle one, longest: the batched call against the oracle
        want_i = cpu_twin_of(layers[i]).attention(q[i].cpu().numpy()[None], [lengths[i] - 1], scale, QH,
                                                  threads=host_threads(), kv_total=lengths[i])[0]
        ok, msg = attn_close(out[i].cpu().numpy(), want_i, ATTN_MAX_ABS, ATTN_REL_L2)
        assert ok, f"sequence {i} ({lengths[i]} tokens) vs oracle: {msg}"
    for i in range(32):
        assert (out[i] - want[i]).abs().max().item() <= 2.0 ** -13 * vmax, i
        assert ((out[i] - want[i]).norm() / want[i].norm()).item() <= 5e-3, i
    assert all(L.errors() == 0 for L in layers)
