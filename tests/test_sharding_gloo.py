"""CPU tests of the multi-GPU host logic with world_size 2 over gloo: range partition, one all-gather of packed
partials, log-sum-exp merge -- checked against the single-rank oracle.  The per-rank attention is the CPU
oracle here (no GPU); on GPUs the same packing / gather / merge code runs on kvb_attn_decode_partial outputs."""
import os
import socket

import numpy as np
import pytest

from helpers import orc, pkg


def test_tile_ranges_and_dealing():
    sh = pkg().sharded
    assert sh.tile_ranges(378944, 8) == [(i * 47360, (i + 1) * 47360) for i in range(7)] + [(331520, 378944)]
    r = sh.tile_ranges(1000, 4)
    assert r[0][0] == 0 and r[-1][1] == 1000 and all(a[1] == b[0] for a, b in zip(r, r[1:]))
    assert all((b - a) % 128 == 0 for a, b in r[:-1])
    assert sh.tile_ranges(100, 2) == [(0, 0), (0, 100)]
    lens = [131072, 16384, 90000, 20000, 65536, 65536, 30000]
    deal = sh.deal_sequences(lens, 3)
    assert sorted(i for d in deal for i in d) == list(range(len(lens)))
    loads = [sum(lens[i] for i in d) for d in deal]
    assert max(loads) - min(loads) <= max(lens)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, T, ret, rows=1):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sh = pkg().sharded
    D, H, QH = 128, 4, 24
    k, v = orc.synth_kv(80, T, H, D, 1), orc.synth_kv(80, T, H, D, 2)
    q = orc.synth_q(80, rows, QH, D)
    T -= rows - 1  # the last `rows` tokens are the query rows of a verify step: row i sees keys 0 .. T - 1 + i
    b, e = sh.tile_ranges(T + rows - 1, world)[rank]
    n = e - b
    lp = n // 64 + 4
    local = orc.CpuLayer(D, H, lp, orc.shuffled_table(rank, lp, lp))
    if n:
        local.append(k[b:e], v[b:e], 0)
    scale = 1.0 / np.sqrt(D)
    # positions in the local cache: the owner of the open tile (last rank) holds the query rows' own keys, the
    # other ranks see all of their range
    if rank == world - 1:
        lpos = np.arange(n - rows, n, dtype=np.int32)
    else:
        lpos = np.full(rows, n - 1, np.int32)
    if n:
        _, m, l, o = local.attention(q, lpos, scale, QH, want_partials=True)
    else:  # a rank without keys contributes the neutral partial
        m = np.full((rows, QH), -np.inf, np.float32); l = np.zeros((rows, QH), np.float32); o = np.zeros((rows, QH, D), np.float32)
    packed = sh.pack_partial(torch.from_numpy(m.reshape(-1)), torch.from_numpy(l.reshape(-1)), torch.from_numpy(o.reshape(-1, D)))
    gathered = sh.all_gather_partials(packed)
    gm, gl, go = sh.unpack_partials(gathered)
    merged = orc.merge_partials(gm.numpy(), gl.numpy(), go.numpy())
    if rank == 0:
        total = T + rows - 1
        full = orc.CpuLayer(D, H, total // 64 + 4, orc.shuffled_table(9, total // 64 + 4, total // 64 + 4))
        full.append(k, v, 0)
        want = full.attention(q, np.arange(total - rows, total, dtype=np.int32), scale, QH).reshape(rows * QH, D)
        ret.put(float(np.abs(merged - want).max() / np.abs(want).max()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("T,rows", [(1000, 1), (100, 1), (1000, 5), (300, 8)])
def test_range_sharded_decode_world2(T, rows):
    """rows = 1: decode.  rows > 1: a verify step whose rows are the last tokens of the sequence (the same partition /
    all-gather / merge with tokens * q_heads rows per rank, what kvb_attn_chunk_partial feeds on GPUs)."""
    import torch.multiprocessing as mp

    pkg()
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, T, ret, rows)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert ret.get(timeout=5) < 1e-5
