"""Cross-GPU test of the range-sharded decode whose partials are exchanged by the kernels over NVLink peer memory
(kvb_attn_decode_sharded).  Runs only where at least two GPUs are visible: two ranks as child processes, one GPU each,
NCCL for the rendezvous only (NVLS off), plain peer stores on the data path.

  * every rank's output equals the single-GPU decode of the unsharded cache and the CPU oracle, over several calls
    (both ring slots, advancing call numbers), including steps that append a token on the rank that owns the open tile;
  * a call whose peer never launches (it stays alive and simply skips the call: a flag that nothing sets) runs out of
    its bounded wait, reports KVB_ERR_WAIT_TIMEOUT in the error word and writes zeros; the context stays usable.
No rank leaves while a kernel is in flight; nothing here faults, traps or hangs a GPU.
"""
import os
import socket

import numpy as np
import pytest

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, attn_close, orc, pkg

pytestmark = pytest.mark.gpu


def _gpu_count():
    import torch

    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, T, ret):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0",
                       "RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank)})
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        p = pkg()
        sh, capi = p.sharded, p.capi
        D, H, QH = 128, 4, 24
        steps = 5
        k, v = orc.synth_kv(90, T + steps, H, D, 1), orc.synth_kv(90, T + steps, H, D, 2)
        q = orc.synth_q(90, steps, QH, D)
        scale = 1.0 / np.sqrt(D)

        def filled(n_tokens, k_rows, v_rows, seed, room):
            room += 96  # the verify steps and the chunk below
            lp = (n_tokens + room + 63) // 64 + 2
            lp += lp & 1
            L = p.KvarnLayer(D, H, QH, lp, torch.from_numpy(orc.shuffled_table(seed, lp, lp)), device=str(dev))
            if n_tokens:
                L.append(torch.from_numpy(k_rows).to(dev), torch.from_numpy(v_rows).to(dev),
                         torch.arange(n_tokens, dtype=torch.int32, device=dev))
            return L

        full = filled(T, k[:T], v[:T], 5, steps + 2)            # the unsharded cache, on every rank, as the reference
        b, e = sh.tile_ranges(T, world)[rank]
        n = e - b
        owner = rank == world - 1
        local = filled(n, k[b:e], v[b:e], 11 + rank, steps + 2)  # this rank's tile range as a cache of its own
        cpu = orc.CpuLayer(D, H, T // 64 + 8, orc.shuffled_table(3, T // 64 + 8, T // 64 + 8))
        cpu.append(k[:T], v[:T], 0)
        ring = sh.PeerRing.symmetric(QH, D, dev)
        dec = sh.RingShardedDecode(local, ring)
        out = torch.empty((QH, D), dtype=torch.float16, device=dev)
        worst = 0.0
        for s in range(steps):
            # one decode step of the sequence: the new token goes to the owner of the open tile, then every rank attends
            row_k, row_v = torch.from_numpy(k[T + s:T + s + 1]).to(dev), torch.from_numpy(v[T + s:T + s + 1]).to(dev)
            gpos = torch.tensor([T + s], dtype=torch.int32, device=dev)
            full.append(row_k, row_v, gpos)
            cpu.append(k[T + s:T + s + 1], v[T + s:T + s + 1], T + s)
            if owner:
                lpos = torch.tensor([n + s], dtype=torch.int32, device=dev)
                local.append(row_k, row_v, lpos)
            else:
                lpos = torch.tensor([n - 1], dtype=torch.int32, device=dev)
            qd = torch.from_numpy(q[s]).to(dev)
            dec.attn_decode(qd, lpos, scale, n + steps + 2, out)
            ref = full.attn_decode(qd, gpos, scale, T + steps + 2)
            torch.cuda.synchronize()
            want = cpu.attention(q[s:s + 1], [T + s], scale, QH, threads=4)[0]
            ok, msg = attn_close(out.float().cpu().numpy(), want, ATTN_MAX_ABS, ATTN_REL_L2)
            assert ok, f"rank {rank} step {s} vs oracle: {msg}"
            ok, msg = attn_close(out.float().cpu().numpy(), ref.float().cpu().numpy().astype(np.float64), ATTN_MAX_ABS, ATTN_REL_L2)
            assert ok, f"rank {rank} step {s} vs the single-GPU decode: {msg}"
            worst = max(worst, float((out.float() - ref.float()).abs().max()))
        assert local.errors() == 0 and full.errors() == 0
        assert int(ring.state[0].item()) == steps
        dist.barrier()
        # ---- verify steps of 3 and 8 rows over the sharded sequence, partials exchanged by the reduce kernel (a ring that
        #      holds eight tokens); against the single-GPU verify of the unsharded cache.  The rows are rolled back after
        #      each step (the same positions are written again).
        ring8 = sh.PeerRing.symmetric(QH, D, dev, tokens=8)
        dec8 = sh.RingShardedDecode(local, ring8)
        base_full, base_local = T + steps, n + steps
        kx, vx = orc.synth_kv(91, 8, H, D, 1), orc.synth_kv(91, 8, H, D, 2)
        for w in (3, 8):
            qw = torch.from_numpy(orc.synth_q(92 + w, w, QH, D)).to(dev)
            kw, vw = torch.from_numpy(kx[:w]).to(dev), torch.from_numpy(vx[:w]).to(dev)
            gpos = torch.arange(base_full, base_full + w, dtype=torch.int32, device=dev)
            lpos = (torch.arange(base_local, base_local + w, dtype=torch.int32, device=dev) if owner
                    else torch.full((w,), n - 1, dtype=torch.int32, device=dev))
            out_w = torch.empty((w, QH, D), dtype=torch.float16, device=dev)
            dec8.attn_verify(qw, kw, vw, lpos, scale, n + steps + 16, out_w, owner=owner)
            ref_w = full.attn_verify(qw, kw, vw, gpos, scale, T + steps + 16)
            torch.cuda.synchronize()
            ok, msg = attn_close(out_w.float().cpu().numpy(), ref_w.float().cpu().numpy().astype(np.float64), 2.0 ** -8, 5e-3)
            assert ok, f"rank {rank} verify of {w} rows vs the single-GPU verify: {msg}"
        assert local.errors() == 0 and full.errors() == 0
        dist.barrier()
        # ---- a chunk of 64 tokens over the sharded sequence (ShardedChunk: per-rank partials, all-to-all of row shares,
        #      merge, gather of the finished rows) against the single-GPU chunk attention of the unsharded cache
        C = 64
        kc, vc = orc.synth_kv(95, C, H, D, 1), orc.synth_kv(95, C, H, D, 2)
        qc = torch.from_numpy(orc.synth_q(96, C, QH, D)).to(dev)
        kcd, vcd = torch.from_numpy(kc).to(dev), torch.from_numpy(vc).to(dev)
        gpos = torch.arange(base_full, base_full + C, dtype=torch.int32, device=dev)
        lpos = (torch.arange(base_local, base_local + C, dtype=torch.int32, device=dev) if owner
                else torch.full((C,), n - 1, dtype=torch.int32, device=dev))
        chunk = sh.ShardedChunk(local, C)
        out_c = torch.empty((C, QH, D), dtype=torch.float16, device=dev)
        chunk.attend(qc, kcd, vcd, lpos, scale, n + steps + 96, out_c)
        ref_c = full.attn_prefill(qc, kcd, vcd, gpos, scale, T + steps + 96)
        torch.cuda.synchronize()
        ok, msg = attn_close(out_c.float().cpu().numpy(), ref_c.float().cpu().numpy().astype(np.float64), 2.0 ** -8, 5e-3)
        assert ok, f"rank {rank} sharded chunk vs the single-GPU chunk: {msg}"
        assert local.errors() == 0 and full.errors() == 0
        dist.barrier()
        # ---- a peer that never launches: rank 0 calls on a fresh ring with a short wait, rank 1 skips the call
        ring2 = sh.PeerRing.symmetric(QH, D, dev, max_spins=2000)
        dist.barrier()
        if rank == 0:
            dec2 = sh.RingShardedDecode(local, ring2)
            out.fill_(1.0)
            dec2.attn_decode(torch.from_numpy(q[0]).to(dev), torch.tensor([n - 1], dtype=torch.int32, device=dev), scale, n + steps + 2, out)
            torch.cuda.synchronize()
            assert local.errors() & capi.ERR_WAIT_TIMEOUT, "the wait should have run out"
            assert float(out.float().abs().max()) == 0.0, "a wait that ran out must give zeros, not a half-merged row"
            local.error_word.zero_()
            again = full.attn_decode(torch.from_numpy(q[0]).to(dev), torch.tensor([T], dtype=torch.int32, device=dev), scale, T + steps + 2)
            torch.cuda.synchronize()
            assert torch.isfinite(again.float()).all() and full.errors() == 0  # the context is still usable
        dist.barrier()  # rank 1 learns on the host that the step is over; nobody left with work in flight
        ret.put((rank, worst))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("T", [5000, 1100])
def test_ring_sharded_decode_on_two_gpus(T):
    import torch.multiprocessing as mp

    pkg()
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, T, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    got = dict(ret.get(timeout=5) for _ in range(2))
    assert set(got) == {0, 1}
