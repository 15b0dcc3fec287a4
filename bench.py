#!/usr/bin/env python3
"""Benchmark of the KVarN quantized-KV hot path on B200.

Contract line (`python bench.py --gpus N --steps K --warmup W`, under torchrun for N > 1): batch-1 decode of ONE
sequence of 378,944 tokens (5,921 pages of 64 tokens) across 16 attention layers, 24 query heads / 4 KV heads /
head_dim 128, seed-shuffled page table per layer.  One step = for each layer: append 1 new token (on the rank that
owns the open tile), then one decode query over the whole cache.  On N > 1 GPUs the context is cut into contiguous
tile ranges, one per rank (strong scaling: the total work is fixed); every rank attends its range and the (m, l, o)
partials are exchanged by the kernels themselves over NVLink peer memory (kvb_attn_decode_sharded).

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # the CPU path (oracle port) on the host cores
    python bench.py --workload decode32k|decodectx|batch32|verify131k|prefill262k|append   # one other workload alone

Prints ONE JSON line (rank 0).  `value` = algorithmic HBM bytes of the whole sequence per step / device time (max over
ranks) with inputs resident in HBM; `e2e` = the same step through the C ABI with host buffers (H2D of q/k/v, D2H of
the outputs, every step).  On one GPU the line also carries a `blocks` object with the other workloads of the path
(32,768-token decode, 32 batched sequences, verify steps at 131,072 tokens, a 1,024-token prefill chunk over 262,144
tokens, quantise-append alone), each with its time, achieved rate and fraction of the measured peak.
The headline numbers are for caches written with sinkhorn_iters = 0 (the bit-exact regime).
"""
import argparse
import json
import math
import os
import random
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, H, QH, LAYERS = 128, 4, 24, 16
LONG_CTX = 378944
# DRAM bytes (read + write) one decode call moves per token of context, from ncu captures of attn_kernel: 213.92 MB
# read + 4.73 MB written at 378,944 tokens (581.6 B per token at 131,072): the codes and axes the kernel fetches (the
# second page's copy of the per-dim scales is skipped) plus the partials written; traffic grows in proportion to the
# context (same pages per token, same splits per SM).
TRAFFIC_BYTES_PER_TOKEN = 577.0
SEALED_B, TAIL_B = 140, 512  # algorithmic bytes per sealed / open-tile token per KV head (codes + 12 B of axes | fp16 K+V rows)


def decode_bytes(kv_len: int) -> int:
    """Algorithmic bytes one decode call must move: codes and axes of every sealed token, fp16 rows of the
    open tile, q in, out back, one page id per page."""
    sealed = (kv_len // 128) * 128
    return sealed * H * SEALED_B + (kv_len - sealed) * H * TAIL_B + 2 * QH * D * 2 + 4 * ((kv_len + 63) // 64)


def append_bytes(tokens: int) -> int:
    """Rows read (K and V) + the same rows written to the stage."""
    return 2 * tokens * H * D * 2 * 2


def shuffled_table(seed: int, logical_pages: int, physical_pages: int):
    """A seeded page table: logical page -> distinct physical page (the pages of a sequence are scattered)."""
    import numpy as np

    return np.random.default_rng([seed, 99]).permutation(physical_pages)[:logical_pages].astype(np.int32)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 100 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j["hbm_gbs"]), float(j.get("bf16_tflops_sustained", 1388.5)), "measured"
    return 6650.0, 1400.0, "fallback"


def cpu_threads():
    return os.cpu_count() or 1


def long_config(n, layers_n=LAYERS):
    return {"workload": f"decode_ctx{LONG_CTX}_{layers_n}layers_b1: one sequence of {LONG_CTX} tokens (5,921 pages), append 1 token + decode per layer",
            "layers": layers_n, "ctx": LONG_CTX, "q_heads": QH, "kv_heads": H, "head_dim": D, "page_tokens": 64,
            "kv_format": "kvarn128 K4V4 sinkhorn_iters 0 (P1 planes)",
            "parallelism": "single GPU" if n == 1 else f"sp{n}: contiguous tile ranges per rank, open tile and appends on the last rank, "
                                                       "(m, l, o) partials exchanged by peer stores inside reduce_kernel",
            "l2": f"{layers_n} layers x {LONG_CTX * H * 146 / n / 1e6:.0f} MB of KV per rank between revisits (L2: 126 MB); no explicit flush"}


# ------------------------------------------------------------------------------------------------------------
# The CPU arm: the oracle port on the host cores, same sequence, one layer per step.
# ------------------------------------------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import kvarn_oracle as orc

    orc.build()
    threads = cpu_threads()
    total = args.warmup + args.steps
    lp = (LONG_CTX + total + 63) // 64 + 2
    lp += lp & 1
    layer = orc.CpuLayer(D, H, lp, shuffled_table(0, lp, lp))
    k, v = orc.synth_kv(0, LONG_CTX + 1, H, D, 1), orc.synth_kv(0, LONG_CTX + 1, H, D, 2)
    layer.append(k[:LONG_CTX], v[:LONG_CTX], 0)
    q = orc.synth_q(0, 1, QH, D)
    pos = LONG_CTX
    times = []
    for s in range(total):
        t0 = time.perf_counter()
        layer.append(k[LONG_CTX:], v[LONG_CTX:], pos)  # the bench's per-step row, replayed at the next position
        layer.attention(q, [pos], 1.0 / math.sqrt(D), QH, threads=threads)
        dt = time.perf_counter() - t0
        if s >= args.warmup:
            times.append(dt)
        pos += 1
    per_layer = sum(times) / len(times)
    nbytes = decode_bytes(LONG_CTX + 1) + append_bytes(1)
    gbs = nbytes / per_layer / 1e9
    sample = (f"1 of {LAYERS} layers per step (append 1 token + decode at {LONG_CTX} tokens), oracle port in C, {threads} threads; "
              "same seeded K/V/q as layer 0 of the GPU arm")
    print(json.dumps({
        "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_layer * 1e3, "layers_timed": 1, "us_per_layer": per_layer * 1e6,
        "extrapolated_ms_per_step_16_layers": per_layer * LAYERS * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": long_config(args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------------------------------------
class _Env:
    """Device, process group and helpers shared by the workloads."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        import __graft_entry__ as entry

        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
        self.pkg = entry.load_package()
        self.pkg.capi.load()  # fails loudly when the CUDA library is missing: there is no fallback
        self.gen = torch.Generator(device=self.dev)
        self.gen.manual_seed(7 + 1000 * self.rank)
        self.scale = 1.0 / math.sqrt(D)

    def synth(self, tokens, heads):
        x = self.torch.randn((tokens, heads, D), generator=self.gen, device=self.dev, dtype=self.torch.float32)
        x[..., [3, 17, 64, 101]] *= 20.0
        return x.to(self.torch.float16)

    def layer(self, tokens, room, seed, kv=None, iters=0):
        """A layer pre-filled with `tokens` tokens (synthetic, or the given (k, v) host arrays) and room for `room` more."""
        torch = self.torch
        lp = (tokens + room + 63) // 64 + 2
        lp += lp & 1
        L = self.pkg.KvarnLayer(D, H, QH, lp, torch.from_numpy(shuffled_table(seed, lp, lp)), sinkhorn_iters=iters, device=str(self.dev))
        for c0 in range(0, tokens, 8192):
            n = min(8192, tokens - c0)
            if kv is None:
                k, v = self.synth(n, H), self.synth(n, H)
            else:
                k, v = (torch.from_numpy(a[c0:c0 + n]).to(self.dev) for a in kv)
            L.append(k, v, torch.arange(c0, c0 + n, dtype=torch.int32, device=self.dev))
        return L

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, n):
        """ms per call of fn over n calls: CUDA events on the current stream, barrier + synchronize on both sides, max
        over ranks."""
        torch = self.torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        self.barrier()
        ms = e0.elapsed_time(e1)
        if self.world > 1:
            t = torch.tensor([ms], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / n

    def graph(self, body):
        """Capture `body` into a CUDA graph (after one eager run); falls back to eager replay if capture fails."""
        torch = self.torch
        body()
        torch.cuda.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=torch.cuda.Stream(device=self.dev)):
                body()
            torch.cuda.synchronize()
            return g.replay, True
        except Exception:  # noqa: BLE001 -- e.g. a collective that cannot be captured on this stack
            torch.cuda.synchronize()
            return body, False

    def release(self):
        import gc

        gc.collect()
        self.torch.cuda.empty_cache()

    def finish(self, result):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()
        if self.rank == 0:
            print(json.dumps(result))


# ------------------------------------------------------------------------------------------------------------
# The contract workload: one 378,944-token sequence, range-sharded over the ranks.
# ------------------------------------------------------------------------------------------------------------
def measure_long(E, args, layers_n, with_cpu=True):
    import numpy as np

    torch = E.torch
    sh = E.pkg.sharded
    from oracle import kvarn_oracle as orc  # checker + cpu_baseline leg + the seeded inputs both arms share

    steps, warm = args.steps, max(args.warmup, 3)
    total_steps = warm + 3 * steps + 16
    b, e = sh.tile_ranges(LONG_CTX, E.world)[E.rank]
    n = e - b
    owner = E.rank == E.world - 1  # holds the open tile, receives the appends
    room = total_steps + 2 if owner else 2
    # layer 0: the seeded K/V the CPU arm uses (numpy generator, same seed and streams); other layers: device generator
    k0, v0 = orc.synth_kv(0, LONG_CTX + 1, H, D, 1), orc.synth_kv(0, LONG_CTX + 1, H, D, 2)
    layers = [E.layer(n, room, 100 * E.rank + i, kv=(k0[b:e], v0[b:e]) if i == 0 else None) for i in range(layers_n)]
    step_row = np.concatenate([k0[LONG_CTX], v0[LONG_CTX]], axis=0)  # [2H, D]: the row appended every step on layer 0
    del k0, v0
    host_gen = torch.Generator()
    host_gen.manual_seed(12345)  # the same q and per-step rows on every rank
    qkv_h = torch.randn((layers_n, QH + 2 * H, D), generator=host_gen).to(torch.float16)
    qkv_h[:, QH:, [3, 17, 64, 101]] *= 20.0
    qkv_h[0, :QH] = torch.from_numpy(orc.synth_q(0, 1, QH, D)[0])
    qkv_h[0, QH:] = torch.from_numpy(step_row)
    qkv = qkv_h.to(E.dev)
    outs = torch.empty((layers_n, QH, D), dtype=torch.float16, device=E.dev)
    kv_len_max = n + room
    pos = torch.full((1,), n - 1 if not owner else n, dtype=torch.int32, device=E.dev)
    pos_fixed = torch.full((1,), n - 1, dtype=torch.int32, device=E.dev)
    for L in layers:
        L.workspace(kv_len_max, 1)
    ring = sh.PeerRing.symmetric(QH, D, E.dev) if E.world > 1 else None
    rdec = [sh.RingShardedDecode(L, ring) for L in layers] if ring is not None else None
    packed = torch.empty(QH * (D + 2), dtype=torch.float32, device=E.dev)
    torch.cuda.synchronize()

    def decode(i, p):
        if E.world == 1:
            layers[i].attn_decode(qkv[i, :QH], p, E.scale, kv_len_max, out=outs[i])
        else:
            rdec[i].attn_decode(qkv[i, :QH], p, E.scale, kv_len_max, outs[i])

    def step_body():  # per layer: append the new token (owner of the open tile), then decode
        for i, L in enumerate(layers):
            if owner:
                L.append_decode(qkv[i, :QH], qkv[i, QH:QH + H], qkv[i, QH + H:], pos, E.scale, kv_len_max, out=outs[i], ring=ring)
            else:
                decode(i, pos_fixed)
        if owner:
            pos.add_(1)

    def decode_only_body():
        for i in range(layers_n):
            decode(i, pos_fixed)

    def local_only_body():  # the same launches without any exchange: partial export + merge of the rank's own partial
        for i, L in enumerate(layers):
            L.attn_decode_partial_packed(qkv[i, :QH], pos_fixed, E.scale, kv_len_max, packed)
            E.pkg.cache.merge_partials_packed(packed, 1, QH, D, outs[i])

    g_step, graphed = E.graph(step_body)
    g_dec, _ = E.graph(decode_only_body)
    g_local = E.graph(local_only_body)[0] if E.world > 1 else None
    for _ in range(warm):
        g_step()
    with ClockSampler(E.local) as clk:
        ms_step = E.timed(g_step, steps)
        for _ in range(3):
            g_dec()
        ms_dec = E.timed(g_dec, steps)
        ms_local = None
        if g_local is not None:
            for _ in range(3):
                g_local()
            ms_local = E.timed(g_local, steps)
        # end to end: host buffers in, host buffers out, every step
        h_in = qkv_h.pin_memory()
        h_out = torch.empty_like(outs, device="cpu").pin_memory()

        def e2e_step():
            qkv.copy_(h_in, non_blocking=True)
            g_step()
            h_out.copy_(outs, non_blocking=True)

        for _ in range(3):
            e2e_step()
        ms_e2e = E.timed(e2e_step, steps)
    clocks = clk.summary()
    errs = sum(L.errors() for L in layers)

    # ---- parity at full size: every rank's oracle partial over the bytes its GPU holds, merged on rank 0, against the
    #      output of the measured path (layer 0, final position)
    cur = int(pos.item()) if owner else n  # local length now
    decode(0, torch.full((1,), cur - 1, dtype=torch.int32, device=E.dev) if owner else pos_fixed)
    torch.cuda.synchronize()
    got = outs[0].float().cpu().numpy()
    threads = max(1, cpu_threads() // E.world)
    cpu = orc.CpuLayer(D, H, layers[0].pages, layers[0].table.cpu().numpy())
    L0 = layers[0]
    cpu.k_code[:] = L0.k_code.cpu().numpy(); cpu.v_code[:] = L0.v_code.cpu().numpy()
    cpu.k_scale[:] = L0.k_scale.cpu().numpy().view(np.uint16); cpu.v_scale[:] = L0.v_scale.cpu().numpy().view(np.uint16)
    cpu.stage[:] = L0.stage.cpu().numpy().view(np.uint16).reshape(cpu.stage.shape)
    q0 = qkv_h[0, :QH].numpy()[None]
    t_cpu = None
    if E.world == 1:
        best = None
        for _ in range(3 if with_cpu else 1):
            t0 = time.perf_counter()
            want = cpu.attention(q0, [cur - 1], E.scale, QH, threads=threads, kv_total=cur)[0]
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        t_cpu = best
    else:
        _, pm, pl, po = cpu.attention(q0, [cur - 1], E.scale, QH, threads=threads, kv_total=cur, want_partials=True)
        mine = torch.from_numpy(np.concatenate([pm[0][:, None], pl[0][:, None], po[0]], axis=1)).to(E.dev)
        allp = torch.empty((E.world,) + tuple(mine.shape), dtype=mine.dtype, device=E.dev)
        E.dist.all_gather_into_tensor(allp.view(-1, mine.shape[1]), mine)
        a = allp.cpu().numpy()
        want = orc.merge_partials(a[:, :, 0], a[:, :, 1], a[:, :, 2:])
    err = float(np.abs(got - want).max() / np.abs(want).max())
    rel = float(np.sqrt(((got - want) ** 2).sum() / (want.astype(np.float64) ** 2).sum()))

    global_len = LONG_CTX + (cur - n if owner else 0)
    if E.world > 1:
        t = torch.tensor([global_len], device=E.dev)
        E.dist.all_reduce(t, op=E.dist.ReduceOp.MAX)
        global_len = int(t.item())
    peak, _, kind = peaks()
    step_bytes = layers_n * (decode_bytes(global_len) + append_bytes(1))
    local_bytes = decode_bytes(n)  # this rank's range (rank 0 prints)
    us_dec = ms_dec * 1e3 / layers_n
    res = {
        "metric": "decode_attn_hbm_gbs", "value": step_bytes / (ms_step * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": E.world,
        "steps": steps, "warmup": warm, "ms_per_step": ms_step, "us_per_layer": ms_step * 1e3 / layers_n,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": long_config(E.world, layers_n),
        "pct_of_hbm_peak": 100.0 * step_bytes / (ms_step * 1e-3) / 1e9 / (peak * E.world),
        "roofline": {"bound": "hbm", "kernel": "attn_kernel (+ reduce_kernel, timed together: decode-only graph over the layers)",
                     "achieved": local_bytes / (us_dec * 1e-6) / 1e9, "peak": peak, "peak_kind": kind, "unit": "GB/s",
                     "frac": local_bytes / (us_dec * 1e-6) / 1e9 / peak, "traffic": TRAFFIC_BYTES_PER_TOKEN * n,
                     "us_per_launch": us_dec, "algorithmic_bytes_per_launch": local_bytes,
                     "note": "per GPU: bytes of rank 0's tile range / max-over-ranks time" if E.world > 1 else "one GPU, whole sequence"},
        "e2e": {"value": step_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": E.world * qkv.numel() * 2, "d2h_bytes_per_step": E.world * outs.numel() * 2},
        "gpu_launches": steps * layers_n * 3,
        "graph_captured": graphed, "error_words": errs,
        "parity": {"max_abs_over_ref_max": err, "rel_l2": rel,
                   "checked": f"layer 0 decode at {global_len} tokens vs the CPU oracle over the bytes the GPUs hold"
                              + (" (per-rank oracle partials merged on rank 0)" if E.world > 1 else "")},
        "clocks": clocks,
    }
    if E.world > 1:
        us_local = ms_local * 1e3 / layers_n
        res["combine"] = {"us_per_layer_with_exchange": us_dec, "us_per_layer_without_exchange": us_local,
                          "us_per_layer_exchange": max(0.0, us_dec - us_local), "share_of_layer_time": max(0.0, 1.0 - us_local / us_dec),
                          "bytes_per_peer_per_layer": QH * (D + 2) * 8, "how": "peer stores + bounded polling inside reduce_kernel; no collective library on the data path"}
    if t_cpu is not None and with_cpu:
        res["cpu_baseline"] = {"value": decode_bytes(cur) / t_cpu / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                               "sample": f"decode attention of 1 of {layers_n} layers at {cur} tokens, best of 3, oracle port in C"}
    del layers, rdec, ring
    E.release()
    return res


def run_contract(args):
    E = _Env()
    res = measure_long(E, args, args.layers or LAYERS)
    if args.blocks and E.world == 1:
        sub = argparse.Namespace(**vars(args))
        sub.steps, sub.warmup = min(args.steps, 20), 3
        blocks = {}
        for name, fn in (("decode_ctx32768_16layers", measure_decode32k), ("batch32_len16k_131k", measure_batch),
                         ("verify_ctx131072_widths4to8", measure_verify), ("prefill_chunk1024_prefix262144", measure_prefill),
                         ("append_chunk1024", measure_append)):
            try:
                blocks[name] = fn(E, sub)
            except Exception as exc:  # noqa: BLE001 -- a failing extra must not take the contract line down
                blocks[name] = {"failed": repr(exc)[:300]}
            E.release()
        res["blocks"] = blocks
    elif args.blocks:  # the workload that shards without any exchange, at every N: whole sequences dealt to the ranks
        sub = argparse.Namespace(**vars(args))
        sub.steps, sub.warmup = min(args.steps, 20), 3
        try:
            res["blocks"] = {"batch32_len16k_131k": measure_batch(E, sub)}
        except Exception as exc:  # noqa: BLE001
            res["blocks"] = {"batch32_len16k_131k": {"failed": repr(exc)[:300]}}
    E.finish(res)


# ------------------------------------------------------------------------------------------------------------
# The other workloads of the path.  Each returns a dict with us / achieved / frac.
# ------------------------------------------------------------------------------------------------------------
def measure_decode32k(E, args):
    """Batch-1 decode at 32,768 tokens x 16 layers: per layer append 1 token, then decode (one sequence per GPU)."""
    torch = E.torch
    ctx = 32768
    total_steps = max(args.warmup, 3) + 2 * args.steps + 8
    kv_len_max = ctx + total_steps + 1
    layers = [E.layer(ctx, total_steps + 2, 100 * E.rank + i) for i in range(LAYERS)]
    qkv = torch.cat([torch.randn((LAYERS, QH, D), generator=E.gen, device=E.dev).to(torch.float16),
                     E.synth(LAYERS, 2 * H)], dim=1)
    outs = torch.empty((LAYERS, QH, D), dtype=torch.float16, device=E.dev)
    pos = torch.full((1,), ctx, dtype=torch.int32, device=E.dev)
    pos_fixed = torch.full((1,), ctx, dtype=torch.int32, device=E.dev)
    for L in layers:
        L.workspace(kv_len_max, 1)

    def step_body():
        for i, L in enumerate(layers):
            L.append_decode(qkv[i, :QH], qkv[i, QH:QH + H], qkv[i, QH + H:], pos, E.scale, kv_len_max, out=outs[i])
        pos.add_(1)

    def decode_only_body():
        for i, L in enumerate(layers):
            L.attn_decode(qkv[i, :QH], pos_fixed, E.scale, kv_len_max, out=outs[i])

    g_step, _ = E.graph(step_body)
    g_dec, _ = E.graph(decode_only_body)
    for _ in range(max(args.warmup, 3)):
        g_step()
    ms_step = E.timed(g_step, args.steps)
    for _ in range(3):
        g_dec()
    ms_dec = E.timed(g_dec, args.steps)
    peak, _, kind = peaks()
    step_bytes = decode_bytes(ctx + 1) + append_bytes(1)
    us, us_dec = ms_step * 1e3 / LAYERS, ms_dec * 1e3 / LAYERS
    return {"workload": "decode at 32,768 tokens x 16 layers, append 1 token + decode per layer", "us": us,
            "achieved": step_bytes / (us * 1e-6) / 1e9, "unit": "GB/s", "frac": step_bytes / (us * 1e-6) / 1e9 / peak,
            "attention_call_alone": {"us": us_dec, "achieved": decode_bytes(ctx + 1) / (us_dec * 1e-6) / 1e9,
                                     "frac": decode_bytes(ctx + 1) / (us_dec * 1e-6) / 1e9 / peak},
            "peak": peak, "peak_kind": kind, "error_words": sum(L.errors() for L in layers)}


def measure_decode_ctx(E, args):
    """Decode attention alone (no append) at --ctx tokens over --layers layers; the case the ncu captures use."""
    torch = E.torch
    ctx = args.ctx or 131072
    layers_n = args.layers or max(2, min(16, int(400e6 // (ctx * H * 146)) + 1))
    iters = getattr(args, "iters", 0)  # > 0: caches written with that many Sinkhorn iterations (per-key / per-dim factors in the kernel)
    layers = [E.layer(ctx, 8, i, iters=iters) for i in range(layers_n)]
    q = torch.randn((layers_n, QH, D), generator=E.gen, device=E.dev).to(torch.float16)
    pos = torch.full((1,), ctx - 1, dtype=torch.int32, device=E.dev)
    outs = torch.empty((layers_n, QH, D), dtype=torch.float16, device=E.dev)
    for L in layers:
        L.workspace(ctx + 8, 1)

    def step():
        for i, L in enumerate(layers):
            L.attn_decode(q[i], pos, E.scale, ctx + 8, out=outs[i])

    run, graphed = E.graph(step)
    with ClockSampler(E.local) as clk:
        for _ in range(max(args.warmup, 3)):
            run()
        ms = E.timed(run, args.steps)
    peak, _, kind = peaks()
    us = ms * 1e3 / layers_n
    nbytes = decode_bytes(ctx)
    return {
        "metric": "decode_attn_hbm_gbs", "value": nbytes / (us * 1e-6) / 1e9, "unit": "GB/s", "n_gpus": E.world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "us_per_layer": us, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"decode_attention_only_ctx{ctx}" + (f"_sinkhorn{iters}" if iters else ""), "layers": layers_n, "q_heads": QH, "kv_heads": H, "head_dim": D,
                   "l2": f"{layers_n} layers x {ctx * H * 146 / 1e6:.0f} MB between revisits"},
        "roofline": {"bound": "hbm", "achieved": nbytes / (us * 1e-6) / 1e9, "peak": peak, "peak_kind": kind, "unit": "GB/s",
                     "frac": nbytes / (us * 1e-6) / 1e9 / peak, "traffic": TRAFFIC_BYTES_PER_TOKEN * ctx if D == 128 else None},
        "graph_captured": graphed, "clocks": clk.summary(), "gpu_launches": args.steps * layers_n * 2,
        "error_words": sum(L.errors() for L in layers),
    }


def measure_batch(E, args):
    """32 independent sequences, lengths seed-uniform in 16K..131K, dealt to the ranks longest-first; a step = one
    batched decode call (kvb_attn_decode_batch) over the rank's sequences."""
    torch = E.torch
    rnd = random.Random(0)
    lengths = [rnd.randint(16384, 131072) for _ in range(32)]
    mine = E.pkg.sharded.deal_sequences(lengths, E.world)[E.rank]
    seqs = [(E.layer(lengths[i], 8, i), lengths[i]) for i in mine]
    q = torch.randn((len(seqs), QH, D), generator=E.gen, device=E.dev).to(torch.float16)
    outs = torch.empty((len(seqs), QH, D), dtype=torch.float16, device=E.dev)
    batch = E.pkg.DecodeBatch([L for L, _ in seqs], [n + 8 for _, n in seqs])
    pos_all = torch.tensor([n - 1 for _, n in seqs], dtype=torch.int32, device=E.dev)

    def step_batched():
        batch.attn_decode(q, pos_all, E.scale, out=outs)

    run, graphed = E.graph(step_batched)
    with ClockSampler(E.local) as clk:
        for _ in range(max(args.warmup, 3)):
            run()
        ms = E.timed(run, args.steps)
    peak, _, kind = peaks()
    total = sum(decode_bytes(n) for n in lengths)
    gbs = total / (ms * 1e-3) / 1e9
    return {"workload": "one batched decode call over 32 sequences of 16K..131K tokens (2.4 M tokens), sharded by sequence",
            "us": ms * 1e3, "achieved": gbs, "unit": "GB/s", "frac": gbs / (peak * E.world), "peak": peak, "peak_kind": kind,
            "total_tokens": sum(lengths), "n_gpus": E.world, "parallelism": f"dp{E.world} (longest first, no collective)",
            "graph_captured": graphed, "clocks": clk.summary(), "gpu_launches": args.steps * 2,
            "error_words": sum(L.errors() for L, _ in seqs)}


def measure_append(E, args):
    """Quantise-append alone: chunks of --chunk tokens (default 1,024, the prefill chunk) written at the same positions
    every step (a roll-back followed by a re-append), over enough layers that the rows read and the planes written
    exceed L2."""
    torch = E.torch
    T = getattr(args, "chunk", 0) or 1024
    iters = getattr(args, "iters", 0)
    layers_n = max(4, min(64, int(300e6 // (T * H * D * 2 * 2)) + 1))
    lp = (T + 63) // 64 + 2
    lp += lp & 1
    layers = [E.pkg.KvarnLayer(D, H, QH, lp, torch.from_numpy(shuffled_table(i, lp, lp)), sinkhorn_iters=iters, device=str(E.dev))
              for i in range(layers_n)]
    k = [E.synth(T, H) for _ in range(layers_n)]
    v = [E.synth(T, H) for _ in range(layers_n)]
    pos = torch.arange(0, T, dtype=torch.int32, device=E.dev)

    def step():
        for i, L in enumerate(layers):
            L.append(k[i], v[i], pos)

    run, graphed = E.graph(step)
    with ClockSampler(E.local) as clk:
        for _ in range(max(args.warmup, 3)):
            run()
        ms = E.timed(run, args.steps)
    errs = sum(L.errors() for L in layers)
    peak, _, kind = peaks()
    tiles, tail = T // 128, T % 128
    # rows read + planes written for the sealed tiles + stage rows written for the open tail (and, as the reference
    # keeps them for roll-back, for the last sealed tile)
    nbytes = 2 * T * H * D * 2 + tiles * 128 * H * 146 * (D // 128) + (tail + (128 if tiles else 0)) * H * D * 2 * 2
    us = ms * 1e3 / layers_n
    return {"workload": f"quantise-append of {T} tokens per call, sinkhorn_iters {iters}", "us": us, "achieved": nbytes / (us * 1e-6) / 1e9,
            "unit": "GB/s", "frac": nbytes / (us * 1e-6) / 1e9 / peak, "peak": peak, "peak_kind": kind, "bound": "hbm",
            "algorithmic_bytes_per_launch": nbytes, "tokens_per_s": T / (us * 1e-6), "layers": layers_n,
            "graph_captured": graphed, "error_words": errs, "clocks": clk.summary(),
            "gpu_launches": args.steps * layers_n * (2 if T > 128 else 1)}


def measure_verify(E, args):
    """MTP draft-verify at 131,072 tokens: append 1+k rows (k seeded in 3..7), causal attention of those rows; the
    drafts are rolled back after every step, so the context stays at 131,072."""
    torch = E.torch
    ctx, layers_n = 131072, args.layers if getattr(args, "layers", 0) and args.workload == "verify131k" else 4
    layers = [E.layer(ctx, 16, i) for i in range(layers_n)]
    rnd = random.Random(0)
    widths = [1 + rnd.randint(3, 7) for _ in range(16)]
    q = torch.randn((layers_n, 8, QH, D), generator=E.gen, device=E.dev).to(torch.float16)
    kv = [E.synth(8, 2 * H) for _ in range(layers_n)]
    pos = torch.arange(ctx, ctx + 8, dtype=torch.int32, device=E.dev)
    outs = torch.empty((layers_n, 8, QH, D), dtype=torch.float16, device=E.dev)
    for L in layers:
        L.workspace(ctx + 16, 8)
    runs, per_width = {}, {}
    for w in sorted(set(widths)):
        def body(w=w):
            for i, L in enumerate(layers):
                L.attn_verify(q[i, :w], kv[i][:w, :H], kv[i][:w, H:], pos[:w], E.scale, ctx + 16, out=outs[i, :w])
        runs[w] = E.graph(body)[0]
    seq = [runs[w] for w in widths]
    it = {"i": 0}

    def step():
        seq[it["i"] % len(seq)]()
        it["i"] += 1

    with ClockSampler(E.local) as clk:
        for _ in range(max(args.warmup, 3)):
            step()
        it["i"] = 0
        ms = E.timed(step, args.steps)
        for w in sorted(runs):
            for _ in range(2):
                runs[w]()
            per_width[str(w)] = E.timed(runs[w], max(3, args.steps // 4)) * 1e3 / layers_n
    peak, peak_tf, kind = peaks()
    used = [widths[i % len(widths)] for i in range(args.steps)]
    nbytes = decode_bytes(ctx)
    flops = sum(4.0 * QH * w * ctx * D for w in used) / len(used)
    us = ms * 1e3 / layers_n
    return {"workload": "verify steps of 1+k rows (k in 3..7, seeded) over 131,072 tokens: append + causal attention", "us": us,
            "achieved": nbytes / (us * 1e-6) / 1e9, "unit": "GB/s", "frac": nbytes / (us * 1e-6) / 1e9 / peak, "peak": peak, "peak_kind": kind,
            "tflops": flops / (us * 1e-6) / 1e12, "frac_of_tensor_peak": flops / (us * 1e-6) / 1e12 / peak_tf,
            "us_per_layer_by_width": per_width, "widths": used[:16], "layers": layers_n, "clocks": clk.summary(),
            "gpu_launches": args.steps * layers_n * 3, "error_words": sum(L.errors() for L in layers)}


def measure_prefill(E, args):
    """Quantise-append a 1,024-token chunk and run causal chunk attention over a 262,144-token prefix; the chunk is
    rolled back after every step."""
    torch = E.torch
    ctx, chunk = (args.ctx if getattr(args, "ctx", 0) and args.workload == "prefill262k" else 262144), 1024
    L = E.layer(ctx, chunk + 8, 0)
    q = torch.randn((chunk, QH, D), generator=E.gen, device=E.dev).to(torch.float16)
    k, v = E.synth(chunk, H), E.synth(chunk, H)
    pos = torch.arange(ctx, ctx + chunk, dtype=torch.int32, device=E.dev)
    out = torch.empty_like(q)
    L.prefill_workspace(ctx + chunk + 8, chunk)  # allocated before the timed region

    def step():
        L.attn_prefill(q, k, v, pos, E.scale, ctx + chunk + 8, out=out)

    step()
    with ClockSampler(E.local) as clk:
        for _ in range(max(args.warmup, 1)):
            step()
        ms = E.timed(step, args.steps)
    flops = 4.0 * QH * D * (chunk * ctx + chunk * (chunk + 1) / 2)
    tf = flops / (ms * 1e-3) / 1e12
    _, peak_tf, kind = peaks()
    return {"workload": f"prefill chunk of 1,024 tokens over a {ctx}-token quantised prefix: append + causal chunk attention",
            "us": ms * 1e3, "achieved": tf, "unit": "TFLOP/s", "frac": tf / peak_tf, "peak": peak_tf, "peak_kind": kind + " (sustained bf16)",
            "bound": "tensor", "clocks": clk.summary(), "error_words": L.errors()}


def measure_chunk_sharded(E, args):
    """The prefill chunk (1,024 tokens over a 262,144-token prefix) or a verify step (8 rows over 131,072 tokens) over a
    sequence whose tile ranges live on the N ranks: the new rows are appended on the rank that owns the open tile,
    every rank attends its own range (kvb_attn_chunk_partial), one all-gather of the partials, every rank merges."""
    torch = E.torch
    sh = E.pkg.sharded
    prefill = args.workload == "prefill262k"
    ctx, tokens = ((args.ctx or 262144), 1024) if prefill else (131072, 8)
    b, e = sh.tile_ranges(ctx, E.world)[E.rank]
    n = e - b
    owner = E.rank == E.world - 1
    L = E.layer(n, tokens + 8, 100 * E.rank)
    host_gen = torch.Generator()
    host_gen.manual_seed(4321)  # the same q and new rows on every rank
    q = torch.randn((tokens, QH, D), generator=host_gen).to(torch.float16).to(E.dev)
    kv = torch.randn((tokens, 2 * H, D), generator=host_gen)
    kv[..., [3, 17, 64, 101]] *= 20.0
    kv = kv.to(torch.float16).to(E.dev)
    pos = (torch.arange(n, n + tokens, dtype=torch.int32, device=E.dev) if owner
           else torch.full((tokens,), n - 1, dtype=torch.int32, device=E.dev))
    out = torch.empty((tokens, QH, D), dtype=torch.float16, device=E.dev)
    chunk = sh.ShardedChunk(L, tokens)
    ring_dec = None if prefill else sh.RingShardedDecode(L, sh.PeerRing.symmetric(QH, D, E.dev, tokens=8))
    kv_len_max = n + tokens + 8
    if tokens > 8:
        L.prefill_workspace(kv_len_max, tokens)
    else:
        L.workspace(kv_len_max, tokens)

    def step():  # the drafts / the chunk are rolled back after every step: the same rows are appended at the same positions
        if ring_dec is not None:  # verify step: partials exchanged over peer memory inside the reduce kernel
            ring_dec.attn_verify(q, kv[:, :H], kv[:, H:], pos, E.scale, kv_len_max, out, owner=owner)
        else:
            chunk.attend(q, kv[:, :H], kv[:, H:], pos, E.scale, kv_len_max, out)

    def step_nccl():
        chunk.attend(q, kv[:, :H], kv[:, H:], pos, E.scale, kv_len_max, out)

    def step_local():  # without the collective: append + partial only
        if owner:
            L.append(kv[:, :H], kv[:, H:], pos)
        L.attn_chunk_partial_packed(q, pos, E.scale, kv_len_max, chunk.send[:tokens * chunk.per_token])

    step()
    with ClockSampler(E.local) as clk:
        for _ in range(max(args.warmup, 3)):
            step()
        ms = E.timed(step, args.steps)
        for _ in range(3):
            step_local()
        ms_local = E.timed(step_local, args.steps)
        ms_nccl = None
        if ring_dec is not None:
            for _ in range(3):
                step_nccl()
            ms_nccl = E.timed(step_nccl, args.steps)
    peak, peak_tf, kind = peaks()
    flops = 4.0 * QH * D * (tokens * ctx + tokens * (tokens + 1) / 2)
    tf = flops / (ms * 1e-3) / 1e12
    nbytes = decode_bytes(ctx)
    res = {"workload": (f"prefill chunk of 1,024 tokens over a {ctx}-token prefix" if prefill else "verify step of 8 rows over 131,072 tokens")
                       + f", tile ranges on {E.world} GPUs: append on the owner, per-rank partials, "
                       + ("one all-gather, merge" if prefill else "exchange over peer memory inside the merge kernel"),
           "us": ms * 1e3, "us_without_collective": ms_local * 1e3, "collective_share": max(0.0, 1.0 - ms_local / ms),
           "bytes_gathered_per_rank": tokens * QH * (D + 2) * 4, "n_gpus": E.world, "clocks": clk.summary(), "error_words": L.errors()}
    if ms_nccl is not None:
        res["exchange"] = "peer stores + bounded polling inside reduce_kernel (kvb_attn_rows_sharded)"
        res["us_with_nccl_all_gather_instead"] = ms_nccl * 1e3
    if prefill:
        res.update({"achieved": tf, "unit": "TFLOP/s", "frac": tf / (peak_tf * E.world), "peak": peak_tf, "peak_kind": kind + " (sustained bf16, per GPU)", "bound": "tensor"})
    else:
        gbs = nbytes / (ms * 1e-3) / 1e9
        res.update({"achieved": gbs, "unit": "GB/s", "frac": gbs / (peak * E.world), "peak": peak, "peak_kind": kind, "bound": "hbm"})
    return res


def run_single(args, fn, metric, unit):
    """One of the other workloads alone, printed in the contract's line format."""
    E = _Env()
    if E.world > 1 and args.workload in ("prefill262k", "verify131k"):
        fn = measure_chunk_sharded
    r = fn(E, args)
    if "metric" not in r:
        r = {"metric": metric, "value": r["achieved"], "unit": unit, "n_gpus": E.world, "steps": args.steps, "warmup": max(args.warmup, 3),
             "ms_per_step": r["us"] * 1e-3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
             "data": "synthetic", "config": {"workload": r["workload"], "q_heads": QH, "kv_heads": H, "head_dim": D},
             "roofline": {"bound": r.get("bound", "hbm"), "achieved": r["achieved"], "peak": r["peak"], "peak_kind": r["peak_kind"],
                          "unit": unit, "frac": r["frac"], "traffic": None}, **{k: v for k, v in r.items() if k not in ("workload",)}}
    E.finish(r)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="long379k",
                    choices=["long379k", "decode32k", "decodectx", "batch32", "verify131k", "prefill262k", "append"],
                    help="long379k is the contract line; the others run one other workload of the path alone")
    ap.add_argument("--layers", type=int, default=0, help="layers held (long379k: 16; decodectx: sized to exceed L2; verify131k: 4)")
    ap.add_argument("--no-blocks", dest="blocks", action="store_false", help="long379k on one GPU: skip the other workloads' blocks")
    ap.add_argument("--chunk", type=int, default=0, help="append: tokens per append call (default 1024)")
    ap.add_argument("--iters", type=int, default=0, help="append, decodectx: Sinkhorn iterations of the encoder (0 = bit-exact regime, 16 = engine default)")
    ap.add_argument("--head-dim", type=int, default=128, choices=[128, 256],
                    help="decodectx / append: 256 is the reference engine's own geometry")
    ap.add_argument("--ctx", type=int, default=0, help="context for decodectx (default 131072) / prefix length for prefill262k (default 262144)")
    args = ap.parse_args()
    if args.head_dim != 128:
        if args.workload not in ("decodectx", "append") or args.impl != "b200":
            ap.error("--head-dim 256 is for --workload decodectx / append")
        global D, SEALED_B, TAIL_B
        D, SEALED_B, TAIL_B = 256, 280, 1024
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "long379k":
        run_contract(args)
    else:
        fn, metric, unit = {"decode32k": (measure_decode32k, "decode_attn_hbm_gbs", "GB/s"),
                            "decodectx": (measure_decode_ctx, "decode_attn_hbm_gbs", "GB/s"),
                            "batch32": (measure_batch, "decode_attn_hbm_gbs", "GB/s"),
                            "verify131k": (measure_verify, "verify_attn_hbm_gbs", "GB/s"),
                            "prefill262k": (measure_prefill, "prefill_chunk_tflops", "TFLOP/s"),
                            "append": (measure_append, "append_hbm_gbs", "GB/s")}[args.workload]
        run_single(args, fn, metric, unit)


if __name__ == "__main__":
    main()
