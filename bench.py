#!/usr/bin/env python3
"""Benchmark of the KVarN quantized-KV decode hot path on B200.

Workload at every N (one process per GPU, no data-path collective, weak scaling): batch-1 decode at a
32,768-token context across 16 attention layers, 24 query heads / 4 KV heads / head_dim 128, seed-shuffled
page table of 64-token pages per layer.  One step = for each layer: append 1 new token (rotate + stage,
sealing a tile every 128 steps), then one decode query over the whole cache.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # the CPU path (oracle port) on the host cores

Prints ONE JSON line (rank 0).  `value` = algorithmic HBM bytes per step / device time with inputs resident
in HBM; `e2e` = the same through the C ABI with host buffers (H2D of q/k/v, D2H of the outputs, per step).
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, H, QH, LAYERS, CTX = 128, 4, 24, 16, 32768
TRAFFIC_BYTES_PER_TOKEN = 602.3
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
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def cpu_threads():
    return os.cpu_count() or 1


def cpu_decode_sample(cpu_layer, q16, pos, threads, reps):
    """Times the oracle port's decode attention (one layer at the bench context) on the host cores."""
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        out = cpu_layer.attention(q16, [pos], 1.0 / math.sqrt(D), QH, threads=threads)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best, out


def run_reference(args):
    """The CPU path: oracle port of append + decode attention, all host threads, one layer per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import kvarn_oracle as orc

    orc.build()
    threads = cpu_threads()
    lp = CTX // 64 + 4
    table = orc.shuffled_table(0, lp, lp + 2)
    layer = orc.CpuLayer(D, H, lp + 2, table)
    k, v = orc.synth_kv(0, CTX + 64, H, D, 1), orc.synth_kv(0, CTX + 64, H, D, 2)
    layer.append(k[:CTX], v[:CTX], 0)
    q = orc.synth_q(0, 1, QH, D)
    pos = CTX
    times = []
    for s in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        layer.append(k[pos:pos + 1], v[pos:pos + 1], pos)
        layer.attention(q, [pos], 1.0 / math.sqrt(D), QH, threads=threads)
        dt = time.perf_counter() - t0
        if s >= args.warmup:
            times.append(dt)
        pos += 1
    per_layer = sum(times) / len(times)
    nbytes = decode_bytes(CTX + 1) + append_bytes(1)
    gbs = nbytes / per_layer / 1e9
    sample = f"1 of {LAYERS} layers per step (append 1 token + decode at {CTX}), oracle port, {threads} threads"
    print(json.dumps({
        "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_layer * LAYERS * 1e3, "us_per_layer": per_layer * 1e6,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": config_dict(args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def config_dict(n):
    return {"workload": "decode_ctx32768_16layers_b1 (BASELINE config 1), one sequence per GPU", "layers": LAYERS, "ctx": CTX,
            "q_heads": QH, "kv_heads": H, "head_dim": D, "page_tokens": 64, "kv_format": "kvarn128 K4V4 iters0 (P1 planes)",
            "parallelism": f"dp{n} (sequences sharded, no collective)",
            "l2": "16 layers x 19 MB of KV per step exceed the 126 MB L2; no explicit flush"}


def run_gpu(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    pkg = entry.load_package()
    pkg.capi.load()  # fails loudly when the CUDA library is missing: there is no fallback
    from oracle import kvarn_oracle as orc  # checker + cpu_baseline leg only

    scale = 1.0 / math.sqrt(D)
    total_steps = args.warmup + 3 * args.steps + 8
    kv_len_max = CTX + total_steps + 1
    lp = (kv_len_max + 63) // 64 + 2
    lp += lp & 1
    gen = torch.Generator(device=dev)
    gen.manual_seed(1000 * rank)

    def synth(tokens, heads):
        x = torch.randn((tokens, heads, D), generator=gen, device=dev, dtype=torch.float32)
        x[..., [3, 17, 64, 101]] *= 20.0
        return x.to(torch.float16)

    layers = []
    for li in range(LAYERS):
        table = torch.from_numpy(shuffled_table(100 * rank + li, lp, lp))
        L = pkg.KvarnLayer(D, H, QH, lp, table, device=str(dev))
        for c0 in range(0, CTX, 4096):  # prefill by appends
            L.append(synth(4096, H), synth(4096, H), torch.arange(c0, c0 + 4096, dtype=torch.int32, device=dev))
        layers.append(L)
    # per-step inputs (resident): one q/k/v set per layer, replayed every step; only the position advances
    qkv = torch.empty((LAYERS, QH + 2 * H, D), dtype=torch.float16, device=dev)
    qkv[:, :QH] = torch.randn((LAYERS, QH, D), generator=gen, device=dev).to(torch.float16)
    qkv[:, QH:] = synth(LAYERS, 2 * H)
    outs = torch.empty((LAYERS, QH, D), dtype=torch.float16, device=dev)
    pos = torch.full((1,), CTX, dtype=torch.int32, device=dev)
    for L in layers:
        L.workspace(kv_len_max, 1)
    torch.cuda.synchronize()

    def step_body():
        for li, L in enumerate(layers):
            L.append(qkv[li, QH:QH + H].unsqueeze(0), qkv[li, QH + H:].unsqueeze(0), pos)
            L.attn_decode(qkv[li, :QH], pos, scale, kv_len_max, out=outs[li])
        pos.add_(1)

    def decode_only_body():
        for li, L in enumerate(layers):
            L.attn_decode(qkv[li, :QH], pos_fixed, scale, kv_len_max, out=outs[li])

    step_body()  # warm every kernel once outside capture (function attributes are set on first use)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=dev)
    g_step, g_dec = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_step, stream=side):
        step_body()
    pos_fixed = torch.full((1,), CTX, dtype=torch.int32, device=dev)
    with torch.cuda.graph(g_dec, stream=side):
        decode_only_body()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        g_step.replay()
    with ClockSampler(local) as clk:
        ms_step = timed(g_step.replay, args.steps) / args.steps
        # decode-only graph: the dominant kernel in isolation (16 layers x 19 MB > L2 between revisits)
        for _ in range(3):
            g_dec.replay()
        ms_dec = timed(g_dec.replay, args.steps) / args.steps
        # end to end: host buffers in, host buffers out, every step
        h_in = torch.empty_like(qkv, device="cpu").pin_memory()
        h_in.copy_(qkv)
        h_out = torch.empty_like(outs, device="cpu").pin_memory()

        def e2e_step():
            qkv.copy_(h_in, non_blocking=True)
            g_step.replay()
            h_out.copy_(outs, non_blocking=True)

        for _ in range(3):
            e2e_step()
        ms_e2e = timed(e2e_step, args.steps) / args.steps
    clocks = clk.summary()

    cur = int(pos.item())  # context after all steps
    step_bytes = LAYERS * (decode_bytes(cur) + append_bytes(1))
    dec_bytes = decode_bytes(CTX + 1)
    peak, peak_kind = peaks()
    value = world * step_bytes / (ms_step * 1e-3) / 1e9
    e2e = world * step_bytes / (ms_e2e * 1e-3) / 1e9
    achieved = dec_bytes / (ms_dec * 1e-3 / LAYERS) / 1e9

    result = None
    if rank == 0:
        # parity at full size + CPU baseline on a bounded sample: one layer's decode on the host cores
        L0 = layers[0]
        cpu = orc.CpuLayer(D, H, lp, L0.table.cpu().numpy())
        cpu.k_code[:] = L0.k_code.cpu().numpy(); cpu.v_code[:] = L0.v_code.cpu().numpy()
        cpu.k_scale[:] = L0.k_scale.cpu().numpy().view(np.uint16); cpu.v_scale[:] = L0.v_scale.cpu().numpy().view(np.uint16)
        cpu.stage[:] = L0.stage.cpu().numpy().view(np.uint16).reshape(cpu.stage.shape)
        cpu.kv_total = cur
        pos_chk = torch.full((1,), cur - 1, dtype=torch.int32, device=dev)
        got = L0.attn_decode(qkv[0, :QH], pos_chk, scale, kv_len_max).float().cpu().numpy()
        threads = cpu_threads()
        t_cpu, want = cpu_decode_sample(cpu, qkv[0, :QH].cpu().numpy(), cur - 1, threads, reps=3)
        err = float(np.abs(got - want[0]).max() / np.abs(want).max())
        result = {
            "metric": "decode_attn_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "us_per_layer": ms_step * 1e3 / LAYERS,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": config_dict(world),
            "pct_of_hbm_peak": 100.0 * value / world / peak,
            "roofline": {"bound": "hbm", "kernel": "attn_kernel (+ reduce_kernel, timed together)", "achieved": achieved,
                         "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "us_per_launch": ms_dec * 1e3 / LAYERS, "algorithmic_bytes_per_launch": dec_bytes},
            "cpu_baseline": {"value": decode_bytes(cur) / t_cpu / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                             "sample": f"decode attention of 1 of {LAYERS} layers at {cur} tokens, best of 3, oracle port"},
            "e2e": {"value": e2e, "unit": "GB/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": world * qkv.numel() * 2,
                    "d2h_bytes_per_step": world * outs.numel() * 2},
            "gpu_launches": args.steps * LAYERS * 3,
            "parity": {"max_abs_over_ref_max": err, "checked": f"layer 0 decode at {cur} tokens vs CPU oracle"},
            "clocks": clocks,
        }
        # DRAM bytes per launch: one ncu capture at 131,072 tokens (profiles/attn_kernel_decode_ctx131072.md),
        # 596.7 B per token of context, scaled to this context (traffic grows in proportion to it)
        result["roofline"]["traffic"] = TRAFFIC_BYTES_PER_TOKEN * (CTX + 1)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(result))


# ------------------------------------------------------------------------------------------------------------
# Other workloads of BASELINE.json (not the contract line): selected with --workload.
# ------------------------------------------------------------------------------------------------------------
class _Env:
    """Device, process group and helpers shared by the extra workloads."""

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
        self.pkg.capi.load()
        self.gen = torch.Generator(device=self.dev)
        self.gen.manual_seed(7 + 1000 * self.rank)
        self.scale = 1.0 / math.sqrt(D)

    def synth(self, tokens, heads):
        x = self.torch.randn((tokens, heads, D), generator=self.gen, device=self.dev, dtype=self.torch.float32)
        x[..., [3, 17, 64, 101]] *= 20.0
        return x.to(self.torch.float16)

    def layer(self, tokens, room, seed):
        """A layer pre-filled with `tokens` synthetic tokens and room for `room` more."""
        torch = self.torch
        lp = (tokens + room + 63) // 64 + 2
        lp += lp & 1
        L = self.pkg.KvarnLayer(D, H, QH, lp, torch.from_numpy(shuffled_table(seed, lp, lp)), device=str(self.dev))
        for c0 in range(0, tokens, 8192):
            n = min(8192, tokens - c0)
            L.append(self.synth(n, H), self.synth(n, H), torch.arange(c0, c0 + n, dtype=torch.int32, device=self.dev))
        return L

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, n):
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

    def finish(self, result):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()
        if self.rank == 0:
            print(json.dumps(result))


def run_long(args):
    """BASELINE config 4A: one 378,944-token sequence, batch-1 decode, range-sharded over the ranks; per layer each
    rank attends its tile range, one all-gather of (m, l, o) partials, every rank merges."""
    E = _Env()
    torch = E.torch
    sh = E.pkg.sharded
    ctx, layers_n = 378944, args.layers or 4
    b, e = sh.tile_ranges(ctx, E.world)[E.rank]
    n = e - b
    layers = [E.layer(n, 8, 100 * E.rank + i) for i in range(layers_n)]
    q = torch.randn((layers_n, QH, D), generator=E.gen, device=E.dev).to(torch.float16)
    if E.world > 1:
        E.dist.broadcast(q, 0)
    pos = torch.full((1,), n - 1, dtype=torch.int32, device=E.dev)
    outs = torch.empty((layers_n, QH, D), dtype=torch.float16, device=E.dev)
    for L in layers:
        L.workspace(n + 8, 1)
    dec = [sh.ShardedDecode(L) for L in layers] if E.world > 1 else []

    def step():
        for i, L in enumerate(layers):
            if E.world == 1:
                L.attn_decode(q[i], pos, E.scale, n + 8, out=outs[i])
            else:
                dec[i].attn_decode(q[i], pos, E.scale, n + 8, outs[i])

    packed = torch.empty(QH * (D + 2), dtype=torch.float32, device=E.dev)

    def step_local():  # the same without the collective: partial + merge of the rank's own partial
        for i, L in enumerate(layers):
            L.attn_decode_partial_packed(q[i], pos, E.scale, n + 8, packed)
            E.pkg.cache.merge_partials_packed(packed, 1, QH, D, outs[i])

    ring_info = None
    if E.world == 1:
        run, graphed = E.graph(step)
        with ClockSampler(E.local) as clk:
            for _ in range(max(args.warmup, 3)):
                run()
            ms = E.timed(run, args.steps)
            run_l, _ = E.graph(step_local)
            for _ in range(3):
                run_l()
            ms_local = E.timed(run_l, args.steps)
    else:
        # (1) NCCL all-gather between the partial and the merge kernel, launched eagerly (a captured collective
        #     stalled a 2-rank run here); (2) the library's own exchange: peer stores + arrival flags, no collective
        #     library on the data path, whole step captured in one CUDA graph.
        graphed = False
        with ClockSampler(E.local) as clk:
            for _ in range(max(args.warmup, 3)):
                step()
            ms_nccl = E.timed(step, args.steps)
            ref = outs.clone()
            for _ in range(3):
                step_local()
            ms_local = E.timed(step_local, args.steps)
            ms = ms_nccl
            try:
                ring = sh.PeerRing.symmetric(QH, D, E.dev)
                rdec = [sh.RingShardedDecode(L, ring) for L in layers]

                def step_ring():
                    for i in range(layers_n):
                        rdec[i].attn_decode(q[i], pos, E.scale, n + 8, outs[i])

                step_ring()
                torch.cuda.synchronize()
                diff = float((outs.float() - ref.float()).abs().max())
                run_r, graphed = E.graph(step_ring)
                for _ in range(max(args.warmup, 3)):
                    run_r()
                ms_ring = E.timed(run_r, args.steps)
                run_lg, _ = E.graph(step_local)  # the same launches without any exchange, also graph-replayed
                for _ in range(3):
                    run_lg()
                ms_local_g = E.timed(run_lg, args.steps)
                errs = sum(L.errors() for L in layers)
                ring_info = {"us_per_layer": ms_ring * 1e3 / layers_n, "max_abs_diff_vs_nccl_path": diff, "graph_captured": graphed,
                             "error_words": errs, "us_per_layer_nccl_eager": ms_nccl * 1e3 / layers_n,
                             "us_per_layer_no_exchange_graph": ms_local_g * 1e3 / layers_n,
                             "exchange_share_of_layer_time": max(0.0, 1.0 - ms_local_g / ms_ring)}
                if errs == 0 and diff < 1e-2:
                    ms, ms_local = ms_ring, ms_local_g
            except Exception as exc:  # noqa: BLE001 -- symmetric memory unavailable: keep the NCCL numbers, say why
                ring_info = {"unavailable": repr(exc)[:200]}
    peak, kind = peaks()
    nbytes = decode_bytes(ctx)
    us_layer = ms * 1e3 / layers_n
    E.finish({
        "metric": "decode_attn_hbm_gbs", "value": nbytes / (us_layer * 1e-6) / 1e9, "unit": "GB/s", "n_gpus": E.world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "us_per_layer": us_layer,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "decode_ctx378944_b1 (BASELINE config 4A), context range-sharded by tiles", "layers": layers_n,
                   "ctx": ctx, "q_heads": QH, "kv_heads": H, "head_dim": D, "parallelism": f"sp{E.world} (tile ranges; partials exchanged by peer stores over NVLink, NCCL all-gather as the baseline)",
                   "l2": f"{layers_n} layers x {n * H * 146 / 1e6:.0f} MB per rank between revisits"},
        "pct_of_hbm_peak": 100.0 * nbytes / (us_layer * 1e-6) / 1e9 / (peak * E.world), "peak_kind": kind,
        "combine": {"us_per_layer_with_gather": us_layer, "us_per_layer_partial_and_merge_only": ms_local * 1e3 / layers_n,
                    "share_of_layer_time": max(0.0, 1.0 - ms_local / ms) if E.world > 1 else 0.0, "graph_captured": graphed,
                    "bytes_per_rank_per_layer": QH * (D + 2) * 4, "peer_ring": ring_info},
        "clocks": clk.summary(), "gpu_launches": args.steps * layers_n * (2 if E.world == 1 else 3),
    })


def run_decode_ctx(args):
    """Decode attention alone (no append) at --ctx tokens over --layers layers; the case the ncu captures use."""
    E = _Env()
    torch = E.torch
    ctx = args.ctx or 131072
    layers_n = args.layers or max(2, min(16, int(400e6 // (ctx * H * 146)) + 1))
    layers = [E.layer(ctx, 8, i) for i in range(layers_n)]
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
    peak, kind = peaks()
    us = ms * 1e3 / layers_n
    nbytes = decode_bytes(ctx)
    E.finish({
        "metric": "decode_attn_hbm_gbs", "value": nbytes / (us * 1e-6) / 1e9, "unit": "GB/s", "n_gpus": E.world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "us_per_layer": us, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"decode_attention_only_ctx{ctx}", "layers": layers_n, "q_heads": QH, "kv_heads": H, "head_dim": D,
                   "l2": f"{layers_n} layers x {ctx * H * 146 / 1e6:.0f} MB between revisits"},
        "roofline": {"bound": "hbm", "achieved": nbytes / (us * 1e-6) / 1e9, "peak": peak, "peak_kind": kind, "unit": "GB/s",
                     "frac": nbytes / (us * 1e-6) / 1e9 / peak, "traffic": TRAFFIC_BYTES_PER_TOKEN * ctx if D == 128 else None},
        "graph_captured": graphed, "clocks": clk.summary(), "gpu_launches": args.steps * layers_n * 2,
    })


def run_batch(args):
    """BASELINE config 4B: 32 independent sequences, lengths seed-uniform in 16K..131K, sharded by sequence; one
    layer per sequence, a step = one decode call per local sequence."""
    import random

    E = _Env()
    torch = E.torch
    rnd = random.Random(0)
    lengths = [rnd.randint(16384, 131072) for _ in range(32)]
    mine = E.pkg.sharded.deal_sequences(lengths, E.world)[E.rank]
    seqs = [(E.layer(lengths[i], 8, i), lengths[i]) for i in mine]
    q = torch.randn((len(seqs), QH, D), generator=E.gen, device=E.dev).to(torch.float16)
    poss = [torch.full((1,), n - 1, dtype=torch.int32, device=E.dev) for _, n in seqs]
    outs = torch.empty((len(seqs), QH, D), dtype=torch.float16, device=E.dev)
    for L, n in seqs:
        L.workspace(n + 8, 1)

    def step_serial():
        for i, (L, n) in enumerate(seqs):
            L.attn_decode(q[i], poss[i], E.scale, n + 8, out=outs[i])

    # The sequences are independent: dealt over a few streams (longest first) the fixed part of one call -- first
    # requests, merge, the reduce kernel -- runs under the page streaming of the others.  Inside the captured graph
    # the streams become parallel branches.
    n_streams = max(1, min(args.streams or 8, len(seqs)))
    side = [torch.cuda.Stream(device=E.dev) for _ in range(n_streams)]
    lanes = E.pkg.sharded.deal_sequences([n for _, n in seqs], n_streams)

    def step_streams():
        cur = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(cur)
        for st, lane in zip(side, lanes):
            st.wait_event(fork)
            with torch.cuda.stream(st):
                for i in lane:
                    L, n = seqs[i]
                    L.attn_decode(q[i], poss[i], E.scale, n + 8, out=outs[i])
            join = torch.cuda.Event()
            join.record(st)
            cur.wait_event(join)

    # One batched call for all local sequences (kvb_attn_decode_batch): one grid whose CTAs are cut in proportion
    # to the sequence lengths, one reduce launch.  This is the measured path; the per-sequence variants are reported
    # beside it.
    batch = E.pkg.DecodeBatch([L for L, _ in seqs], [n + 8 for _, n in seqs])
    pos_all = torch.tensor([n - 1 for _, n in seqs], dtype=torch.int32, device=E.dev)

    def step_batched():
        batch.attn_decode(q, pos_all, E.scale, out=outs)

    run1, graphed1 = E.graph(step_serial)
    for _ in range(3):
        run1()
    ms_serial = E.timed(run1, max(3, args.steps // 2))
    ref = outs.clone()
    run2, _ = E.graph(step_streams)
    for _ in range(3):
        run2()
    ms_streams = E.timed(run2, max(3, args.steps // 2))
    same_streams = bool(torch.equal(ref, outs))
    outs.zero_()
    run, graphed = E.graph(step_batched)
    with ClockSampler(E.local) as clk:
        for _ in range(max(args.warmup, 3)):
            run()
        ms = E.timed(run, args.steps)
    same = float((ref.float() - outs.float()).abs().max().item() / ref.float().abs().max().item())
    peak, kind = peaks()
    total = sum(decode_bytes(n) for n in lengths)
    E.finish({
        "metric": "decode_attn_hbm_gbs", "value": total / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": E.world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": "decode_batch32_len16k-131k (BASELINE config 4B), sharded by sequence", "sequences": 32,
                   "total_tokens": sum(lengths), "q_heads": QH, "kv_heads": H, "head_dim": D, "parallelism": f"dp{E.world} (LPT by length, no collective)",
                   "l2": f"{total / 1e9:.2f} GB of KV per step"},
        "pct_of_hbm_peak": 100.0 * total / (ms * 1e-3) / 1e9 / (peak * E.world), "peak_kind": kind, "graph_captured": graphed,
        "call": "kvb_attn_decode_batch (one call per step)", "max_abs_diff_vs_one_call_per_sequence_over_max": same,
        "one_call_per_sequence": {"ms_per_step_one_stream": ms_serial, "ms_per_step_streams": ms_streams, "streams": n_streams,
                                  "same_output": same_streams},
        "clocks": clk.summary(), "gpu_launches": args.steps * 2,
    })


def run_append(args):
    """Quantise-append alone: chunks of --chunk tokens (default 1,024, the prefill chunk; 4,096 = BASELINE config 0)
    written at the same positions every step (a roll-back followed by a re-append), over enough layers that the
    rows read and the planes written exceed L2."""
    E = _Env()
    torch = E.torch
    T = args.chunk or 1024
    layers_n = args.layers or max(4, min(64, int(300e6 // (T * H * D * 2 * 2)) + 1))
    lp = (T + 63) // 64 + 2
    lp += lp & 1
    layers = [E.pkg.KvarnLayer(D, H, QH, lp, torch.from_numpy(shuffled_table(i, lp, lp)), sinkhorn_iters=args.iters, device=str(E.dev))
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
    peak, kind = peaks()
    tiles, tail = T // 128, T % 128
    # rows read + planes written for the sealed tiles + stage rows written for the open tail (and, as the reference
    # keeps them for roll-back, for the last sealed tile)
    nbytes = 2 * T * H * D * 2 + tiles * 128 * H * 146 * (D // 128) + (tail + (128 if tiles else 0)) * H * D * 2 * 2
    us = ms * 1e3 / layers_n
    E.finish({
        "metric": "append_hbm_gbs", "value": nbytes / (us * 1e-6) / 1e9, "unit": "GB/s", "n_gpus": E.world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "us_per_layer": us, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"append_chunk{T}_iters{args.iters}", "layers": layers_n, "kv_heads": H, "head_dim": D,
                   "l2": f"{layers_n} layers x {nbytes / 1e6:.1f} MB between revisits"},
        "roofline": {"bound": "hbm", "achieved": nbytes / (us * 1e-6) / 1e9, "peak": peak, "peak_kind": kind, "unit": "GB/s",
                     "frac": nbytes / (us * 1e-6) / 1e9 / peak, "traffic": None, "algorithmic_bytes_per_launch": nbytes},
        "tokens_per_s": T / (us * 1e-6), "graph_captured": graphed, "error_words": errs, "clocks": clk.summary(),
        "gpu_launches": args.steps * layers_n * (2 if T > 128 else 1),
    })


def run_verify(args):
    """BASELINE config 2: MTP draft-verify at 131,072 tokens: append 1+k rows (k seeded in 3..7), causal attention of
    those rows; the drafts are rolled back after every step, so the context stays at 131,072."""
    import random

    E = _Env()
    torch = E.torch
    ctx, layers_n = 131072, args.layers or 4
    layers = [E.layer(ctx, 16, i) for i in range(layers_n)]
    rnd = random.Random(0)
    widths = [1 + rnd.randint(3, 7) for _ in range(16)]
    q = torch.randn((layers_n, 8, QH, D), generator=E.gen, device=E.dev).to(torch.float16)
    kv = [E.synth(8, 2 * H) for _ in range(layers_n)]
    pos = torch.arange(ctx, ctx + 8, dtype=torch.int32, device=E.dev)
    outs = torch.empty((layers_n, 8, QH, D), dtype=torch.float16, device=E.dev)
    for L in layers:
        L.workspace(ctx + 16, 8)
    runs = {}
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
    peak, kind = peaks()
    used = [widths[i % len(widths)] for i in range(args.steps)]
    nbytes = decode_bytes(ctx)
    flops = sum(4.0 * QH * w * ctx * D for w in used) / len(used)
    us_layer = ms * 1e3 / layers_n
    E.finish({
        "metric": "verify_attn_hbm_gbs", "value": nbytes / (us_layer * 1e-6) / 1e9, "unit": "GB/s", "n_gpus": E.world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "us_per_layer": us_layer, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "mtp_verify_ctx131072 (BASELINE config 2)", "layers": layers_n, "widths": used[:16], "q_heads": QH,
                   "kv_heads": H, "head_dim": D, "l2": f"{layers_n} layers x 77 MB between revisits"},
        "pct_of_hbm_peak": 100.0 * nbytes / (us_layer * 1e-6) / 1e9 / peak, "peak_kind": kind,
        "tflops": flops / (us_layer * 1e-6) / 1e12, "clocks": clk.summary(), "gpu_launches": args.steps * layers_n * 3,
    })


def run_prefill(args):
    """BASELINE config 3: quantise-append a 1,024-token chunk and run causal chunk attention over a 262,144-token
    prefix; the chunk is rolled back after every step."""
    E = _Env()
    torch = E.torch
    ctx, chunk = args.ctx or 262144, 1024
    L = E.layer(ctx, chunk + 8, 0)
    q = torch.randn((chunk, QH, D), generator=E.gen, device=E.dev).to(torch.float16)
    k, v = E.synth(chunk, H), E.synth(chunk, H)
    pos = torch.arange(ctx, ctx + chunk, dtype=torch.int32, device=E.dev)
    out = torch.empty_like(q)

    def step():
        L.attn_prefill(q, k, v, pos, E.scale, ctx + chunk + 8, out=out)

    step()
    with ClockSampler(E.local) as clk:
        for _ in range(max(args.warmup, 1)):
            step()
        ms = E.timed(step, args.steps)
    flops = 4.0 * QH * D * (chunk * ctx + chunk * (chunk + 1) / 2)
    tf = flops / (ms * 1e-3) / 1e12
    peak_tf = 1388.5
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak_tf = float(json.load(open(p))["bf16_tflops_sustained"])
    E.finish({
        "metric": "prefill_chunk_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": E.world, "steps": args.steps,
        "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"prefill_chunk1024_prefix{ctx} (BASELINE config 3)", "layers": 1, "q_heads": QH, "kv_heads": H, "head_dim": D},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": tf / peak_tf, "traffic": None},
        "clocks": clk.summary(),
    })


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode32k",
                    choices=["decode32k", "decodectx", "long379k", "batch32", "verify131k", "prefill262k", "append"],
                    help="decode32k is the contract line; the others are BASELINE configs 4A, 4B, 2 and 3")
    ap.add_argument("--layers", type=int, default=0, help="layers held for long379k / verify131k (default 4)")
    ap.add_argument("--streams", type=int, default=0, help="batch32: streams the independent sequences are dealt over (default 8)")
    ap.add_argument("--chunk", type=int, default=0, help="append: tokens per append call (default 1024)")
    ap.add_argument("--iters", type=int, default=0, help="append: Sinkhorn iterations of the encoder (0 = bit-exact regime, 16 = engine default)")
    ap.add_argument("--head-dim", type=int, default=128, choices=[128, 256],
                    help="decodectx / append: 256 is the reference engine's own geometry (runs on the general kernels)")
    ap.add_argument("--ctx", type=int, default=0, help="context for decodectx (default 131072) / prefix length for prefill262k (default 262144)")
    args = ap.parse_args()
    if args.head_dim != 128:
        if args.workload not in ("decodectx", "append") or args.impl != "b200":
            ap.error("--head-dim 256 is for --workload decodectx / append")
        global D, SEALED_B, TAIL_B
        D, SEALED_B, TAIL_B = 256, 280, 1024
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "decode32k":
        run_gpu(args)
    else:
        {"decodectx": run_decode_ctx, "long379k": run_long, "batch32": run_batch, "verify131k": run_verify, "prefill262k": run_prefill,
         "append": run_append}[args.workload](args)


if __name__ == "__main__":
    main()
