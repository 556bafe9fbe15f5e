#!/usr/bin/env python
"""Benchmark of the KIVI 2-bit decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2|cfg1|cfg3|small] [--path auto|fp32|mma]
                    [--scaling strong|weak] [--gather auto|peer|nccl]

One "step" = one layer-step of fused decode attention over the packed cache of
the workload (B*Hkv units, Sq quantized + Sr residual tokens each); the steps
are replayed from a CUDA graph (one pass over the rotating layer buffers per
replay), so small workloads are not bound by host launch overhead -- at N GPUs
too when the exchange is the fused one, whose call counter lives on the device.
At N GPUs the (batch, kv_head) units are sharded over the ranks and the
per-layer outputs all-gathered: --scaling strong (default) keeps the workload's
global batch and gives every rank 1/N of its units, --scaling weak gives every
rank the whole workload (global batch = N * B).  Prints ONE JSON line.

metric: 2-bit KV decode-attention HBM GB/s = algorithmic bytes / time, where
algorithmic bytes = units*[Sq*(D/2 + 16*D/G) + Sr*2*D*T] + 2*B*Hq*D*T.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, Hkv, n_rep, D, G, R, n_quant, n_res)
    "cfg2": (64, 8, 4, 128, 32, 128, 32640, 128),    # Llama-3-8B shape, batch 64, 32k context: the headline workload
    "cfg1": (16, 8, 4, 128, 32, 128, 3968, 128),     # same shape, batch 16, 4096-token context
    "cfg3": (4, 8, 4, 128, 32, 128, 131072, 128),    # same shape, batch 4, 128k-token context
    "small": (2, 8, 4, 128, 32, 128, 992, 128),
    "long": (2, 8, 4, 128, 32, 128, 65536, 128),     # few units, long history: profiling case
    "mid": (16, 8, 4, 128, 32, 128, 16384, 128),
    "prof": (14, 8, 4, 128, 32, 128, 16384, 128),    # ~one wave of CTAs with long streams: ncu case (235 MB)
}
LAYERS = 32          # Llama-3-8B depth, for the tokens/s figure


def alg_bytes(B, Hkv, n_rep, D, G, n_quant, n_res, tbytes=2):
    return B * Hkv * (n_quant * (D // 2 + 16 * D // G) + n_res * 2 * D * tbytes) + 2 * B * Hkv * n_rep * D * tbytes


NOMINAL_HBM_GBS = 8000.0          # the ~8 TB/s the target is quoted on
MIN_TIMED_SECONDS = 0.25          # the timed region is repeated until it is at least this long


def traffic_factor():
    """DRAM bytes of the attention kernel per algorithmic byte, as measured with
    ncu: read from the line `dram_traffic_over_algorithmic: <x>` of the kernel's
    profile summary, so the number is stated in one place only."""
    try:
        with open(os.path.join(ROOT, "profiles", "attn_mma_kernel_prof.md")) as f:
            for line in f:
                if line.startswith("dram_traffic_over_algorithmic:"):
                    return float(line.split(":")[1].split()[0])
    except Exception:
        pass
    return None


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi polled every 100 ms in the background; samples are kept with
    their wall-clock time so that only those taken under load are used."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self, windows):
        """windows: list of (t0, t1) wall-clock intervals (time.time()) under load."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        import datetime
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            p = [x.strip() for x in line.split(",")]
            if len(p) < 7:
                continue
            try:
                ts = datetime.datetime.strptime(p[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                f_sm, f_mx = float(p[1]), float(p[2])
            except ValueError:
                continue
            if not any(a - 0.05 <= ts <= b + 0.05 for a, b in windows):
                continue
            sm.append(f_sm); mx.append(f_mx)
            for n, v in zip(names, p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_unit_tensors(U, T, D, seed, device, dtype):
    """Seeded synthetic K/V [U, T, D] generated on the device: N(0,1); keys
    with 4 outlier channels per head x10, values with 2% of tokens x8."""
    g = torch.Generator(device=device).manual_seed(seed)
    k = torch.empty(U, T, D, device=device, dtype=dtype)
    v = torch.empty(U, T, D, device=device, dtype=dtype)
    step = max(1, (1 << 28) // (T * D))
    for u0 in range(0, U, step):
        u1 = min(U, u0 + step)
        kk = torch.randn(u1 - u0, T, D, device=device, generator=g)
        ch = torch.rand(u1 - u0, D, device=device, generator=g).argsort(dim=1)[:, :4]
        mul = torch.ones(u1 - u0, D, device=device)
        mul.scatter_(1, ch, 10.0)
        k[u0:u1] = (kk * mul[:, None, :]).to(dtype)
        vv = torch.randn(u1 - u0, T, D, device=device, generator=g)
        tokm = (torch.rand(u1 - u0, T, device=device, generator=g) < 0.02).float() * 7.0 + 1.0
        v[u0:u1] = (vv * tokm[:, :, None]).to(dtype)
        del kk, vv
    return k, v


def unit_bytes(U, n_rep, D, G, n_quant, n_res, tbytes=2):
    """alg_bytes() for U (batch, kv_head) units."""
    return U * (n_quant * (D // 2 + 16 * D // G) + n_res * 2 * D * tbytes) + 2 * U * n_rep * D * tbytes


def cpu_attention_sample(B_s, Hkv, n_rep, D, G, n_quant, n_res, iters, threads):
    """The reference's CPU path for one decode layer-step on a slice of the
    batch: attention over the served fp32 cache (already round-tripped history
    || residual, cache/manager.py:263-286), plus 1/G of a flush round trip."""
    from oracle import kivi_oracle as ko
    torch.set_num_threads(threads)
    T = n_quant + n_res
    K = ko.make_keys(B_s, Hkv, T, D, seed=1).to(torch.bfloat16)
    V = ko.make_values(B_s, Hkv, T, D, seed=1).to(torch.bfloat16)
    q = ko.make_queries(B_s, Hkv * n_rep, D, seed=1).to(torch.bfloat16).float()
    kf, vf = K.float(), V.float()
    kq = ko.roundtrip_groups(kf[:, :, :n_quant].reshape(B_s, Hkv, n_quant // G, G, D).transpose(3, 4).contiguous(), G)
    kf[:, :, :n_quant] = kq.transpose(3, 4).reshape(B_s, Hkv, n_quant, D)
    vf[:, :, :n_quant] = ko.roundtrip_groups(vf[:, :, :n_quant].contiguous(), G)
    chunk_k = kf[:, :, :G].transpose(2, 3).contiguous()
    chunk_v = vf[:, :, :G].contiguous()
    ko.attention(q.unsqueeze(2), kf, vf)
    ts = []
    for _ in range(iters):
        t0 = time.perf_counter()
        ko.attention(q.unsqueeze(2), kf, vf)
        t1 = time.perf_counter()
        ko.roundtrip_groups(chunk_k, G); ko.roundtrip_groups(chunk_v, G)
        t2 = time.perf_counter()
        ts.append((t1 - t0) + (t2 - t1) / G)
    return statistics.median(ts)


def run_reference(args, wl):
    """--impl reference: the reference's CPU path (oracle port of its torch
    mirror + attention formula) on the host cores, one bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    B, Hkv, n_rep, D, G, R, n_quant, n_res = wl
    threads = os.cpu_count() or 1
    B_s = 1                                   # one batch row of the workload per step
    iters = max(1, args.steps)
    for _ in range(max(0, args.warmup - 1)):
        cpu_attention_sample(B_s, Hkv, n_rep, D, G, n_quant, n_res, 1, threads)
    t = cpu_attention_sample(B_s, Hkv, n_rep, D, G, n_quant, n_res, iters, threads)
    by = alg_bytes(B_s, Hkv, n_rep, D, G, n_quant, n_res)
    gbs = by / t / 1e9
    sample = f"B={B_s} of {B} batch rows (Hkv={Hkv}, {n_quant}+{n_res} tokens), scaled by bytes"
    line = {"impl": "reference", "metric": "kivi_2bit_decode_attention_hbm_gbs", "value": gbs, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": t * 1e3 * (B / B_s), "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 and args.scaling == "strong" else "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "B_global": B if (args.gpus == 1 or args.scaling == "strong") else B * args.gpus,
                       "units_per_gpu": (B * Hkv + args.gpus - 1) // args.gpus if (args.gpus > 1 and args.scaling == "strong") else B * Hkv,
                       "Hkv": Hkv, "Hq": Hkv * n_rep, "D": D, "G": G, "n_quant": n_quant, "n_res": n_res,
                       "parallelism": "reference CPU path on rank 0's host cores, one batch row per step"},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def run_ours(args, wl):
    from intel_kivi_hybrid_b200 import cabi
    from intel_kivi_hybrid_b200.parallel import unit_partition
    import torch.distributed as dist
    B, Hkv, n_rep, D, G, R, n_quant, n_res = wl
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    sampler = ClockSampler(local) if rank == 0 else None     # started early: nvidia-smi needs a moment to come up
    dtype = torch.bfloat16
    path = {"auto": cabi.ATTN_AUTO, "fp32": cabi.ATTN_FP32, "mma": cabi.ATTN_MMA}[args.path]
    strong = world > 1 and args.scaling == "strong"
    # strong: the workload's B*Hkv units are split over the ranks; weak: every rank holds all of them
    U_total = B * Hkv if (strong or world == 1) else world * B * Hkv
    u0, u1 = unit_partition(U_total, rank, world)
    U = u1 - u0
    assert U > 0, f"{U_total} units cannot be spread over {world} ranks"
    T = n_quant + n_res
    by_rank = unit_bytes(U, n_rep, D, G, n_quant, n_res)
    by_total = unit_bytes(U_total, n_rep, D, G, n_quant, n_res)
    # layer-sized stores are rotated so no step finds its inputs in L2
    n_buf = 2 if by_rank > (1 << 29) else 8
    stores = []
    k, v = make_unit_tensors(U, T, D, 1000 + rank, dev, dtype)
    k0, v0 = k[:1].cpu(), v[:1].cpu()             # this rank's first unit, kept for the oracle check
    for i in range(n_buf):
        st = cabi.LayerStore(U, D, G, R, n_quant, dtype, dev)
        if i == 0:
            cabi.load_state(st, k, v, n_quant)
        else:                                  # same bytes, different addresses
            for name in ("k_codes", "k_scales", "k_zeros", "v_codes", "v_scales", "v_zeros", "k_res", "v_res"):
                getattr(st, name).copy_(getattr(stores[0], name))
            st.quant_len, st.res_start, st.res_len = n_quant, 0, n_res
        stores.append(st)
    del k, v
    torch.cuda.empty_cache()
    q = torch.randn(U, n_rep, D, device=dev, generator=torch.Generator(device=dev).manual_seed(7 + rank)).to(dtype)
    out = torch.empty_like(q)
    gathered = torch.empty(U_total, n_rep, D, device=dev, dtype=dtype) if world > 1 else None
    equal_shards = U * world == U_total
    # the exchange of a step: an NCCL all-gather after the kernels, or the
    # attention's last kernel storing its rows into every rank's buffer itself
    pg, pg_host, gather_note = None, None, None
    wait_stats = torch.zeros(2, dtype=torch.int64, device=dev)
    if world > 1 and args.gather in ("peer", "auto"):
        from intel_kivi_hybrid_b200.parallel import PeerGather
        try:                                   # raises on every rank or on none
            pg = PeerGather(U_total, n_rep, D, dtype, rank, world, device_epoch=True)   # replayable from a CUDA graph
            pg_host = PeerGather(U_total, n_rep, D, dtype, rank, world)      # host-kept epoch: the end-to-end loop
        except RuntimeError as exc:
            pg, gather_note = None, f"peer-gather setup failed ({exc}); NCCL all-gather used"
    if world > 1 and not equal_shards and pg is None:
        raise SystemExit("ragged unit shards need --gather peer/auto (the NCCL path uses all_gather_into_tensor)")

    def attend(store, q=q, stats=None, want_rows=False):
        if pg is not None:
            store.attention_gather(q, pg.descriptor(wait_stats=stats), dtype, n_rep, path=path, num_splits=args.splits)
            # (finding the buffer of the last call reads the device-kept counter back: only the self-check asks)
            return pg.gathered() if want_rows else None
        store.attention(q, out=out, n_rep=n_rep, path=path, num_splits=args.splits)
        if world > 1:
            dist.all_gather_into_tensor(gathered, out)
            return gathered
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- parity, before anything is timed ------------------------------------------
    # (1) this rank's first unit against the CPU oracle in fp64 (rank 0's figure is
    #     reported); (2) at N > 1 the gathered rows of every rank must be bit for bit
    #     what that rank computes alone, for the exchange in use and, with the fused
    #     exchange, on both halves of its double buffer.  A fused exchange that fails
    #     (2) is replaced by the NCCL all-gather on every rank, and the line says so.
    from oracle import kivi_oracle as ko            # the checker, never the thing measured
    alone = stores[0].attention(q, n_rep=n_rep, path=path, num_splits=args.splits).clone()
    ref = ko.kivi_decode_attention(q[:1].cpu().reshape(1, n_rep, D), k0.reshape(1, 1, T, D), v0.reshape(1, 1, T, D),
                                   n_quant, G, "half_away", dtype=torch.float64).float().reshape(n_rep, D)
    rel = lambda got: float(((got.float().cpu() - ref).abs().amax(-1) / ref.abs().amax(-1)).max())
    # the kernel's own error (fp32 output) and what the bf16 output of the timed steps adds (half an ulp: 2e-3)
    oracle_err = rel(stores[0].attention(q, n_rep=n_rep, path=path, num_splits=args.splits, out_dtype=torch.float32)[0])
    oracle_err_bf16_out = rel(alone[0])
    gather_ok = None
    if world > 1:
        def gathered_equals_alone():
            ok = 1
            for _ in range(2):
                g = attend(stores[0], want_rows=True)
                torch.cuda.synchronize()
                ok &= int(torch.equal(g[u0:u1], alone))
            ok &= int(cabi.device_fault() == 0)
            t_ok = torch.tensor([ok], device=dev)
            dist.all_reduce(t_ok, op=dist.ReduceOp.MIN)
            return bool(t_ok.item())
        try:
            gather_ok = gathered_equals_alone()
        except RuntimeError as exc:
            print(f"[bench] rank {rank}: exchange failed its self-check: {exc}", file=sys.stderr)
            gather_ok = False
        if not gather_ok and pg is not None and equal_shards:
            gather_note = "fused exchange failed its bitwise self-check; NCCL all-gather used"
            pg.close(); pg_host.close()
            pg = pg_host = None
            cabi.device_fault_clear()
            gather_ok = gathered_equals_alone()
    del k0, v0

    def step(i, stats=None):
        attend(stores[i % n_buf], stats=stats)

    for i in range(max(3, args.warmup)):
        step(i)
    launches_per_step = cabi.lib.kivi_last_launch_count()
    barrier()
    # Launch-bound case (small workloads): capture one pass over the rotating layer
    # buffers in a CUDA graph and replay it; a "step" is still one layer-step.
    def capture(fn):
        """One pass of fn over the rotating layer buffers as a CUDA graph (None if capture is unavailable)."""
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(n_buf):
                    fn(i)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(n_buf):
                    fn(i)
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            return g
        except Exception as exc:          # capture unavailable: time plain launches instead
            print(f"[bench] CUDA graph capture failed ({exc}); timing plain launches", file=sys.stderr)
            torch.cuda.synchronize()
            return None

    # at N > 1 only the fused exchange is replayable (its call counter lives on the
    # device); every rank must take the same decision, or none replays
    graph = None
    if args.graph and (world == 1 or pg is not None):
        graph = capture(lambda i: step(i, wait_stats if pg is not None else None))
        if world > 1:
            ok = torch.tensor([int(graph is not None)], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if not bool(ok.item()):
                graph = None

    def timed(n_steps, use_graph, stats=None, fn=None, g=None):
        """(total ms, sorted per-step ms) of n_steps steps, CUDA events on the launching stream."""
        fn = fn or (lambda i: step(i, stats))
        if use_graph:
            g = g or graph
            reps = max(1, (n_steps + n_buf - 1) // n_buf)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
            ev[0].record()
            for i in range(reps):
                g.replay()
                ev[i + 1].record()
            barrier()
            per = sorted(ev[i].elapsed_time(ev[i + 1]) / n_buf for i in range(reps))
            return ev[0].elapsed_time(ev[-1]) * n_steps / (reps * n_buf), per
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(n_steps + 1)]
        ev[0].record()
        for i in range(n_steps):
            fn(i)
            ev[i + 1].record()
        barrier()
        return ev[0].elapsed_time(ev[-1]), sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(n_steps))

    # the timed region: exactly --steps steps, repeated until it lasts MIN_TIMED_SECONDS
    # (the same number of repeats on every rank)
    est_ms, _ = timed(args.steps, graph is not None)
    rep = torch.tensor([max(1, int(args.min_seconds * 1e3 / max(est_ms, 1e-3)) + 1)], device=dev)
    if world > 1:
        dist.all_reduce(rep, op=dist.ReduceOp.MAX)
    n_timed = args.steps * int(rep.item())
    windows = []
    barrier()
    w0 = time.time()
    total_ms, per = timed(n_timed, graph is not None, stats=wait_stats if pg is not None else None)
    windows.append((w0, time.time()))
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_step = total_ms / n_timed
    value = by_total / (ms_step * 1e-3) / 1e9

    extra = {}
    if graph is not None:
        ng_ms, ng_per = timed(args.steps, False)
        extra["ms_per_step_no_graph"] = statistics.median(ng_per)
    if world > 1:
        # the same steps without the exchange: what every rank needs for its own units
        local = lambda i: stores[i % n_buf].attention(q, out=out, n_rep=n_rep, path=path, num_splits=args.splits)
        g_local = capture(local) if graph is not None else None
        if world > 1:
            ok = torch.tensor([int(g_local is not None)], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if not bool(ok.item()):
                g_local = None
        lo_ms, lo_per = timed(args.steps, g_local is not None, fn=local, g=g_local)
        t = torch.tensor([statistics.median(lo_per), -statistics.median(lo_per)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ws = wait_stats.clone().double()
        wait_us = float(ws[0] / max(float(ws[1]), 1.0)) / 1e3
        tw = torch.tensor([wait_us, -wait_us], device=dev)
        dist.all_reduce(tw, op=dist.ReduceOp.MAX)
        slowest, fastest = float(t[0]), -float(t[1])
        exchange = statistics.median(per) - slowest
        extra["per_rank"] = {
            "ms_local_attention_slowest": slowest, "ms_local_attention_fastest": fastest,
            "ms_step_minus_slowest_local": exchange,
            "us_wait_for_peers_in_kernel_max": float(tw[0]) if pg is not None else None,
            "us_wait_for_peers_in_kernel_min": -float(tw[1]) if pg is not None else None,
            "limiter": ("skew between ranks" if slowest - fastest > max(exchange, 0.0) else
                        "exchange (peer stores, flags, wait)" if exchange > 0.02 * slowest else "the attention kernel itself"),
            "note": "local = the same attention without the exchange, launched the same way as the timed steps "
                    "(replayed from a CUDA graph when they are)"}

    # ---- end to end: host q + host new K/V token in, host out, every step ----
    # through the library's host-to-host decode step (one foreign call per step; the
    # units go in two chunks on separate streams so copies overlap the kernels)
    h_q = q.cpu().pin_memory()
    h_k = torch.randn(U, D).to(dtype).pin_memory()
    h_v = torch.randn(U, D).to(dtype).pin_memory()
    h_out = torch.empty(U_total, n_rep, D, dtype=dtype).pin_memory()
    e2e_store = stores[-1]
    # start from "n_quant quantized + (R - G) in the ring" so flushes happen at the real rate (1 step in G)
    e2e_store.quant_len, e2e_store.res_start, e2e_store.res_len = n_quant - G, 0, R - G
    n_e2e = max(args.steps, G)
    d_q, d_k, d_v = q.clone(), torch.empty(U, 1, D, device=dev, dtype=dtype), torch.empty(U, 1, D, device=dev, dtype=dtype)

    def e2e_step():
        if world > 1 and pg is None:                 # NCCL exchange: the collective is issued from Python
            d_q.copy_(h_q, non_blocking=True); d_k[:, 0].copy_(h_k, non_blocking=True); d_v[:, 0].copy_(h_v, non_blocking=True)
            e2e_store.update(d_k, d_v)
            h_out.copy_(attend(e2e_store, d_q), non_blocking=True)
        elif pg is not None:
            e2e_store.decode_step_host(h_q, h_k, h_v, h_out, n_rep, num_splits=args.splits, path=path,
                                       direct=not args.e2e_staged, gather=pg_host.descriptor(), gather_units=U_total)
        else:
            e2e_store.decode_step_host(h_q, h_k, h_v, h_out, n_rep, num_splits=args.splits, path=path,
                                       chunks=args.e2e_chunks, direct=not args.e2e_staged)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_store.quant_len, e2e_store.res_start, e2e_store.res_len = n_quant - G, 0, R - G
        e2e_step()
    e2e_store.quant_len, e2e_store.res_start, e2e_store.res_len = n_quant - G, 0, R - G
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n_e2e):
        if e2e_store.quant_len + G > e2e_store.max_tokens and e2e_store.res_len == R - 1:
            e2e_store.quant_len, e2e_store.res_start, e2e_store.res_len = n_quant - G, 0, R - G
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / n_e2e
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_val = by_total / (e2e_ms * 1e-3) / 1e9

    # the timed region can be shorter than one polling period of nvidia-smi: every
    # rank keeps the same step loop running (untimed) for about 1.2 s more -- the
    # same number of steps everywhere, because a step holds a collective
    clocks = None
    n_extra = torch.tensor([int(min(20000, max(args.steps, 1.2e3 / max(ms_step, 1e-3)))) if args.min_seconds > 0 else 1],
                           device=dev)
    if world > 1:
        dist.all_reduce(n_extra, op=dist.ReduceOp.MAX)
    w0 = time.time()
    for i in range(int(n_extra.item())):
        step(i)
        if i % 200 == 199:
            torch.cuda.synchronize()
    barrier()
    windows.append((w0, time.time()))
    fault = cabi.device_fault()            # non-zero: a bounded wait inside a kernel ran out
    if sampler is not None:
        clocks = sampler.stop(windows)
        clocks["sampled"] = "timed region plus ~1.2 s of the same step loop right after it"
    if rank == 0:
        peak, which = peaks()
        achieved = by_rank / (statistics.median(per) * 1e-3) / 1e9
        tf = traffic_factor()
        cpu = None
        if world == 1 and not args.no_cpu:
            threads = os.cpu_count() or 1
            t_cpu = cpu_attention_sample(1, Hkv, n_rep, D, G, n_quant, n_res, 3, threads)
            cpu = {"value": alg_bytes(1, Hkv, n_rep, D, G, n_quant, n_res) / t_cpu / 1e9, "unit": "GB/s",
                   "cores": threads, "kind": "port",
                   "sample": f"B=1 of {B} batch rows, 3 timed passes of the reference CPU path (fp32 attention over "
                             f"the served cache + 1/G flush round trip), median"}
        exchange_txt = ("" if world == 1 else " by NCCL" if pg is None else
                        " inside the merge kernel (peer stores over NVLink)")
        line = {"metric": "kivi_2bit_decode_attention_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": args.workload, "B_global": U_total // Hkv, "units_per_gpu": U, "Hkv": Hkv,
                           "Hq": Hkv * n_rep, "D": D, "G": G, "n_quant": n_quant, "n_res": n_res, "path": args.path,
                           "layer_buffers_rotated": n_buf, "cuda_graph": graph is not None,
                           "l2": "inputs larger than L2 (layer buffers rotated)",
                           "parallelism": f"(batch,kv_head) units over {world} GPU(s), all-gather of outputs" + exchange_txt},
                "timed_steps": n_timed,
                "ms_per_step_median": statistics.median(per), "ms_per_step_p10": per[len(per) // 10],
                "ms_per_step_p90": per[min(len(per) - 1, (9 * len(per)) // 10)],
                "decode_tokens_per_s": (U_total // Hkv) / (LAYERS * ms_step * 1e-3),
                "parity": {"oracle_rel_err": oracle_err, "oracle_rel_err_bf16_output": oracle_err_bf16_out,
                           "oracle_sample": "rank 0, first unit against the fp64 CPU oracle, error of an output row over "
                                            "the row's largest reference element; bar 2e-3 for the fp32 output",
                           "gather_bitwise": gather_ok, "gather_note": gather_note},
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "peak_source": which, "frac_nominal": achieved / NOMINAL_HBM_GBS,
                             "nominal_peak": NOMINAL_HBM_GBS,
                             "traffic": by_rank * tf if tf else None,
                             "note": "per GPU: achieved = this rank's algorithmic bytes / median per-step CUDA-event time "
                                     "(attention kernel + split merge); traffic = ncu dram bytes of attn_mma_kernel per "
                                     "algorithmic byte on the profiling workload (profiles/attn_mma_kernel_prof.md), "
                                     "scaled to this launch"},
                "cpu_baseline": cpu,
                "e2e": {"value": e2e_val, "unit": "GB/s", "ms_per_step": e2e_ms,
                        "h2d_bytes_per_step": world * (h_q.numel() + h_k.numel() + h_v.numel()) * 2,
                        "d2h_bytes_per_step": world * h_out.numel() * 2,
                        "note": "pinned host q + new K/V token -> cache update (flush every G steps) -> attention -> "
                                "pinned host out, one kivi_decode_step_host call per step"
                                + (f", staged copies in {args.e2e_chunks} chunk(s)" if args.e2e_staged else
                                   ", kernels reading and writing the pinned buffers directly")},
                "gpu_launches": n_timed * launches_per_step,
                "device_fault": fault,
                "clocks": clocks}
        line.update(extra)
        print(json.dumps(line))
    if pg is not None:
        pg.close(); pg_host.close()
    if world > 1:
        dist.destroy_process_group()


def run_quantize(args):
    """--workload cfg4: bulk prefill flush (Llama-2-7B MHA shapes): B=8, 32 KV heads,
    D=128, 8192 tokens quantized in one kivi_cache_update call per layer (keys per
    channel over 32-token groups, values per token over 32-channel groups)."""
    from intel_kivi_hybrid_b200 import cabi
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    U, S, D, G, R = 8 * 32, 8192, 128, 32, 128
    res = {}
    for name, dtype, eb in (("f32", torch.float32, 4), ("bf16", torch.bfloat16, 2)):
        k, v = make_unit_tensors(8 * 32, S, D, 77, dev, dtype)
        st = cabi.LayerStore(U, D, G, R, S, dtype, dev)
        n_flush, ql, rl = cabi.cache_plan(0, 0, S, G, R)
        by = 2 * U * (ql * D * eb + ql * D // 4 + (ql * D // G) * 8) + 2 * U * rl * D * eb * 2
        for _ in range(max(3, args.warmup)):
            st.reset(); st.update(k, v)
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        ev[0].record()
        for i in range(args.steps):
            st.reset(); st.update(k, v)
            ev[i + 1].record()
        torch.cuda.synchronize()
        per = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps))
        res[name] = {"ms": statistics.median(per), "gbs": by / (statistics.median(per) * 1e-3) / 1e9, "bytes": by,
                     "launches": cabi.lib.kivi_last_launch_count()}
        del k, v, st
        torch.cuda.empty_cache()
    peak, which = peaks()
    line = {"metric": "kivi_quantize_pack_gbs", "value": res["bf16"]["gbs"], "unit": "GB/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["bf16"]["ms"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg4", "units": U, "tokens": S, "D": D, "G": G, "R": R,
                       "l2": "inputs larger than L2 (1.07 GB per tensor)"},
            "f32": res["f32"], "bf16": res["bf16"],
            "roofline": {"bound": "hbm", "achieved": res["bf16"]["gbs"], "peak": peak, "unit": "GB/s",
                         "frac": res["bf16"]["gbs"] / peak, "frac_f32": res["f32"]["gbs"] / peak, "peak_source": which,
                         "traffic": None},
            "gpu_launches": args.steps * res["bf16"]["launches"]}
    print(json.dumps(line))


def run_operators(args):
    """--workload ops: the flat-group operators of the reference's module
    (quantize / dequantize / fused round trip on 2^28 elements, G=32 and 128,
    fp32 and bf16 input) and the dense-cache materialisation behind
    get_full_cache (64 units x 8288 tokens), CUDA-event medians."""
    from intel_kivi_hybrid_b200 import cabi
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    N = 1 << 28

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        ev[0].record()
        for i in range(args.steps):
            fn()
            ev[i + 1].record()
        torch.cuda.synchronize()
        return statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps))

    res = {}
    for name, dtype, eb in (("f32", torch.float32, 4), ("bf16", torch.bfloat16, 2)):
        x = torch.randn(N, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).to(dtype)
        out = torch.empty(N, device=dev)
        for G in (32, 128):
            packed = torch.empty(N // 4, dtype=torch.uint8, device=dev)
            sc, ze = torch.empty(N // G, device=dev), torch.empty(N // G, device=dev)
            ms = timed(lambda: cabi.quantize_keys(x, packed, sc, ze, G))
            res[f"quantize_{name}_G{G}"] = {"ms": ms, "gbs": (N * eb + N // 4 + 8 * N // G) / ms / 1e6}
            ms = timed(lambda: cabi.roundtrip_keys(x, out, G))
            res[f"roundtrip_{name}_G{G}"] = {"ms": ms, "gbs": (N * eb + 4 * N) / ms / 1e6}
            if name == "f32":
                ms = timed(lambda: cabi.dequantize_keys(packed, sc, ze, out, G))
                res[f"dequantize_G{G}"] = {"ms": ms, "gbs": (N // 4 + 8 * N // G + 4 * N) / ms / 1e6}
            del packed, sc, ze
        del x, out
        torch.cuda.empty_cache()
    U, T, D, G, R = 64, 8192 + 96, 128, 32, 128
    k, v = make_unit_tensors(8 * 8, T, D, 9, dev, torch.bfloat16)
    st = cabi.LayerStore(U, D, G, R, T, torch.bfloat16, dev)
    st.update(k, v)
    ko_, vo_ = st.materialize()
    del ko_, vo_
    ms = timed(lambda: st.materialize())
    res["materialize_bf16_ring"] = {"ms": ms, "gbs": (2 * U * T * D * 4 + U * st.quant_len * 128) / ms / 1e6,
                                    "note": "includes the allocation of the two output tensors"}
    peak, which = peaks()
    head = res["quantize_bf16_G32"]
    line = {"metric": "kivi_operator_gbs", "value": head["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "ops", "elements": N, "headline": "quantize_bf16_G32",
                       "l2": "inputs larger than L2 (0.5-1 GB per tensor)"},
            "operators": res,
            "roofline": {"bound": "hbm", "achieved": head["gbs"], "peak": peak, "unit": "GB/s", "frac": head["gbs"] / peak,
                         "peak_source": which, "traffic": None},
            "gpu_launches": args.steps}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gather", default="auto", choices=["auto", "nccl", "peer"],
                    help="N>1: how the attention outputs are all-gathered: by NCCL after the kernels, or by the "
                         "attention's last kernel through peer memory (auto = the latter if it passes a self-check)")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N>1: strong = the workload's global batch sharded over the GPUs (the configuration the "
                         "workloads are defined on), weak = every GPU holds the whole workload")
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS) + ["cfg4", "ops"])
    ap.add_argument("--path", default="auto", choices=["auto", "fp32", "mma"])
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--min-seconds", type=float, default=MIN_TIMED_SECONDS,
                    help="repeat the --steps timed steps until the timed region lasts this long (0: exactly --steps; "
                         "used for profiler runs)")
    ap.add_argument("--e2e-staged", action="store_true",
                    help="end-to-end step through explicit staging copies instead of kernels accessing the pinned host buffers")
    ap.add_argument("--e2e-chunks", type=int, default=1, help="with --e2e-staged: chunks of units whose copies and kernels overlap")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graph", dest="graph", action="store_false",
                    help="launch every step from Python instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.workload == "ops":
        return run_operators(args)
    if args.workload == "cfg4":
        return run_quantize(args)
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
