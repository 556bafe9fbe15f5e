#!/usr/bin/env python
"""Benchmark of the KIVI 2-bit decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2|cfg1|cfg3|small] [--path auto|fp32|mma]

One "step" = one layer-step of fused decode attention over the packed cache of
the workload (B*Hkv units, Sq quantized + Sr residual tokens each); on one GPU
the steps are replayed from a CUDA graph (one pass over the rotating layer
buffers per replay), so small workloads are not bound by host launch overhead.  At N GPUs
every rank holds the workload's units (weak scaling: global batch = N * B) and
the per-layer outputs are all-gathered over NCCL.  Prints ONE JSON line.

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
    "cfg2": (64, 8, 4, 128, 32, 128, 32640, 128),    # BASELINE configs[2]: B=64, 32k context
    "cfg1": (16, 8, 4, 128, 32, 128, 3968, 128),     # configs[1]: B=16, 4096 context
    "cfg3": (4, 8, 4, 128, 32, 128, 131072, 128),    # configs[3]: B=4, 128k context
    "small": (2, 8, 4, 128, 32, 128, 992, 128),
    "long": (2, 8, 4, 128, 32, 128, 65536, 128),     # few units, long history: profiling case
    "mid": (16, 8, 4, 128, 32, 128, 16384, 128),
    "prof": (14, 8, 4, 128, 32, 128, 16384, 128),    # ~one wave of CTAs with long streams: ncu case (235 MB)
}
LAYERS = 32          # Llama-3-8B depth, for the tokens/s figure


def alg_bytes(B, Hkv, n_rep, D, G, n_quant, n_res, tbytes=2):
    return B * Hkv * (n_quant * (D // 2 + 16 * D // G) + n_res * 2 * D * tbytes) + 2 * B * Hkv * n_rep * D * tbytes


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


def make_unit_tensors(B, Hkv, T, D, seed, device, dtype):
    """Seeded synthetic K/V [B*Hkv, T, D] generated on the device: N(0,1); keys
    with 4 outlier channels per head x10, values with 2% of tokens x8."""
    g = torch.Generator(device=device).manual_seed(seed)
    U = B * Hkv
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
            "ms_per_step": t * 1e3 * (B / B_s), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "B_per_gpu": B, "Hkv": Hkv, "Hq": Hkv * n_rep, "D": D, "G": G,
                       "n_quant": n_quant, "n_res": n_res,
                       "parallelism": "reference CPU path on rank 0's host cores, one batch row per step"},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def run_ours(args, wl):
    from intel_kivi_hybrid_b200 import cabi
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
    U = B * Hkv
    T = n_quant + n_res
    # two layer-sized stores are rotated so no step finds its inputs in L2
    n_buf = 2 if alg_bytes(*wl[:5], n_quant, n_res) > (1 << 29) else 8
    stores = []
    k, v = make_unit_tensors(B, Hkv, T, D, 1000 + rank, dev, dtype)
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
    q = torch.randn(U, n_rep, D, device=dev, generator=torch.Generator(device=dev).manual_seed(7)).to(dtype)
    out = torch.empty_like(q)
    gathered = torch.empty(world * U, n_rep, D, device=dev, dtype=dtype) if world > 1 else None
    # the exchange of a step: an NCCL all-gather after the kernels, or the
    # attention's last kernel storing its rows into every rank's buffer itself
    pg = None
    if world > 1 and args.gather in ("peer", "auto"):
        from intel_kivi_hybrid_b200.parallel import PeerGather
        try:                                   # raises on every rank or on none
            pg = PeerGather(world * U, n_rep, D, dtype, rank, world)
        except RuntimeError as exc:
            if rank == 0:
                print(f"[bench] {exc}; falling back to the NCCL all-gather", file=sys.stderr)
        if pg is not None:
            # self-check before anything is timed: two fused steps (both halves of the
            # double buffer) must reproduce the NCCL all-gather bit for bit on every
            # rank with no wait having run out; otherwise all ranks use NCCL
            ok = 1
            try:
                stores[0].attention(q, out=out, n_rep=n_rep, path=path, num_splits=args.splits)
                dist.all_gather_into_tensor(gathered, out)
                for _ in range(2):
                    stores[0].attention_gather(q, pg.descriptor(), dtype, n_rep, path=path, num_splits=args.splits)
                    torch.cuda.synchronize()
                    ok &= int(torch.equal(pg.gathered(), gathered))
                ok &= int(cabi.device_fault() == 0)
            except RuntimeError as exc:
                print(f"[bench] rank {rank}: fused gather failed its self-check: {exc}", file=sys.stderr)
                ok = 0
            t_ok = torch.tensor([ok], device=dev)
            dist.all_reduce(t_ok, op=dist.ReduceOp.MIN)
            if int(t_ok.item()) == 0:
                if rank == 0:
                    print("[bench] fused gather failed its self-check; using the NCCL all-gather", file=sys.stderr)
                pg.close()
                pg = None

    def attend(store, q=q):
        if pg is not None:
            store.attention_gather(q, pg.descriptor(), dtype, n_rep, path=path, num_splits=args.splits)
            return pg.gathered()[rank * U:(rank + 1) * U]
        store.attention(q, out=out, n_rep=n_rep, path=path, num_splits=args.splits)
        if world > 1:
            dist.all_gather_into_tensor(gathered, out)
        return out

    def step(i):
        attend(stores[i % n_buf])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    launches_per_step = cabi.lib.kivi_last_launch_count()
    barrier()
    # Launch-bound case (small workloads): capture one pass over the rotating layer
    # buffers in a CUDA graph and replay it; a "step" is still one layer-step.
    graph = None
    if args.graph and world == 1:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(n_buf):
                    step(i)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(n_buf):
                    step(i)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
        except Exception as exc:          # capture unavailable: time plain launches instead
            print(f"[bench] CUDA graph capture failed ({exc}); timing plain launches", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    windows = []
    w0 = time.time()
    if graph is not None:
        n_rep_g = max(1, (args.steps + n_buf - 1) // n_buf)          # replays; each = n_buf steps
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(n_rep_g + 1)]
        ev[0].record()
        for i in range(n_rep_g):
            graph.replay()
            ev[i + 1].record()
        barrier()
        windows.append((w0, time.time()))
        total_ms = ev[0].elapsed_time(ev[-1]) * args.steps / (n_rep_g * n_buf)
        per = sorted(ev[i].elapsed_time(ev[i + 1]) / n_buf for i in range(n_rep_g))
    else:
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        ev[0].record()
        for i in range(args.steps):
            step(i)
            ev[i + 1].record()
        barrier()
        windows.append((w0, time.time()))
        total_ms = ev[0].elapsed_time(ev[-1])
        per = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps))
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_step = total_ms / args.steps
    by = alg_bytes(B, Hkv, n_rep, D, G, n_quant, n_res)
    value = world * by / (ms_step * 1e-3) / 1e9

    # ---- end to end: host q + host new K/V token in, host out, every step ----
    # one pinned staging buffer [q | new K token | new V token] and one copy per step
    nq = q.numel()
    h_in = torch.empty(nq + 2 * U * D, dtype=dtype).pin_memory()
    h_in[:nq] = q.cpu().reshape(-1)
    h_in[nq:] = torch.randn(2 * U * D).to(dtype)
    d_in = torch.empty(nq + 2 * U * D, device=dev, dtype=dtype)
    q_e2e = d_in[:nq].view(U, n_rep, D)
    d_kv = d_in[nq:].view(2, U, 1, D)
    h_out = torch.empty(U, n_rep, D, dtype=dtype).pin_memory()
    e2e_store = stores[-1]
    # start from "n_quant quantized + (R - G) in the ring" so flushes happen at the real rate (1 step in G)
    e2e_store.quant_len, e2e_store.res_start, e2e_store.res_len = n_quant - G, 0, R - G
    n_e2e = max(args.steps, G)

    def e2e_step():
        d_in.copy_(h_in, non_blocking=True)
        e2e_store.update(d_kv[0], d_kv[1])
        h_out.copy_(attend(e2e_store, q_e2e), non_blocking=True)
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
    e2e_val = world * by / (e2e_ms * 1e-3) / 1e9

    # the timed region can be shorter than one polling period of nvidia-smi: every
    # rank keeps the same step loop running (untimed) for about 1.2 s more -- the
    # same number of steps everywhere, because a step holds a collective
    clocks = None
    n_extra = int(min(20000, max(args.steps, 1.2e3 / max(ms_step, 1e-3))))
    w0 = time.time()
    for i in range(n_extra):
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
        achieved = by / (statistics.median(per) * 1e-3) / 1e9
        cpu = None
        if world == 1 and not args.no_cpu:
            threads = os.cpu_count() or 1
            t_cpu = cpu_attention_sample(1, Hkv, n_rep, D, G, n_quant, n_res, 3, threads)
            cpu = {"value": alg_bytes(1, Hkv, n_rep, D, G, n_quant, n_res) / t_cpu / 1e9, "unit": "GB/s",
                   "cores": threads, "kind": "port",
                   "sample": f"B=1 of {B} batch rows, 3 timed passes of the reference CPU path (fp32 attention over "
                             f"the served cache + 1/G flush round trip), median"}
        line = {"metric": "kivi_2bit_decode_attention_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": args.workload, "B_per_gpu": B, "Hkv": Hkv, "Hq": Hkv * n_rep, "D": D, "G": G,
                           "n_quant": n_quant, "n_res": n_res, "path": args.path, "layer_buffers_rotated": n_buf,
                           "cuda_graph": graph is not None,
                           "l2": "inputs larger than L2 (layer buffers rotated)",
                           "parallelism": f"(batch,kv_head) units x{world}, all-gather of outputs"
                                          + ("" if world == 1 else " by NCCL" if pg is None else
                                             " inside the merge kernel (peer stores over NVLink)")},
                "ms_per_step_median": statistics.median(per), "ms_per_step_p10": per[len(per) // 10],
                "ms_per_step_p90": per[min(len(per) - 1, (9 * len(per)) // 10)],
                "decode_tokens_per_s": world * B / (LAYERS * ms_step * 1e-3),
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "peak_source": which, "traffic": by * 1.026,
                             "note": "achieved = algorithmic bytes / median per-step CUDA-event time (attention kernel + split merge); "
                                     "traffic = ncu dram bytes of attn_mma_kernel on the 235 MB prof workload (1.026x its "
                                     "algorithmic bytes), scaled to this launch"},
                "cpu_baseline": cpu,
                "e2e": {"value": e2e_val, "unit": "GB/s", "ms_per_step": e2e_ms,
                        "h2d_bytes_per_step": h_in.numel() * 2, "d2h_bytes_per_step": h_out.numel() * 2,
                        "note": "host q + new K/V token -> cache update (flush every G steps) -> attention -> host out"},
                "gpu_launches": args.steps * launches_per_step,
                "device_fault": fault,
                "clocks": clocks}
        print(json.dumps(line))
    if pg is not None:
        pg.close()
    if world > 1:
        dist.destroy_process_group()


def run_quantize(args):
    """--workload cfg4: bulk prefill flush (BASELINE configs[4]): B=8, 32 KV heads,
    D=128, 8192 tokens quantized in one kivi_cache_update call per layer (keys per
    channel over 32-token groups, values per token over 32-channel groups)."""
    from intel_kivi_hybrid_b200 import cabi
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    U, S, D, G, R = 8 * 32, 8192, 128, 32, 128
    res = {}
    for name, dtype, eb in (("f32", torch.float32, 4), ("bf16", torch.bfloat16, 2)):
        k, v = make_unit_tensors(8, 32, S, D, 77, dev, dtype)
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
    k, v = make_unit_tensors(8, 8, T, D, 9, dev, torch.bfloat16)
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
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS) + ["cfg4", "ops"])
    ap.add_argument("--path", default="auto", choices=["auto", "fp32", "mma"])
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graph", dest="graph", action="store_false",
                    help="launch every step from Python instead of replaying a CUDA graph (single GPU only)")
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
