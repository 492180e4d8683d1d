"""Benchmark of the sparse-INT4 decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): BASELINE config 1 — 28 stacked layers, each with its own seeded K/V
(fp16, ~N(0,1), four fixed K channels x8), batch 1, 24 query / 8 KV heads, head_dim 128,
32 768 tokens of context in pages of 16 (2048 pages), retention 0.25 + first and last page;
one decode step = for every layer: page scores from the INT4 metadata -> top-k + compact
index -> split-K sparse attention over the selected packed pages.  Data are synthetic.
With N > 1 every rank runs the same workload on its own independent sequence (batch
sharding, no collective in the data path): weak scaling.

Prints ONE JSON line (rank 0).  `value` is tokens/s with the cache resident in HBM and the
step replayed from a CUDA graph; `e2e` is the same step driven through the Python API with
host buffers (H2D of the new token's q/k/v, pack-on-append, attention incl. the tail, D2H of
the outputs inside the timed region); `roofline` is for the attention kernel; `cpu_baseline`
is the CPU oracle port of the same chain on the host cores.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(layers=28, B=1, Hq=24, Hkv=8, D=128, ctx=32768, page=16, retention=0.25, sinks=1, window=1)
PAGE_ATTN_BYTES = 1024 + 512 + 1024 + 64      # K payload, K scale+min rows, V payload, V scale+min


# --------------------------------------------------------------------------- helpers

def seeds(layer):
    base = 1000 * 1 + 10 * layer
    return base, base + 1, base + 2


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# --------------------------------------------------------------------------- CPU oracle arm

def cpu_chain_setup(n_layers, cfg, threads):
    """Seeded inputs for n_layers on the host, quantised by the oracle (not timed)."""
    import numpy as np
    import torch
    import oracle
    oracle.set_num_threads(threads)
    layers = []
    for li in range(n_layers):
        sk, sv, sq = seeds(li)
        K = torch.from_numpy(np.random.default_rng(sk).standard_normal((cfg["B"], cfg["Hkv"], cfg["ctx"], cfg["D"]), dtype=np.float32))
        K[..., [3, 17, 64, 100]] *= 8.0
        V = torch.from_numpy(np.random.default_rng(sv).standard_normal((cfg["B"], cfg["Hkv"], cfg["ctx"], cfg["D"]), dtype=np.float32))
        Q = torch.from_numpy(np.random.default_rng(sq).standard_normal((cfg["B"], cfg["Hq"], 1, cfg["D"]), dtype=np.float32)).half()
        kv = oracle.quantize_k_int4(K.half(), cfg["page"]) + oracle.quantize_v_int4(V.half())
        layers.append((Q, kv))
    return layers


def cpu_chain_step(layers, cfg):
    """One pass of the hot path per layer on the CPU oracle: scores -> select -> compact -> attention."""
    import oracle
    P = cfg["ctx"] // cfg["page"]
    k_max = math.ceil(cfg["retention"] * P)
    bucket = k_max + cfg["sinks"] + cfg["window"]
    for Q, kv in layers:
        s = oracle.page_scores_int4_fast(Q, kv[1], kv[2])
        m = oracle.select_pages_vectorized(s, cfg["retention"], cfg["sinks"], cfg["window"], k_max_static=k_max)
        c = oracle.build_compact_selection(m, bucket)
        oracle.sparse_attn_int4(Q, *kv, selected_page_ids=c, page_size=cfg["page"])


def time_cpu_chain(cfg, sample_layers, reps, threads):
    layers = cpu_chain_setup(sample_layers, cfg, threads)
    cpu_chain_step(layers, cfg)  # warm-up
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        cpu_chain_step(layers, cfg)
        ts.append(time.perf_counter() - t0)
    per_layer = statistics.median(ts) / sample_layers
    return per_layer, ts


def run_reference(args):
    """The reference arm: the CPU port of the reference's eager chain on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = dict(CFG)
    threads = os.cpu_count() or 1
    sample = 2
    layers = cpu_chain_setup(sample, cfg, threads)
    for _ in range(max(args.warmup, 1)):
        cpu_chain_step(layers, cfg)
    ts = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        cpu_chain_step(layers, cfg)
        ts.append(time.perf_counter() - t0)
    per_layer = sum(ts) / len(ts) / sample
    ms_step = per_layer * cfg["layers"] * 1e3
    val = 1e3 / ms_step
    sample_txt = f"{sample} of {cfg['layers']} layers per step (scores+select+compact+attention), time scaled x{cfg['layers'] // sample}"
    print(json.dumps({
        "impl": "reference", "metric": "sparse-INT4 decode tokens/s at 32k ctx", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "config": workload_config(cfg, 1),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample_txt},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(cfg, n_gpus):
    name = "BASELINE config 1" if (cfg["layers"], cfg["B"], cfg["ctx"]) == (CFG["layers"], CFG["B"], CFG["ctx"]) else "variant of BASELINE config 1"
    return {"workload": f"{name}: {cfg['layers']} layers x (page scores -> top-k+compact -> sparse INT4 attention), batch {cfg['B']} per GPU",
            "layers": cfg["layers"], "batch_per_gpu": cfg["B"], "q_heads": cfg["Hq"], "kv_heads": cfg["Hkv"],
            "head_dim": cfg["D"], "context": cfg["ctx"], "page_size": cfg["page"], "retention": cfg["retention"],
            "sinks": cfg["sinks"], "window_pages": cfg["window"], "sharding": f"batch x{n_gpus} (independent sequences)",
            "l2": "inputs larger than L2 (%.2f GB cache)" % (cfg["layers"] * cfg["B"] * cfg["Hkv"] * cfg["ctx"] * (cfg["D"] + 2 * cfg["D"] * 2 // cfg["page"] + 4) / 1e9)}


# --------------------------------------------------------------------------- GPU arm

def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from flashquest_b200 import _lib
    from flashquest_b200.cache.persistent_int4 import PersistentInt4KVCache
    from flashquest_b200.eager.decode_step import QuestDecodeInt4
    _lib.lib()   # fail loudly here if the CUDA library is missing

    cfg = dict(CFG)
    if args.layers:
        cfg["layers"] = args.layers
    if args.ctx:
        cfg["ctx"] = args.ctx
    if args.batch:
        cfg["B"] = args.batch
    Lr, B, Hq, Hkv, D, S, page = cfg["layers"], cfg["B"], cfg["Hq"], cfg["Hkv"], cfg["D"], cfg["ctx"], cfg["page"]
    extra = 256   # room for the tokens appended by the end-to-end run
    cache = PersistentInt4KVCache(batch_size=B, num_layers=Lr, num_kv_heads=Hkv, head_dim=D, max_seq_len=S + extra,
                                  page_size=page, device=dev, dtype=torch.float16)
    qs = []
    for li in range(Lr):
        sk, sv, sq = seeds(li + 100 * rank)
        g = torch.Generator(device=dev)
        K = torch.randn(B, Hkv, S, D, device=dev, generator=g.manual_seed(sk))
        K[..., [3, 17, 64, 100]] *= 8.0
        V = torch.randn(B, Hkv, S, D, device=dev, generator=g.manual_seed(sv))
        cache.update_quantized(K.half(), V.half(), li)           # bulk pack-on-append
        qs.append(torch.randn(B, Hq, 1, D, device=dev, generator=g.manual_seed(sq)).half())
        del K, V
    step = QuestDecodeInt4(cache, num_q_heads=Hq, retention=cfg["retention"], num_sinks=cfg["sinks"],
                           window_pages=cfg["window"], q_dtype=torch.float16, n_split=args.n_split or None)
    Q = torch.stack(qs)       # (L,B,Hq,1,D)

    def one_step():
        for li in range(Lr):
            step.attend(Q[li], li)

    # ---- warm-up (eager), then capture the whole step in a CUDA graph ----
    one_step()
    torch.cuda.synchronize()
    launches_per_step = step.launches
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        one_step()
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        one_step()
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- timed region: K graph replays, CUDA events ----
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        barrier()
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        barrier()
        ms_total = e0.elapsed_time(e1)
        # keep the GPU busy a little longer so the 200 ms sampler sees the loaded clocks
        t_end = time.time() + 0.7
        while time.time() < t_end:
            graph.replay()
        torch.cuda.synchronize()
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = world * B * 1e3 / ms_step
    status = _lib.lib().fq_device_status()

    # ---- roofline of the dominant kernel (attention): back-to-back launches of it alone ----
    from flashquest_b200._lib import check, dtype_code, lib, ptr, stream_ptr
    L = lib()

    def attn_only():
        for li in range(Lr):
            q3 = Q[li].reshape(B, Hq, D)
            Ks, Km, Kp, Vp, Vs, Vm = (cache.K_scale[li], cache.K_mn[li], cache.K_packed[li], cache.V_packed[li],
                                      cache.V_scale[li], cache.V_mn[li])
            comp, O = step.compact[li], step.O[li]
            check(L.fq_sparse_decode_int4(
                ptr(q3), dtype_code(q3), q3.stride(0), q3.stride(1), ptr(Kp), Kp.stride(0), Kp.stride(1),
                ptr(Ks), ptr(Km), Ks.stride(0), Ks.stride(1), Ks.stride(2), ptr(Vp), Vp.stride(0), Vp.stride(1),
                ptr(Vs), ptr(Vm), Vs.stride(0), Vs.stride(1), ptr(comp), comp.stride(0), comp.stride(1), step.bucket,
                None, None, 1, 0, 0, 0, 0, B, Hq, Hkv, S, S // page, D, page, step.sm_scale,
                ptr(O), O.stride(0), O.stride(1), ptr(step.lse[li]), ptr(step.workspace[li]), step.workspace.shape[1],
                step.n_split, stream_ptr(dev)))
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2, capture_error_mode="thread_local"):
        attn_only()
    for _ in range(3):
        g2.replay()
    torch.cuda.synchronize()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for _ in range(args.steps):
        g2.replay()
    a1.record()
    torch.cuda.synchronize()
    attn_us = a0.elapsed_time(a1) * 1e3 / (args.steps * Lr)
    # algorithmic bytes: union over the query heads of a KV group of the selected pages
    n_rep = Hq // Hkv
    P = S // page
    union_pages = per_head_pages = 0
    for li in range(Lr):
        ids = step.compact[li].long()                                 # (B,Hq,bucket)
        m = torch.zeros(B, Hq, P + 1, dtype=torch.bool, device=dev)
        m.scatter_(2, torch.where(ids >= 0, ids, torch.full_like(ids, P)), True)
        m = m[:, :, :P]
        per_head_pages += int(m.sum())
        union_pages += int(m.view(B, Hkv, n_rep, P).any(dim=2).sum())
    alg_bytes = union_pages * PAGE_ATTN_BYTES / Lr
    peak, peak_kind = measured_peak()
    achieved = alg_bytes / (attn_us * 1e-6) / 1e9
    # DRAM bytes per launch from the committed ncu summary (config 1 only)
    traffic = None
    if (Lr, B, S) == (CFG["layers"], CFG["B"], CFG["ctx"]) or args.layers:
        try:
            with open(os.path.join(ROOT, "profiles", "sparse_decode_int4_config1.md")) as f:
                mt = re.search(r"dram_bytes_per_launch:\s*(\d+)", f.read())
            traffic = int(mt.group(1)) if mt and B == CFG["B"] and S == CFG["ctx"] else None
        except OSError:
            pass
    roofline = {"bound": "hbm", "kernel": "sparse_decode_int4_kernel", "achieved": achieved, "peak": peak,
                "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                "algorithmic_bytes_per_launch": alg_bytes, "per_head_bytes_per_launch": per_head_pages * PAGE_ATTN_BYTES / Lr,
                "avg_launch_us": attn_us, "frac_of_8TBs": achieved / 8000.0}

    # ---- end to end through the Python API with host buffers ----
    e2e = run_e2e(torch, dist, world, dev, cache, step, cfg, args, barrier)

    # ---- the attention kernel at batched shapes (rank 0, N = 1, default workload only) ----
    batched = None
    if rank == 0 and world == 1 and not (args.layers or args.ctx or args.batch) and not args.no_batched:
        del graph, g2
        cache = step = None
        torch.cuda.empty_cache()
        batched = [attention_batched(torch, dev, bn, 10) for bn in (16, 64)]

    # ---- CPU baseline (rank 0, N = 1 only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        per_layer, ts = time_cpu_chain(dict(CFG), 2, 3, threads)
        cpu = {"value": 1.0 / (per_layer * CFG["layers"]), "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"2 of 28 layers x 3 repetitions of scores+select+compact+attention on the C oracle, scaled to 28 layers"}

    if rank == 0:
        print(json.dumps({
            "metric": "sparse-INT4 decode tokens/s at 32k ctx", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(cfg, world), "clocks": clk.summary(), "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps, "roofline": roofline, "attention_batched": batched,
            "cpu_baseline": cpu,
            "device_status": status,
        }))
    if world > 1:
        dist.destroy_process_group()


def attention_batched(torch, dev, Bn, steps):
    """Attention launch alone at batch Bn (one layer, 32k context each, same selection rule):
    the shape where the bytes, not the launch chain, set the time."""
    from flashquest_b200.eager.criticality import page_scores_int4_fast
    from flashquest_b200.eager.selection import select_pages_compact
    from flashquest_b200.kernel.kv_quant import quantize_k_int4, quantize_v_int4
    from flashquest_b200.kernel.sparse_int4_fwd_compact import flash_attn_sparse_int4_fwd_compact
    Hq, Hkv, D, S, page = CFG["Hq"], CFG["Hkv"], CFG["D"], CFG["ctx"], CFG["page"]
    g = torch.Generator(device=dev).manual_seed(4242)
    parts = []
    for _ in range(Bn):                       # one sequence at a time keeps the fp32 source small
        K = torch.randn(1, Hkv, S, D, device=dev, generator=g)
        K[..., [3, 17, 64, 100]] *= 8.0
        V = torch.randn(1, Hkv, S, D, device=dev, generator=g)
        parts.append(quantize_k_int4(K.half(), page) + quantize_v_int4(V.half()))
        del K, V
    kv = tuple(torch.cat([x[i] for x in parts]) for i in range(6))
    del parts
    Q = torch.randn(Bn, Hq, 1, D, device=dev, generator=g).half()
    k_max = int(CFG["retention"] * (S // page))
    bucket = k_max + CFG["sinks"] + CFG["window"]
    comp = select_pages_compact(page_scores_int4_fast(Q, kv[1], kv[2]), CFG["retention"], CFG["sinks"], CFG["window"],
                                k_max_static=k_max, BUCKET_MAX=bucket)

    def run():
        return flash_attn_sparse_int4_fwd_compact(Q, *kv, selected_page_ids=comp, page_size=page)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / steps
    ids = comp.reshape(Bn, Hq, -1).long()
    P = S // page
    m = torch.zeros(Bn, Hq, P + 1, dtype=torch.bool, device=dev)
    m.scatter_(2, torch.where(ids >= 0, ids, torch.full_like(ids, P)), True)
    m = m[:, :, :P]
    per_head = int(m.sum()) * PAGE_ATTN_BYTES
    union = int(m.view(Bn, Hkv, Hq // Hkv, P).any(dim=2).sum()) * PAGE_ATTN_BYTES
    peak, _ = measured_peak()
    return {"batch": Bn, "avg_launch_us": us, "union_bytes": union, "per_head_bytes": per_head,
            "GBs_union": union / us / 1e3, "GBs_per_head": per_head / us / 1e3,
            "frac_union": union / us / 1e3 / peak, "frac_per_head": per_head / us / 1e3 / peak}


def run_e2e(torch, dist, world, dev, cache, step, cfg, args, barrier):
    """Per step and layer: pinned host q/k/v of the new token -> device, pack-on-append,
    score/select/attend incl. the staged tail; one D2H read of all layers' outputs."""
    Lr, B, Hq, Hkv, D = cfg["layers"], cfg["B"], cfg["Hq"], cfg["Hkv"], cfg["D"]
    n = args.steps + max(args.warmup, 3)
    g = torch.Generator().manual_seed(7)
    hq = torch.randn(n, Lr, B, Hq, 1, D, generator=g).half().pin_memory()
    hk = torch.randn(n, Lr, B, Hkv, 1, D, generator=g).half().pin_memory()
    hv = torch.randn(n, Lr, B, Hkv, 1, D, generator=g).half().pin_memory()
    out_host = torch.empty(Lr, B, Hq, D, dtype=torch.float16).pin_memory()
    dq = torch.empty(Lr, B, Hq, 1, D, dtype=torch.float16, device=dev)
    dk = torch.empty(Lr, B, Hkv, 1, D, dtype=torch.float16, device=dev)
    dv = torch.empty(Lr, B, Hkv, 1, D, dtype=torch.float16, device=dev)

    # one CUDA graph per step: H2D copies of the step's q/k/v from pinned staging buffers, the 28-layer
    # step (sequence length read on the device), D2H copy of the outputs
    sq, sk, sv = (torch.empty_like(t[0]).pin_memory() for t in (hq, hk, hv))

    def h2d():
        dq.copy_(sq, non_blocking=True)
        dk.copy_(sk, non_blocking=True)
        dv.copy_(sv, non_blocking=True)

    replay = step.capture_step_graph(dk, dv, dq, before=h2d, after=lambda: out_host.copy_(step.O, non_blocking=True))

    def one(i):
        sq.copy_(hq[i]); sk.copy_(hk[i]); sv.copy_(hv[i])          # this step's inputs into the pinned staging buffers
        replay()
        torch.cuda.current_stream().synchronize()

    w = max(args.warmup, 3)
    for i in range(w):
        one(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(w, n):
        one(i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    h2d = hq[0].numel() * 2 + hk[0].numel() * 2 + hv[0].numel() * 2
    return {"value": world * B * 1e3 / (ms / args.steps), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": ms / args.steps,
            "path": "pinned host q/k/v -> one CUDA graph (H2D copies, fq_decode_step_int4_dev: append+score+select+attend per layer, D2H of O) -> host O"}



# --------------------------------------------------------------------------- secondary workload: AWQ GEMV

def run_awq(args):
    """AWQ W4A16 GEMV on the Llama-3.2-3B projection shapes (BASELINE config 3's linears): a CUDA
    graph of 28 launches over 28 distinct seeded weight sets (1.5 GB, nothing served from L2)."""
    import torch
    from flashquest_b200 import _lib
    from flashquest_b200.kernel.fused_proj import awq_gemv_fused
    from flashquest_b200.quant import AWQLinear
    _lib.lib()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    layers, group = 28, 128
    peak, peak_kind = measured_peak()

    def linear(K, N, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), dtype=torch.int32, device=dev, generator=g)
        qz = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // group, N // 8), dtype=torch.int32, device=dev, generator=g)
        sc = (torch.rand(K // group, N, device=dev, generator=g) * 0.019 + 0.001).half()
        return AWQLinear(qw, sc, qz, group_size=group)

    rows = []
    for name, K, Ns in (("qkv", 3072, (3072, 1024, 1024)), ("gate_up", 3072, (8192, 8192)),
                        ("down", 8192, (3072,)), ("o", 3072, (3072,))):
        for M in (1, 4, 8):
            projs = [[linear(K, N, 7 * li + i) for i, N in enumerate(Ns)] for li in range(layers)]
            x = torch.randn(1, M, K, device=dev).half()
            for pj in projs:
                awq_gemv_fused(x, pj)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                for pj in projs:
                    awq_gemv_fused(x, pj)
            for _ in range(max(args.warmup, 3)):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (args.steps * layers)
            nbytes = sum(K * N // 2 + (K // group) * N * 2 + (K // group) * N // 2 for N in Ns)
            rows.append({"proj": name, "M": M, "us_per_launch": round(us, 2), "bytes": nbytes,
                         "GBs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / peak, 3)})
            del projs, g
    print(json.dumps({"metric": "AWQ W4A16 GEMV weight bytes per second", "unit": "GB/s", "workload": "awq",
                      "peak": peak, "peak_kind": peak_kind, "steps": args.steps, "rows": rows,
                      "device_status": _lib.lib().fq_device_status()}))


# --------------------------------------------------------------------------- secondary workload: TurboQuant

def run_turbo(args):
    """BASELINE config 2: TurboQuant K3-V3, context 32k, batch 16 (overridable), 24/8 heads, D 128,
    retention 0.25: pack-on-append throughput of a bulk append and the sparse decode attention."""
    import torch
    from flashquest_b200 import _lib
    from flashquest_b200.eager.criticality import page_scores_int4_fast
    from flashquest_b200.eager.selection import select_pages_vectorized
    from flashquest_b200.kernel.kv_quant import quantize_k_turbo, quantize_v_turbo
    from flashquest_b200.kernel.sparse_turbo_fwd import flash_attn_sparse_turbo_fwd
    _lib.lib()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, Hq, Hkv, D, S, page = args.batch or 16, 24, 8, 128, args.ctx or 32768, 16
    peak, peak_kind = measured_peak()
    g = torch.Generator(device=dev).manual_seed(11)

    def heavy(shape):            # N(0,1) with Student-t (df 3) outliers on 8 of the 128 channels
        x = torch.randn(shape, device=dev, generator=g)
        t = torch.randn(shape[:-1] + (8,), device=dev, generator=g)
        chi = torch.randn(shape[:-1] + (8, 3), device=dev, generator=g).pow(2).sum(-1).div(3).sqrt()
        x[..., [3, 17, 29, 41, 64, 77, 100, 119]] = t / chi
        return x.half()

    kv, times = [], []
    for b in range(B):           # one sequence at a time keeps the fp16 source small
        K, V = heavy((1, Hkv, S, D)), heavy((1, Hkv, S, D))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        qk = quantize_k_turbo(K, page)
        qv = quantize_v_turbo(V)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        kv.append(qk + qv)
        del K, V
    pack_ms = statistics.median(times[1:] or times)
    in_bytes = 2 * Hkv * S * D * 2
    out_bytes = 2 * Hkv * S * (D // 8 + D // 4 + 2) + 2 * Hkv * (S // page) * D * 2
    cat = [torch.cat([k[i] for k in kv]) for i in range(8)]
    del kv
    K_msb, K_lsb, K_st, K_sr, K_mr, V_msb, V_lsb, V_st = cat
    Q = torch.randn(B, Hq, 1, D, device=dev, generator=g).half()
    mask = select_pages_vectorized(page_scores_int4_fast(Q, K_sr, K_mr), 0.25, 1, 1)

    def attend():
        return flash_attn_sparse_turbo_fwd(Q, K_msb, K_lsb, K_st, V_msb, V_lsb, V_st, selection_mask=mask, page_size=page)

    for _ in range(max(args.warmup, 3)):
        attend()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        attend()
    e1.record()
    torch.cuda.synchronize()
    attn_us = e0.elapsed_time(e1) * 1e3 / args.steps
    per_tok = 2 * (D // 8 + D // 4 + 2)
    n_rep = Hq // Hkv
    per_head = int(mask.sum()) * page * per_tok
    union = int(mask.view(B, Hkv, n_rep, -1).any(2).sum()) * page * per_tok
    print(json.dumps({
        "metric": "TurboQuant K3-V3: pack-on-append and sparse decode attention", "workload": "turbo",
        "config": {"batch": B, "q_heads": Hq, "kv_heads": Hkv, "head_dim": D, "context": S, "page_size": page, "retention": 0.25},
        "pack": {"ms_per_sequence": pack_ms, "tokens_per_s": S / (pack_ms * 1e-3), "GBs": (in_bytes + out_bytes) / (pack_ms * 1e-3) / 1e9,
                 "frac": (in_bytes + out_bytes) / (pack_ms * 1e-3) / 1e9 / peak,
                 "what": "quantize_k_turbo (planes + scales + page metadata) and quantize_v_turbo of one 32k sequence"},
        "attention": {"us_per_call": attn_us, "union_bytes": union, "per_head_bytes": per_head,
                      "GBs_union": union / attn_us / 1e3, "frac": union / attn_us / 1e3 / peak,
                      "what": "flash_attn_sparse_turbo_fwd: WHT of Q, compact list, attention, inverse WHT (4 launches)"},
        "peak": peak, "peak_kind": peak_kind, "device_status": _lib.lib().fq_device_status()}))


# --------------------------------------------------------------------------- secondary workload: Llama decode

def run_llama(args):
    """BASELINE config 3 shape: random-init Llama-3.2-3B architecture with AWQ 4-bit weights, greedy
    decode with the cache already holding 32 768 tokens per layer.  The cache is filled with seeded
    synthetic K/V (the prefill path is not built), then `steps` decode steps are timed end to end:
    embedding gather, 28 x (norms, AWQ GEMVs, RoPE, append + sparse attention, SwiGLU), lm_head, argmax."""
    import torch
    from flashquest_b200 import _lib
    from flashquest_b200.eager.llama_decode import LlamaConfig, LlamaInt4Decoder, random_llama_weights
    _lib.lib()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    cfg = LlamaConfig()
    if args.layers:
        cfg.layers = args.layers
    S = args.ctx or 32768
    w = random_llama_weights(cfg, dev, seed=3)
    dec = LlamaInt4Decoder(cfg, w, batch_size=1, max_seq_len=S + 256, page_size=16, retention=0.25, num_sinks=1, window_pages=1,
                           device=dev)
    g = torch.Generator(device=dev)
    for li in range(cfg.layers):
        K = torch.randn(1, cfg.kv_heads, S, cfg.head_dim, device=dev, generator=g.manual_seed(2 * li))
        K[..., [3, 17, 64, 100]] *= 8.0
        V = torch.randn(1, cfg.kv_heads, S, cfg.head_dim, device=dev, generator=g.manual_seed(2 * li + 1))
        dec.cache.update_quantized(K.half(), V.half(), li)
        del K, V
    ids = torch.tensor([1], dtype=torch.int32, device=dev)
    for _ in range(2):
        ids = dec.decode_step(ids).clone()                     # stream steps (one foreign call each)
    replay = dec.capture_decode_graph(ids)                     # then one CUDA graph replayed per token
    for _ in range(max(args.warmup, 3)):
        replay()
    torch.cuda.synchronize()
    l0 = dec.launches + dec.attn.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index or 0) as clk:
        e0.record()
        for _ in range(args.steps):
            replay()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    wbytes = cfg.layers * sum(K * N // 2 + (K // 128) * N * 2 + (K // 128) * N // 2 for K, N in
                              ((cfg.hidden, (cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim), (cfg.q_heads * cfg.head_dim, cfg.hidden),
                               (cfg.hidden, 2 * cfg.ffn), (cfg.ffn, cfg.hidden))) + cfg.vocab * cfg.hidden * 2
    print(json.dumps({
        "metric": "Llama-3.2-3B-shaped AWQ decode tokens/s at 32k ctx (sparse INT4 attention)", "workload": "llama",
        "value": 1e3 / ms, "unit": "tokens/s", "ms_per_token": ms, "steps": args.steps,
        "config": {"hidden": cfg.hidden, "layers": cfg.layers, "q_heads": cfg.q_heads, "kv_heads": cfg.kv_heads, "head_dim": cfg.head_dim,
                   "ffn": cfg.ffn, "vocab": cfg.vocab, "context": S, "retention": 0.25, "weights": "random-init AWQ 4-bit, group 128",
                   "cache": "synthetic K/V (prefill not built)"},
        "weight_bytes_per_token": wbytes, "weight_GBs": wbytes / ms / 1e6,
        "gpu_launches": dec.launches + dec.attn.launches - l0, "clocks": clk.summary(),
        "device_status": _lib.lib().fq_device_status()}))


# --------------------------------------------------------------------------- secondary workload: context split

def run_ctxsplit(args):
    """One very long sequence split by page range over the ranks (torchrun, N >= 2): per decode step
    local scores -> all-gather of top-k candidates -> global top-k -> local sparse attention ->
    all-gather of (O, lse) -> LSE merge.  Reports the step time (max over ranks, CUDA events) and the
    share spent in the two exchanges."""
    import torch
    import torch.distributed as dist
    from flashquest_b200 import _lib
    from flashquest_b200.eager import context_split as cs
    from flashquest_b200.kernel.kv_quant import quantize_k_int4, quantize_v_int4
    _lib.lib()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world < 2:
        if rank == 0:
            print(json.dumps({"workload": "ctxsplit", "unavailable": "needs torchrun with at least 2 ranks"}))
        return
    dist.init_process_group("nccl", device_id=dev)
    Hq, Hkv, D, page = CFG["Hq"], CFG["Hkv"], CFG["D"], CFG["page"]
    S = args.ctx or 524288                     # the whole sequence
    P = S // page
    lo, hi = cs.page_range(rank, world, P)
    g = torch.Generator(device=dev).manual_seed(900 + rank)
    n_tok = (hi - lo) * page
    K = torch.randn(1, Hkv, n_tok, D, device=dev, generator=g)
    K[..., [3, 17, 64, 100]] *= 8.0
    V = torch.randn(1, Hkv, n_tok, D, device=dev, generator=g)
    kv = quantize_k_int4(K.half(), page) + quantize_v_int4(V.half())
    del K, V
    q = torch.randn(1, Hq, 1, D, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).half()   # same on every rank
    kw = dict(P_global=P, page_size=page, retention=CFG["retention"], num_sinks=CFG["sinks"], window_pages=CFG["window"])

    def step(timings=None):
        return cs.decode_context_split_int4(q, kv[0], kv[1], kv[2], kv[3], kv[4], kv[5], timings=timings, **kw)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    tm = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(tm)
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = e0.elapsed_time(e1) / args.steps
    seg = lambda a, b: sum(x.elapsed_time(y) for x, y in zip(tm[a], tm[b])) / args.steps
    parts = torch.tensor([ms, seg("start", "scored"), seg("scored", "selected"), seg("selected", "attended"),
                          seg("attended", "merged")], device=dev)
    dist.all_reduce(parts, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms, t_sc, t_sel, t_att, t_mrg = [float(x) for x in parts]
        print(json.dumps({
            "metric": "context-split sparse INT4 decode, one layer-step of one sequence", "workload": "ctxsplit", "n_gpus": world,
            "config": {"context": S, "pages": P, "pages_per_rank": hi - lo, "q_heads": Hq, "kv_heads": Hkv, "head_dim": D,
                       "page_size": page, "retention": CFG["retention"]},
            "ms_per_layer_step": ms, "steps": args.steps,
            "phases_ms_max_over_ranks": {"local_scores": t_sc, "global_topk_incl_candidate_allgather": t_sel,
                                         "compact_and_local_attention": t_att, "o_lse_allgather_and_merge": t_mrg},
            "device_status": _lib.lib().fq_device_status()}))
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (small captures)")
    ap.add_argument("--ctx", type=int, default=0, help="override the context length (small captures)")
    ap.add_argument("--batch", type=int, default=0, help="override the batch per GPU (profiles of batched shapes)")
    ap.add_argument("--n-split", type=int, default=0, help="override the split-K factor of the attention kernel")
    ap.add_argument("--workload", default="decode", choices=["decode", "awq", "turbo", "llama", "ctxsplit"],
                    help="decode = the headline metric; awq = secondary table for the W4A16 GEMV (1 GPU)")
    ap.add_argument("--no-batched", action="store_true", help="skip the batched-attention leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "awq":
        run_awq(args)
    elif args.workload == "turbo":
        run_turbo(args)
    elif args.workload == "llama":
        run_llama(args)
    elif args.workload == "ctxsplit":
        run_ctxsplit(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
