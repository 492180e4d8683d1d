"""Benchmark of the sparse-INT4 decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): BASELINE config 1 — 28 stacked layers, each with its own seeded K/V
(fp16, ~N(0,1), four fixed K channels x8), batch 1, 24 query / 8 KV heads, head_dim 128,
32 768 tokens of context in pages of 16 (2048 pages), retention 0.25 + first and last page;
one decode step = for every layer: page scores from the INT4 metadata -> top-k + compact
index -> split-K sparse attention over the selected packed pages.  Data are synthetic.
With N > 1 every rank runs the same workload on its own independent sequence (batch
sharding, no collective in the data path): weak scaling.  The same line also carries, as extra
keys, BASELINE config 4 (64 sequences x 128k context, retention 0.125, batch-sharded over the
ranks, in waves where a rank's share does not fit its HBM; for N >= 2 one 512k sequence split by
page range with two all-gathers per layer-step) and, at N = 1, the secondary workloads.

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


CPU_SAMPLE_LAYERS = 7      # of 28: the bounded sample of the CPU arm (time scales linearly, layers are independent)


def time_cpu_chain(layers, cfg, reps, threads):
    import oracle
    oracle.set_num_threads(threads)
    cpu_chain_step(layers, cfg)  # warm-up
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        cpu_chain_step(layers, cfg)
        ts.append(time.perf_counter() - t0)
    return statistics.median(ts) / len(layers), ts


def cpu_baseline_leg():
    """The CPU port of the reference's eager chain (C, OpenMP) on the host cores: 7 of the 28 layers,
    with all cores and with one thread."""
    cfg = dict(CFG)
    threads = os.cpu_count() or 1
    layers = cpu_chain_setup(CPU_SAMPLE_LAYERS, cfg, threads)
    per_layer, _ = time_cpu_chain(layers, cfg, 3, threads)
    per_layer_1, _ = time_cpu_chain(layers[:2], cfg, 1, 1)
    return {"value": 1.0 / (per_layer * cfg["layers"]), "unit": "tokens/s", "cores": threads, "kind": "port",
            "single_thread_value": 1.0 / (per_layer_1 * cfg["layers"]),
            "sample": f"{CPU_SAMPLE_LAYERS} of {cfg['layers']} layers x 3 repetitions (median) of scores+select+compact+attention on the C "
                      f"port of the reference's eager chain, all {threads} host threads, scaled x{cfg['layers'] // CPU_SAMPLE_LAYERS}; "
                      "single_thread_value: 2 layers, 1 thread, scaled x14",
            "why_port": "the reference is Python over torch and its source tree is not on the GPU box; its arithmetic is restated in C "
                        "and pinned against the reference's outputs (tests/golden)"}


def run_reference(args):
    """The reference arm: the CPU port of the reference's eager chain on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = dict(CFG)
    threads = os.cpu_count() or 1
    sample = CPU_SAMPLE_LAYERS
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
    sample_txt = (f"{sample} of {cfg['layers']} layers per step (scores+select+compact+attention), all {threads} host threads, "
                  f"time scaled x{cfg['layers'] // sample}")
    print(json.dumps({
        "impl": "reference", "metric": "sparse-INT4 decode tokens/s at 32k ctx", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 codes, bf16 metadata, f16 q; f64 accumulation", "data": "synthetic", "config": workload_config(cfg, 1),
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
        # the collectives here move kilobytes; in-switch reduction buys nothing and a rank that dies while bound
        # to an NVLink multicast object can fault its peers
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
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

    # ---- timed region: blocks of exactly K graph replays between barriers, CUDA events; the block is repeated
    #      until at least 0.5 s have been timed (and at least 5 blocks) and the MEDIAN block is reported ----
    blocks = []
    with ClockSampler(local) as clk:
        t_start = time.time()
        while len(blocks) < 5 or (sum(blocks) < 500.0 and len(blocks) < 400):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record()
            for _ in range(args.steps):
                graph.replay()
            e1.record()
            barrier()
            ms_block = e0.elapsed_time(e1)
            if world > 1:                     # every rank keeps the max over ranks: same loop length everywhere
                t = torch.tensor([ms_block], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms_block = float(t.item())
            blocks.append(ms_block)
        # keep the GPU busy a little longer if the sampler has seen less than 0.7 s of load
        t_end = t_start + 0.9
        while time.time() < t_end:
            graph.replay()
        torch.cuda.synchronize()
    ms_total = statistics.median(blocks)
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
                "traffic_source": "ncu capture of the same workload, profiles/sparse_decode_int4_config1.md (not measured in this run)",
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
        torch.cuda.empty_cache()

    default_workload = not (args.layers or args.ctx or args.batch)
    if not default_workload or args.no_extra:
        config4 = ctxsplit = secondary = None
    else:
        # everything of the headline leg is released first: config 4 needs the HBM
        try:
            del graph, g2
        except NameError:
            pass
        cache = step = None
        torch.cuda.empty_cache()
        config4 = run_config4(torch, dist, world, rank, dev, args)
        ctxsplit = run_ctxsplit_leg(torch, dist, world, rank, dev, args) if world > 1 else None
        secondary = None
        if rank == 0 and world == 1 and not args.no_secondary:
            secondary = {}
            for name, fn in (("awq", run_awq), ("turbo", run_turbo), ("int8", run_int8), ("prefill_attn", run_prefill_attn), ("llama", run_llama)):
                torch.cuda.empty_cache()
                try:
                    secondary[name] = fn(args)
                except Exception as e:                      # a secondary table must not take the headline down
                    secondary[name] = {"error": f"{type(e).__name__}: {e}"}
            torch.cuda.empty_cache()

    # ---- CPU baseline (rank 0, N = 1 only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline_leg()

    if rank == 0:
        print(json.dumps({
            "metric": "sparse-INT4 decode tokens/s at 32k ctx", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int4 codes, bf16 metadata, f16 q; f32 arithmetic", "data": "synthetic",
            "config": workload_config(cfg, world), "clocks": clk.summary(), "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps, "roofline": roofline, "attention_batched": batched,
            "cpu_baseline": cpu,
            "timing": {"blocks": len(blocks), "steps_per_block": args.steps, "reported": "median block",
                       "timed_region_s": sum(blocks) / 1e3, "block_ms_min": min(blocks), "block_ms_max": max(blocks)},
            "config4_batch_sharded": config4, "context_split": ctxsplit, "secondary": secondary,
            "device_status": status,
        }))
    if world > 1:
        dist.destroy_process_group()


def fill_cache_random(torch, cache, li, b, seed, S):
    """Seeded K/V of BASELINE's distribution for one (layer, sequence), packed straight into the cache storage."""
    from flashquest_b200.kernel.kv_quant import quantize_kv_int4_into
    dev = cache.K_packed.device
    Hkv, D = cache.num_kv_heads, cache.head_dim
    g = torch.Generator(device=dev).manual_seed(seed)
    K = torch.randn(1, Hkv, S, D, device=dev, generator=g)
    K[..., [3, 17, 64, 100]] *= 8.0
    K = K.half()
    V = torch.randn(1, Hkv, S, D, device=dev, generator=g).half()
    quantize_kv_int4_into(K, V, cache.page_size, S,
                          K_packed=cache.K_packed[li, b:b + 1], K_scale=cache.K_scale[li, b:b + 1], K_mn=cache.K_mn[li, b:b + 1],
                          V_packed=cache.V_packed[li, b:b + 1], V_scale=cache.V_scale[li, b:b + 1], V_mn=cache.V_mn[li, b:b + 1])


def selected_bytes(torch, compact, Hkv, P):
    """(union bytes over the GQA groups, per-head bytes) of the pages a compact list (B,Hq,bucket) names."""
    B, Hq = compact.shape[0], compact.shape[1]
    ids = compact.reshape(B, Hq, -1).long()
    m = torch.zeros(B, Hq, P + 1, dtype=torch.bool, device=compact.device)
    m.scatter_(2, torch.where(ids >= 0, ids, torch.full_like(ids, P)), True)
    m = m[:, :, :P]
    return int(m.view(B, Hkv, Hq // Hkv, P).any(dim=2).sum()) * PAGE_ATTN_BYTES, int(m.sum()) * PAGE_ATTN_BYTES


def run_config4(torch, dist, world, rank, dev, args):
    """BASELINE config 4, batch-sharded leg: 64 independent sequences of 128k context, 28 layers each with its own
    seeded K/V, retention 0.125 (+ first and last page), batch-sharded over the ranks with no collective in the data
    path.  A rank's share (64 / N sequences x 4.8 GB) is processed in waves of at most 16 sequences where it does
    not fit the HBM; the step time of a rank is the sum over its waves, the job's time the max over the ranks."""
    from flashquest_b200.cache.persistent_int4 import PersistentInt4KVCache
    from flashquest_b200.eager.decode_step import QuestDecodeInt4
    total, S, page, Lr, Hq, Hkv, D, r = 64, 131072, 16, CFG["layers"], CFG["Hq"], CFG["Hkv"], CFG["D"], 0.125
    if total % world != 0:
        return {"unavailable": f"64 sequences do not divide over {world} ranks"}
    per_rank = total // world
    wave_B = min(per_rank, 16)
    n_waves = per_rank // wave_B
    steps = max(3, min(args.steps, 10))
    P = S // page
    ms_waves, attn_us, union_b, head_b = [], [], 0, 0
    for w in range(n_waves):
        cache = PersistentInt4KVCache(batch_size=wave_B, num_layers=Lr, num_kv_heads=Hkv, head_dim=D, max_seq_len=S,
                                      page_size=page, device=dev, dtype=torch.float16)
        for li in range(Lr):
            for b in range(wave_B):
                seq = rank * per_rank + w * wave_B + b
                fill_cache_random(torch, cache, li, b, 4_000_000 + 100 * seq + li, S)
            cache._seen_tokens[li] = S
        step = QuestDecodeInt4(cache, num_q_heads=Hq, retention=r, num_sinks=1, window_pages=1, q_dtype=torch.float16)
        g = torch.Generator(device=dev).manual_seed(77 + rank * 10 + w)
        Q = torch.randn(Lr, wave_B, Hq, 1, D, device=dev, generator=g).half()

        def one_step():
            for li in range(Lr):
                step.attend(Q[li], li)
        one_step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            one_step()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms_waves.append(e0.elapsed_time(e1) / steps)
        if w == 0 and rank == 0:          # the attention kernel alone on this shape, for the roofline fraction
            from flashquest_b200.kernel.sparse_int4_fwd_compact import flash_attn_sparse_int4_fwd_compact
            v = cache.get_views(0)
            comp = step.compact[0].unsqueeze(2)
            run = lambda: flash_attn_sparse_int4_fwd_compact(Q[0], v["K_packed"], v["K_scale"], v["K_mn"], v["V_packed"], v["V_scale"],
                                                             v["V_mn"], selected_page_ids=comp, page_size=page)
            for _ in range(3):
                run()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(5):
                run()
            a1.record()
            torch.cuda.synchronize()
            attn_us.append(a0.elapsed_time(a1) * 1e3 / 5)
            union_b, head_b = selected_bytes(torch, step.compact[0], Hkv, P)
        del graph, step, cache, Q
        torch.cuda.empty_cache()
    ms = sum(ms_waves)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    peak, _ = measured_peak()
    out = {"workload": "BASELINE config 4, batch-sharded: 64 sequences x 131072 tokens, 28 layers x (scores -> top-k+compact -> sparse "
                       "INT4 attention), retention 0.125 + first and last page, page 16",
           "sequences_per_gpu": per_rank, "waves_per_gpu": n_waves, "sequences_per_wave": wave_B,
           "why_waves": "one sequence is 4.8 GB of packed KV and metadata over 28 layers (308 GB for 64)",
           "ms_per_step_all_sequences": ms, "value": total * 1e3 / ms, "unit": "tokens/s", "steps": steps,
           "timing": "CUDA events around graph replays of each wave, summed over the waves, max over ranks"}
    if attn_us:
        out["attention_one_layer"] = {"batch": wave_B, "avg_launch_us": attn_us[0], "union_bytes": union_b, "per_head_bytes": head_b,
                                      "GBs_union": union_b / attn_us[0] / 1e3, "frac_union": union_b / attn_us[0] / 1e3 / peak,
                                      "frac_per_head": head_b / attn_us[0] / 1e3 / peak}
    return out


def run_ctxsplit_leg(torch, dist, world, rank, dev, args):
    """BASELINE config 4, context-split leg: ONE sequence of 524 288 tokens split over the ranks by page range; one
    layer-step = local scores -> candidate all-gather -> global top-k -> local sparse attention -> (O, lse) all-gather
    -> LSE merge, replayed from one CUDA graph (collectives included).  Also a smaller sequence that one GPU holds,
    where the split result is compared with the single-GPU result."""
    from flashquest_b200.eager import context_split as cs
    from flashquest_b200.eager.criticality import page_scores_int4_fast
    from flashquest_b200.eager.selection import select_pages_compact
    from flashquest_b200.kernel.kv_quant import quantize_k_int4, quantize_v_int4
    from flashquest_b200.kernel.sparse_int4_fwd_compact import flash_attn_sparse_int4_fwd_compact
    Hq, Hkv, D, page, r = CFG["Hq"], CFG["Hkv"], CFG["D"], CFG["page"], 0.125
    out = {}

    def local_kv(seed, n_tok):
        g = torch.Generator(device=dev).manual_seed(seed)
        K = torch.randn(1, Hkv, n_tok, D, device=dev, generator=g)
        K[..., [3, 17, 64, 100]] *= 8.0
        V = torch.randn(1, Hkv, n_tok, D, device=dev, generator=g)
        return quantize_k_int4(K.half(), page) + quantize_v_int4(V.half())

    # ---- (a) agreement with one GPU on a 64k-token sequence (every rank builds the whole sequence from one seed) ----
    S0 = 65536
    P0 = S0 // page
    kv = local_kv(4242, S0)
    q = torch.randn(1, Hq, 1, D, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).half()
    k0 = cs.global_k(r, P0)
    comp, mask = select_pages_compact(page_scores_int4_fast(q, kv[1], kv[2]), r, 1, 1, k_max_static=k0, BUCKET_MAX=k0 + 2, return_mask=True)
    O_ref, lse_ref = flash_attn_sparse_int4_fwd_compact(q, *kv, selected_page_ids=comp, page_size=page)
    lo, hi = cs.page_range(rank, world, P0)
    sl = slice(lo * page, hi * page)
    dec = cs.ContextSplitInt4(batch_size=1, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D, page_size=page, P_global=P0, retention=r,
                              num_sinks=1, window_pages=1, q_dtype=torch.float16, device=dev)
    loc = (q, kv[0][:, :, sl].contiguous(), kv[1][:, :, lo:hi].contiguous(), kv[2][:, :, lo:hi].contiguous(),
           kv[3][:, :, sl].contiguous(), kv[4][:, :, sl].contiguous(), kv[5][:, :, sl].contiguous())
    O, lse = dec.step(*loc)
    torch.cuda.synchronize()
    chk = torch.tensor([(O.float() - O_ref.float()).abs().max().item(), (lse - lse_ref).abs().max().item(),
                        0.0 if torch.equal(dec.local_mask(), mask[..., lo:hi]) else 1.0], device=dev)
    dist.all_reduce(chk, op=dist.ReduceOp.MAX)
    out["agreement_with_one_gpu"] = {"context": S0, "max_abs_dO": float(chk[0]), "max_abs_dLSE": float(chk[1]),
                                     "page_sets_equal_on_every_rank": bool(chk[2] == 0)}
    del kv, dec, loc, comp, mask
    torch.cuda.empty_cache()

    # ---- (b) the 512k sequence ----
    S = 524288
    P = S // page
    lo, hi = cs.page_range(rank, world, P)
    kv = local_kv(900 + rank, (hi - lo) * page)
    dec = cs.ContextSplitInt4(batch_size=1, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D, page_size=page, P_global=P, retention=r,
                              num_sinks=1, window_pages=1, q_dtype=torch.float16, device=dev)
    steps = max(5, args.steps)
    # phases apart, stream-launched (the events sit between the phases)
    tm = {}

    def mark(name):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        tm.setdefault(name, []).append(ev)
    for _ in range(3):
        dec.step(q, *kv)
    torch.cuda.synchronize()
    dist.barrier()
    for _ in range(steps):
        dec.step(q, *kv, marks=mark)
    torch.cuda.synchronize()
    seg = lambda a, b: statistics.median(x.elapsed_time(y) for x, y in zip(tm[a], tm[b]))
    phases = torch.tensor([seg("start", "candidates"), seg("candidates", "gathered"), seg("gathered", "attended"),
                           seg("attended", "gathered2"), seg("gathered2", "merged"), seg("start", "merged")], device=dev)
    dist.all_reduce(phases, op=dist.ReduceOp.MAX)
    # the whole layer-step from one graph
    replay = dec.capture(q, *kv)
    for _ in range(3):
        replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ph = [float(x) for x in phases]
    limit = "candidate all-gather" if ph[1] >= ph[3] else "(O, lse) all-gather"
    out.update({
        "workload": "BASELINE config 4, context split: one sequence of 524288 tokens (32768 pages) split by page range, retention 0.125, "
                    "one layer-step",
        "pages_per_rank": hi - lo, "k_global": dec.k, "candidate_slots_per_rank": dec.k_c,
        "ms_per_layer_step_graph": float(t.item()), "ms_per_layer_step_stream": ph[5],
        "phases_ms_stream_max_over_ranks": {"local_scores_topk_candidates": ph[0], "exchange_1_candidate_allgather": ph[1],
                                            "pack_global_topk_compact_attention": ph[2], "exchange_2_o_lse_allgather": ph[3],
                                            "lse_merge": ph[4]},
        "exchange_bytes_per_rank": {"candidates": dec.msg.numel() * 4, "o_lse": dec.msg2.numel()},
        "slower_exchange": limit, "steps": steps,
        "timing": "CUDA events, median over steps, max over ranks; the graph figure replays one captured layer-step"})
    return out


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
    # every step's q | k | v for all layers, side by side in one pinned host array: one H2D copy per step
    nq, nk = Lr * B * Hq * D, Lr * B * Hkv * D
    host_in = torch.randn(n, nq + 2 * nk, generator=g).half().pin_memory()
    out_host = torch.empty(Lr, B, Hq, D, dtype=torch.float16).pin_memory()
    dev_in = torch.empty(nq + 2 * nk, dtype=torch.float16, device=dev)
    dq = dev_in[:nq].view(Lr, B, Hq, 1, D)
    dk = dev_in[nq:nq + nk].view(Lr, B, Hkv, 1, D)
    dv = dev_in[nq + nk:].view(Lr, B, Hkv, 1, D)

    # per step: one asynchronous H2D copy of the step's inputs from pinned memory, then ONE CUDA graph holding the
    # 28-layer step (sequence length read on the device) and the D2H copy of the outputs, then a stream synchronise
    replay = step.capture_step_graph(dk, dv, dq, after=lambda: out_host.copy_(step.O, non_blocking=True))
    stream = torch.cuda.current_stream()

    def one(i):
        dev_in.copy_(host_in[i], non_blocking=True)
        replay()
        stream.synchronize()

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
    h2d = host_in[0].numel() * 2
    return {"value": world * B * 1e3 / (ms / args.steps), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": ms / args.steps,
            "path": "pinned host q|k|v -> one async H2D copy -> one CUDA graph (fq_decode_step_int4_dev: append+score+select+attend per layer, D2H of O) -> stream synchronise -> host O"}



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
    # ---- the tensor-core dequant-GEMM at prefill / batched shapes ----
    from flashquest_b200.kernel.fused_proj import awq_gemm_fused
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        tpeak, tkind = float(pk["bf16_tflops_sustained"]), "measured (cuBLAS bf16, sustained)"
    except Exception:
        tpeak, tkind = 1400.0, "fallback"
    gemm_rows = []
    for name, K, Ns in (("qkv", 3072, (3072, 1024, 1024)), ("gate_up", 3072, (8192, 8192)), ("down", 8192, (3072,))):
        projs = [linear(K, N, 900 + i) for i, N in enumerate(Ns)]
        for M in (512, 4096, 32768):
            x = torch.randn(M, K, device=dev).half()
            for _ in range(3):
                awq_gemm_fused(x, projs)
            torch.cuda.synchronize()
            reps = 5 if M >= 32768 else 20
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                awq_gemm_fused(x, projs)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            flops = 2.0 * M * K * sum(Ns)
            gemm_rows.append({"proj": name, "M": M, "us_per_launch": round(us, 1), "TFLOPs": round(flops / us / 1e6, 1),
                              "frac_of_tensor_peak": round(flops / us / 1e6 / tpeak, 3)})
            del x
        del projs
    return {"metric": "AWQ W4A16 GEMV weight bytes per second", "unit": "GB/s", "workload": "awq",
            "gemm": {"kernel": "awq_gemm_kernel (tcgen05.mma, TMEM accumulators)", "peak_TFLOPs": tpeak, "peak_kind": tkind, "rows": gemm_rows},
            "parity": "unpinned (AutoAWQ's source is not in the reference tree; the oracle restates its published GEMM packing)",
            "peak": peak, "peak_kind": peak_kind, "steps": args.steps, "rows": rows,
            "device_status": _lib.lib().fq_device_status()}


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
    return {
        "metric": "TurboQuant K3-V3: pack-on-append and sparse decode attention", "workload": "turbo",
        "config": {"batch": B, "q_heads": Hq, "kv_heads": Hkv, "head_dim": D, "context": S, "page_size": page, "retention": 0.25},
        "pack": {"ms_per_sequence": pack_ms, "tokens_per_s": S / (pack_ms * 1e-3), "GBs": (in_bytes + out_bytes) / (pack_ms * 1e-3) / 1e9,
                 "frac": (in_bytes + out_bytes) / (pack_ms * 1e-3) / 1e9 / peak,
                 "what": "quantize_k_turbo (planes + scales + page metadata) and quantize_v_turbo of one 32k sequence"},
        "attention": {"us_per_call": attn_us, "union_bytes": union, "per_head_bytes": per_head,
                      "GBs_union": union / attn_us / 1e3, "frac": union / attn_us / 1e3 / peak,
                      "what": "flash_attn_sparse_turbo_fwd: WHT of Q, compact list, attention, inverse WHT (4 launches)"},
        "peak": peak, "peak_kind": peak_kind, "device_status": _lib.lib().fq_device_status()}


# --------------------------------------------------------------------------- secondary workload: INT8 KV and the mask-driven INT4 form

def run_int8(args):
    """The reference's mask-driven decode attention (its default path, `use_compact_kernel=False`) at the BASELINE config 1
    shape, batch 16 (overridable): INT8 KV (`flash_attn_sparse_fwd`) and INT4 KV (`flash_attn_sparse_int4_fwd`), each
    call = mask -> page list + attention (+ merge), replayed from a CUDA graph."""
    import torch
    from flashquest_b200 import _lib
    from flashquest_b200.eager.criticality import page_scores_int4_fast, page_scores_int8_fast
    from flashquest_b200.eager.selection import select_pages_vectorized
    from flashquest_b200.kernel.kv_quant import quantize_k, quantize_k_int4, quantize_v, quantize_v_int4
    from flashquest_b200.kernel.sparse_fwd import flash_attn_sparse_fwd
    from flashquest_b200.kernel.sparse_int4_fwd import flash_attn_sparse_int4_fwd
    _lib.lib()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, Hq, Hkv, D, S, page = args.batch or 16, 24, 8, 128, args.ctx or 32768, 16
    peak, peak_kind = measured_peak()
    n_rep = Hq // Hkv
    out = {"metric": "mask-driven sparse decode attention (INT8 and INT4 KV)", "workload": "int8",
           "config": {"batch": B, "q_heads": Hq, "kv_heads": Hkv, "head_dim": D, "context": S, "page_size": page, "retention": 0.25},
           "peak": peak, "peak_kind": peak_kind}
    for name, qk, qv, score, attend, tok_bytes in (
            ("int8", quantize_k, quantize_v, page_scores_int8_fast, flash_attn_sparse_fwd, 2 * D + 4),
            ("int4", quantize_k_int4, quantize_v_int4, page_scores_int4_fast, flash_attn_sparse_int4_fwd, D + 4)):
        g = torch.Generator(device=dev).manual_seed(1)
        kvs = []
        for _ in range(B):
            K = torch.randn(1, Hkv, S, D, device=dev, generator=g)
            K[..., [3, 17, 64, 100]] *= 8.0
            V = torch.randn(1, Hkv, S, D, device=dev, generator=g)
            kvs.append(qk(K.half(), page) + qv(V.half()))
            del K, V
        kv = tuple(torch.cat([k[i] for k in kvs]) for i in range(6))
        del kvs
        Q = torch.randn(B, Hq, 1, D, device=dev, generator=g).half()
        mask = select_pages_vectorized(score(Q, kv[1], kv[2]), 0.25, 1, 1)

        def call():
            return attend(Q, *kv, selection_mask=mask, page_size=page)

        for _ in range(3):
            call()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            call()
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.steps
        pages = int(mask.view(B, Hkv, n_rep, -1).any(2).sum())
        union = pages * (page * tok_bytes + 2 * D * 2)                # codes + V metadata per token, K metadata per page
        out[name] = {"us_per_call": us, "union_bytes": union, "GBs_union": union / us / 1e3, "frac": union / us / 1e3 / peak}
        del kv, Q, mask, graph
        torch.cuda.empty_cache()
    out["device_status"] = _lib.lib().fq_device_status()
    return out


# --------------------------------------------------------------------------- secondary workload: prefill attention

def run_prefill_attn(args):
    """The dense causal attention of the prefill branch alone (fq_prefill_attention): 24 query / 8 KV heads, head_dim 128,
    fp16, S_q = S_kv = context (default 8192), against the measured tensor peak."""
    import torch
    from flashquest_b200 import _lib
    from flashquest_b200.kernel.prefill_attn import prefill_causal_attention
    _lib.lib()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    S, Hq, Hkv, D = args.ctx or 8192, CFG["Hq"], CFG["Hkv"], CFG["D"]
    g = torch.Generator(device=dev).manual_seed(1)
    q = torch.randn(1, Hq, S, D, device=dev, generator=g).half()
    k = torch.randn(1, Hkv, S, D, device=dev, generator=g).half()
    v = torch.randn(1, Hkv, S, D, device=dev, generator=g).half()
    for _ in range(max(args.warmup, 3)):
        prefill_causal_attention(q, k, v)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        prefill_causal_attention(q, k, v)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    flops = 4.0 * Hq * D * S * (S + 1) / 2           # QK^T and PV over the causal half
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            tpeak = float(json.load(f)["bf16_tflops_sustained"])
    except Exception:
        tpeak = 1400.0
    return {"metric": "prefill causal attention", "workload": "prefill_attn", "kernel": "prefill_attn_tc_kernel (tcgen05.mma, S / O in tensor memory, TMA-staged Q/K/V; fp32 softmax)",
            "config": {"q_heads": Hq, "kv_heads": Hkv, "head_dim": D, "S_q": S, "S_kv": S, "dtype": "f16"},
            "us_per_call": us, "TFLOPs": flops / us / 1e6, "frac_of_tensor_peak": flops / us / 1e6 / tpeak, "peak_TFLOPs": tpeak,
            "device_status": _lib.lib().fq_device_status()}


# --------------------------------------------------------------------------- secondary workload: Llama decode

def llama_batched_leg(torch, cfg, w, dev, Bb, S, steps):
    """The Llama-shaped model decoding Bb sequences at once (not part of config 3): the weights are read once for all
    rows (AWQ GEMV and lm_head on the tensor cores for 2..8 rows); caches filled with synthetic K/V of BASELINE's
    distribution, no prefill."""
    from flashquest_b200 import _lib
    from flashquest_b200.eager.llama_decode import LlamaInt4Decoder
    decb = LlamaInt4Decoder(cfg, w, batch_size=Bb, max_seq_len=S + 256, page_size=16, retention=0.25, num_sinks=1, window_pages=1,
                            device=dev)
    for li in range(cfg.layers):
        for b in range(Bb):
            fill_cache_random(torch, decb.cache, li, b, 5000 + 97 * li + b, S)
        decb.cache._seen_tokens[li] = S
    idb = torch.arange(Bb, dtype=torch.int32, device=dev) * 1000 + 17
    for _ in range(2):
        idb = decb.decode_step(idb).clone()
    rb = decb.capture_decode_graph(idb)
    for _ in range(3):
        rb()
    torch.cuda.synchronize()
    b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    b0.record()
    for _ in range(steps):
        rb()
    b1.record()
    torch.cuda.synchronize()
    msb = b0.elapsed_time(b1) / steps
    return {"batch": Bb, "value": Bb * 1e3 / msb, "unit": "tokens/s", "ms_per_step": msb, "steps": steps, "layers": cfg.layers,
            "cache": f"synthetic K/V, {S} tokens per sequence (no prefill)", "device_status": _lib.lib().fq_device_status()}


def run_llama(args):
    """BASELINE config 3: random-init Llama-3.2-3B architecture with AWQ 4-bit weights; the prompt is 32 768
    uniform-random token ids from Python's seeded generator (the reference's protocol, scripts/bench_flashquest.py:
    136-169 with scripts/bench_common.py:41-44), prefilled through the tensor-core AWQ GEMM, the bulk INT4
    quantise-on-append and the dense causal attention over dequantised pages; then 127 greedy decode steps with
    sparse INT4 KV at retention 0.25, replayed from one CUDA graph: embedding gather, 28 x (norms, AWQ GEMVs,
    RoPE, append + sparse attention, SwiGLU), lm_head, argmax."""
    import random
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
    n_decode = 127
    w = random_llama_weights(cfg, dev, seed=3)
    if args.batch and args.batch > 1:        # the batched decode leg alone (small captures: --layers, --ctx, --steps)
        r = llama_batched_leg(torch, cfg, w, dev, args.batch, S, max(args.steps, 1))
        r.update({"metric": "Llama-3.2-3B-shaped AWQ decode tokens/s, batched (synthetic cache)", "workload": "llama"})
        return r
    dec = LlamaInt4Decoder(cfg, w, batch_size=1, max_seq_len=S + 256, page_size=16, retention=0.25, num_sinks=1, window_pages=1,
                           device=dev)
    from flashquest_b200 import bench_record as br
    prompt_ids = br.synthetic_token_ids(cfg.vocab, S, 0)
    prompt = torch.tensor(prompt_ids, dtype=torch.int32, device=dev)
    # one short prefill first: lazily set kernel attributes and the allocator's pools stay out of the timed one
    warm = LlamaInt4Decoder(cfg, w, batch_size=1, max_seq_len=512, page_size=16, retention=0.25, num_sinks=1, window_pages=1, device=dev)
    warm.prefill(prompt[:300])
    del warm
    torch.cuda.synchronize()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    ids = dec.prefill(prompt).clone()
    p1.record()
    torch.cuda.synchronize()
    prefill_s = p0.elapsed_time(p1) / 1e3
    for _ in range(2):
        ids = dec.decode_step(ids).clone()                     # stream steps (one foreign call each)
    replay = dec.capture_decode_graph(ids)                     # then one CUDA graph replayed per token
    for _ in range(max(args.warmup, 3)):
        replay()
    torch.cuda.synchronize()
    done = 2 + max(args.warmup, 3)
    l0 = dec.launches + dec.attn.launches
    timed = n_decode - done
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index or 0) as clk:
        e0.record()
        for _ in range(timed):
            replay()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / timed
    wbytes = cfg.layers * sum(K * N // 2 + (K // 128) * N * 2 + (K // 128) * N // 2 for K, N in
                              ((cfg.hidden, (cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim), (cfg.q_heads * cfg.head_dim, cfg.hidden),
                               (cfg.hidden, 2 * cfg.ffn), (cfg.ffn, cfg.hidden))) + cfg.vocab * cfg.hidden * 2
    lin_flops = 2.0 * S * cfg.layers * (cfg.hidden * (cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim + cfg.q_heads * cfg.head_dim * cfg.hidden +
                                        3 * cfg.hidden * cfg.ffn)
    record_path = getattr(args, "record", None)
    if record_path:
        # the reference's own record format: prefill + 127 decode steps per repetition on a re-used cache allocation
        rcfg = br.run_config(S, n_decode + 1, 3, 0, model="random-init Llama-3.2-3B architecture (AWQ 4-bit, group 128)", kv_bits=4,
                             retention=0.25, page_size=16, num_sinks=1, window_pages=1, warmup_steps=done, cache_capacity=S + 256,
                             input_sha256=br.input_sha256(prompt_ids), generation="manual-greedy-fixed-output-count-v1",
                             runtime={"cuda": torch.version.cuda, "devices": [str(dev)], "dtype": "torch.float16", "weight_kernel": "fq_awq_gemv / fq_awq_gemm",
                                      "weight_storage_bytes": wbytes})
        rec = br.new_record("flashquest_b200", "AWQ-INT4 + INT4 KV, retention=0.25", rcfg)
        t_wall = time.time()
        for _ in range(rcfg["reps"]):
            dec.cache._seen_tokens = [0] * cfg.layers
            torch.cuda.reset_peak_memory_stats()
            torch.cuda.synchronize()
            t0 = time.monotonic_ns()
            nxt = dec.prefill(prompt).clone()
            torch.cuda.synchronize()
            t1 = time.monotonic_ns()
            rp = dec.capture_decode_graph(nxt)
            torch.cuda.synchronize()
            t1b = time.monotonic_ns()
            for _ in range(n_decode):
                rp()
            torch.cuda.synchronize()
            t2 = time.monotonic_ns()
            rec["samples"].append(br.make_sample(S, n_decode, (t1 - t0) / 1e9, (t2 - t1b) / 1e9,
                                                 round(torch.cuda.max_memory_allocated() / 2 ** 20, 1), round(torch.cuda.max_memory_reserved() / 2 ** 20, 1)))
            del rp
        rec["wall_s"] = time.time() - t_wall
        br.summarize_samples(rec)
        rec["provenance"] = br.provenance({"torch": torch.__version__}, [{"name": torch.cuda.get_device_name(dev)}])
        with open(record_path, "w") as f:
            json.dump(br.export_record(rec), f, indent=1)
    launches = dec.launches + dec.attn.launches - l0
    status = _lib.lib().fq_device_status()
    batched = None
    if not args.layers and not args.ctx:
        del dec, replay
        torch.cuda.empty_cache()
        batched = llama_batched_leg(torch, cfg, w, dev, 8, S, 30)
    return {
        "metric": "Llama-3.2-3B-shaped AWQ decode tokens/s at 32k ctx (sparse INT4 attention)", "workload": "llama",
        "value": 1e3 / ms, "unit": "tokens/s", "ms_per_token": ms, "decode_steps_timed": timed, "decode_steps_total": n_decode,
        "prefill_s": prefill_s, "prefill_tokens_per_s": S / prefill_s, "prefill_linear_TFLOPs": lin_flops / prefill_s / 1e12,
        "decode_s": ms * n_decode / 1e3,
        "config": {"hidden": cfg.hidden, "layers": cfg.layers, "q_heads": cfg.q_heads, "kv_heads": cfg.kv_heads, "head_dim": cfg.head_dim,
                   "ffn": cfg.ffn, "vocab": cfg.vocab, "context": S, "retention": 0.25, "weights": "random-init AWQ 4-bit, group 128",
                   "prompt": "32768 ids from random.Random(0).randrange(vocab), prefilled", "parity": "AWQ arithmetic unpinned"},
        "weight_bytes_per_token": wbytes, "weight_GBs": wbytes / ms / 1e6,
        "gpu_launches": launches, "clocks": clk.summary(), "batch8": batched,
        "device_status": status}


# --------------------------------------------------------------------------- secondary workload: context split

def run_ctxsplit(args):
    """The context-split leg alone (torchrun, N >= 2)."""
    import torch
    import torch.distributed as dist
    from flashquest_b200 import _lib
    _lib.lib()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        if rank == 0:
            print(json.dumps({"workload": "ctxsplit", "unavailable": "needs torchrun with at least 2 ranks"}))
        return
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    out = run_ctxsplit_leg(torch, dist, world, rank, dev, args)
    out["n_gpus"] = world
    out["device_status"] = _lib.lib().fq_device_status()
    if rank == 0:
        print(json.dumps(out))
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
    ap.add_argument("--workload", default="decode", choices=["decode", "awq", "turbo", "int8", "llama", "ctxsplit", "prefill_attn"],
                    help="decode = the headline metric; awq = secondary table for the W4A16 GEMV (1 GPU)")
    ap.add_argument("--no-batched", action="store_true", help="skip the batched-attention leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--record", default=None, help="--workload llama: also write a benchmark record in the reference's schema-3 format to this path")
    ap.add_argument("--no-extra", action="store_true", help="skip BASELINE config 4 (batch-sharded and context-split legs) and the secondary workloads")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary workloads (AWQ GEMV table, TurboQuant, Llama decode)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "awq":
        print(json.dumps(run_awq(args)))
    elif args.workload == "turbo":
        print(json.dumps(run_turbo(args)))
    elif args.workload == "int8":
        print(json.dumps(run_int8(args)))
    elif args.workload == "llama":
        print(json.dumps(run_llama(args)))
    elif args.workload == "prefill_attn":
        print(json.dumps(run_prefill_attn(args)))
    elif args.workload == "ctxsplit":
        run_ctxsplit(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
