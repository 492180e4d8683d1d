"""Benchmark records in the reference's on-disk format (schema version 3), so that runs of this
library line up with the reference's saved evidence (flashquest scripts/bench_common.py:52-83 for the
record, :310-354 for the exported key sets; example:
benchmarks/validation/ablation/<hash>/cells/c32768-s0-sparse.json).

A record holds the run configuration, one sample per repetition (prefill and decode intervals and the
three throughputs derived from them) and the medians over the samples.  Pure host code."""
from __future__ import annotations

import hashlib
import json
import platform
import random
from statistics import median
from typing import Iterable, Optional

SCHEMA_VERSION = 3

RECORD_KEYS = ("schema_version", "backend", "quant", "config", "ctx_len", "decode_steps", "decode_tok_s", "prefill_tok_s",
               "end_to_end_tok_s", "peak_allocated_mib", "peak_reserved_mib", "samples", "wall_s", "oom", "error")
SAMPLE_KEYS = ("input_tokens", "output_tokens", "prefill_s", "decode_s", "request_s", "prefill_tok_s", "decode_tok_s",
               "end_to_end_tok_s", "peak_allocated_mib", "peak_reserved_mib")
CONFIG_KEYS = {"ctx_len", "n_decode", "reps", "seed", "model", "kv_bits", "retention", "page_size", "num_sinks", "window_pages",
               "kv_cache_dtype", "kv_k", "kv_v", "n_gpu_layers", "threads", "revision", "model_cache", "warmup_steps",
               "cache_capacity", "input_sha256", "generation", "runtime", "memory_protocol"}


def synthetic_token_ids(vocab_size: int, ctx_len: int, seed: int) -> list:
    """The reference's prompt: ctx_len ids from Python's seeded generator (scripts/bench_common.py:41-44)."""
    rng = random.Random(seed)
    return [rng.randrange(vocab_size) for _ in range(ctx_len)]


def input_sha256(ids: Iterable[int]) -> str:
    return hashlib.sha256(json.dumps(list(ids), separators=(",", ":")).encode()).hexdigest()


def run_config(ctx_len: int, n_decode: int, reps: int, seed: int, **settings) -> dict:
    """n_decode counts output tokens; the first one comes from the prefill."""
    if ctx_len < 1 or n_decode < 2 or reps < 1:
        raise ValueError("ctx-len >= 1, n-decode >= 2, and reps >= 1 are required")
    return {"ctx_len": ctx_len, "n_decode": n_decode, "reps": reps, "seed": seed, **settings}


def new_record(backend: str, quant: str, config: dict) -> dict:
    return {"schema_version": SCHEMA_VERSION, "backend": backend, "quant": quant, "config": config,
            "ctx_len": config["ctx_len"], "decode_steps": config["n_decode"] - 1,
            "decode_tok_s": None, "prefill_tok_s": None, "end_to_end_tok_s": None,
            "peak_allocated_mib": None, "peak_reserved_mib": None, "samples": [], "wall_s": None, "oom": False, "error": None}


def make_sample(ctx_len: int, decode_steps: int, prefill_s: float, decode_s: float,
                peak_allocated_mib: Optional[float] = None, peak_reserved_mib: Optional[float] = None) -> dict:
    """One repetition: the prefill interval ends with the first output token, the decode interval covers the
    remaining decode_steps tokens (scripts/bench_flashquest.py:136-169)."""
    request_s = prefill_s + decode_s
    return {"input_tokens": ctx_len, "output_tokens": decode_steps + 1, "prefill_s": prefill_s, "decode_s": decode_s,
            "request_s": request_s, "prefill_tok_s": ctx_len / prefill_s, "decode_tok_s": decode_steps / decode_s,
            "end_to_end_tok_s": (decode_steps + 1) / request_s,
            "peak_allocated_mib": peak_allocated_mib, "peak_reserved_mib": peak_reserved_mib}


def summarize_samples(record: dict) -> None:
    """Medians of the throughputs, maxima of the memory counters; every sample is kept."""
    samples = record["samples"]
    if not samples:
        raise ValueError("no completed benchmark samples")
    for key in ("decode_tok_s", "prefill_tok_s", "end_to_end_tok_s"):
        values = [s[key] for s in samples if s.get(key) is not None]
        record[key] = median(values) if values else None
    for key in ("peak_allocated_mib", "peak_reserved_mib"):
        values = [s[key] for s in samples if s.get(key) is not None]
        record[key] = max(values) if values else None


def provenance(packages: Optional[dict] = None, gpus: Optional[list] = None) -> dict:
    return {"python": platform.python_version(), "os": platform.system(), "kernel": platform.release(), "wsl": False,
            "packages": packages or {}, "gpus": gpus or []}


def export_record(record: dict) -> dict:
    """The record restricted to the keys the reference exports, samples likewise."""
    keep = set(RECORD_KEYS) | {"versions", "prompt_kind", "provenance"}
    out = {k: v for k, v in record.items() if k in keep}
    out["config"] = {k: v for k, v in record.get("config", {}).items() if k in CONFIG_KEYS}
    out["samples"] = [{k: v for k, v in s.items() if k in SAMPLE_KEYS} for s in record.get("samples", [])]
    out["error"] = ("out_of_memory" if record.get("oom") else "backend_error") if record.get("error") else None
    return out
