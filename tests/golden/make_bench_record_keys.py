"""Writes tests/golden/bench_record_keys.json: the key sets of a benchmark record the reference saved
(benchmarks/validation/ablation/<hash>/cells/c32768-s0-sparse.json), read as data in the build container.

    python tests/golden/make_bench_record_keys.py /path/to/reference
"""
import glob
import json
import os
import sys

if len(sys.argv) < 2:
    sys.exit("usage: make_bench_record_keys.py /path/to/reference")
ref = sys.argv[1]
path = sorted(glob.glob(os.path.join(ref, "benchmarks/validation/ablation/*/cells/c32768-s0-sparse.json")))[0]
rec = json.load(open(path))
out = {"source": "benchmarks/validation/ablation/<hash>/cells/c32768-s0-sparse.json", "schema_version": rec["schema_version"],
       "record_keys": sorted(rec), "config_keys": sorted(rec["config"]), "sample_keys": sorted(rec["samples"][0]),
       "decode_steps": rec["decode_steps"], "n_decode": rec["config"]["n_decode"],
       "sample0": {k: rec["samples"][0][k] for k in ("input_tokens", "output_tokens", "prefill_s", "decode_s", "request_s",
                                                     "prefill_tok_s", "decode_tok_s", "end_to_end_tok_s")},
       "medians": {k: rec[k] for k in ("decode_tok_s", "prefill_tok_s", "end_to_end_tok_s")},
       "sample_throughputs": [[s["decode_tok_s"], s["prefill_tok_s"], s["end_to_end_tok_s"]] for s in rec["samples"]],
       "input_sha256": rec["config"]["input_sha256"], "ctx_len": rec["ctx_len"], "seed": rec["config"]["seed"]}
json.dump(out, open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "bench_record_keys.json"), "w"), indent=1)
print("wrote bench_record_keys.json")
