"""The benchmark-record writer against the key sets and numbers of a record the reference saved."""
import json
import os

import pytest

from flashquest_b200 import bench_record as br

G = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bench_record_keys.json")))


def test_record_layout_matches_the_reference_record():
    cfg = br.run_config(32768, 128, 3, 0, model="random-init", kv_bits=4, retention=0.25, page_size=16, num_sinks=1, window_pages=1)
    rec = br.new_record("flashquest_b200", "AWQ-INT4 + INT4 KV, retention=0.25", cfg)
    assert rec["schema_version"] == G["schema_version"] == 3
    assert rec["decode_steps"] == G["decode_steps"] == G["n_decode"] - 1
    s0 = G["sample0"]
    sample = br.make_sample(s0["input_tokens"], s0["output_tokens"] - 1, s0["prefill_s"], s0["decode_s"], 1.0, 2.0)
    assert sorted(sample) == G["sample_keys"]
    for k in ("request_s", "prefill_tok_s", "decode_tok_s", "end_to_end_tok_s"):
        assert sample[k] == pytest.approx(s0[k], rel=1e-12), k
    for d, p, e in G["sample_throughputs"]:
        rec["samples"].append({"decode_tok_s": d, "prefill_tok_s": p, "end_to_end_tok_s": e, "peak_allocated_mib": 1.0, "peak_reserved_mib": 2.0})
    br.summarize_samples(rec)
    for k, v in G["medians"].items():
        assert rec[k] == pytest.approx(v, rel=1e-12), k
    exported = br.export_record({**rec, "junk": 1})
    assert "junk" not in exported and set(exported) <= set(G["record_keys"]) | {"error"}
    assert set(exported["config"]) <= set(G["config_keys"])
    with pytest.raises(ValueError):
        br.summarize_samples(br.new_record("x", "y", cfg))
    with pytest.raises(ValueError):
        br.run_config(0, 128, 3, 0)


def test_prompt_ids_are_the_reference_prompt():
    """The 32 768-id prompt of seed 0 hashes to the input_sha256 the reference's record carries."""
    ids = br.synthetic_token_ids(128256, G["ctx_len"], G["seed"])
    assert len(ids) == 32768 and all(0 <= i < 128256 for i in ids)
    assert br.input_sha256(ids) == G["input_sha256"]
