"""The CPU oracle against outputs of the reference itself (tests/golden) and against the
known-answer vectors in the reference's own tests.  No GPU needed."""
import math

import numpy as np
import pytest
import torch

import oracle
from tests._util import DTYPES, bit_equal


# ---------------------------------------------------------------- INT4 quantisation

def _quant_cases(golden):
    return golden.meta["quant"]


def test_int4_quant_bit_exact(golden):
    for case in _quant_cases(golden):
        n = case["name"]
        dt = DTYPES[case["dtype"]]
        K = golden.get("quant_int4", f"q_{n}_K", dtype=dt)
        V = golden.get("quant_int4", f"q_{n}_V", dtype=dt)
        Kp, Ks, Km = oracle.quantize_k_int4(K, case["page"])
        Vp, Vs, Vm = oracle.quantize_v_int4(V)
        for got, key in ((Kp, "Kp"), (Ks, "Ks"), (Km, "Km"), (Vp, "Vp"), (Vs, "Vs"), (Vm, "Vm")):
            want = golden.get("quant_int4", f"q_{n}_{key}")
            assert bit_equal(got, want), f"{n}:{key} differs from the reference"


def test_int4_dequant_bit_exact(golden):
    for case in _quant_cases(golden):
        n = case["name"]
        g = lambda k: golden.get("quant_int4", f"q_{n}_{k}")  # noqa: E731
        Kd = oracle.dequantize_k_int4(g("Kp"), g("Ks"), g("Km"), case["page"])
        Vd = oracle.dequantize_v_int4(g("Vp"), g("Vs"), g("Vm"))
        assert bit_equal(Kd, g("Kd")), n
        assert bit_equal(Vd, g("Vd")), n


def test_handwritten_nibble_vectors(golden):
    hw = golden.meta["handwritten"]
    # low nibble = even channel, high nibble = odd channel
    by = torch.tensor(hw["nibble_unpack"]["bytes"], dtype=torch.uint8).reshape(1, 1, 2, 2)
    one = torch.ones(1, 1, 2, 1, dtype=torch.bfloat16)
    zero = torch.zeros(1, 1, 2, 1, dtype=torch.bfloat16)
    codes = oracle.dequantize_v_int4(by, one, zero).float().reshape(2, 4)
    assert codes.tolist() == [[float(x) for x in r] for r in hw["nibble_unpack"]["codes"]]
    # quantising the integers 0..15 with mn=0, scale=1 returns them as codes
    V = torch.arange(16, dtype=torch.float32).reshape(1, 1, 1, 16)
    Vp, Vs, Vm = oracle.quantize_v_int4(V)
    assert Vs.item() == 1.0 and Vm.item() == 0.0
    assert Vp.flatten().tolist() == [(2 * j) | ((2 * j + 1) << 4) for j in range(8)]


def test_odd_head_dim_rejected():
    with pytest.raises(ValueError, match="even head_dim"):
        oracle.quantize_k_int4(torch.randn(1, 2, 64, 65, dtype=torch.bfloat16), 64)


def test_page_max_identity():
    # reference test: mn + 15*scale ~ page max (tests/test_kv_quant_int4.py:57-64)
    torch.manual_seed(7)
    K = torch.randn(1, 2, 64, 32, dtype=torch.bfloat16)
    _, scale, mn = oracle.quantize_k_int4(K, 64)
    ref = K.float().view(1, 2, 1, 64, 32).max(dim=3).values
    assert torch.allclose(mn.float() + 15.0 * scale.float(), ref, atol=1e-2, rtol=1e-2)


# ---------------------------------------------------------------- WHT / TurboQuant

def test_wht_bit_exact(golden):
    for case in golden.meta["turbo"]:
        n = case["name"]
        dt = DTYPES[case["dtype"]]
        K = golden.get("turbo", f"t_{n}_K", dtype=dt)
        W = oracle.wht_along_head_dim(K)
        assert bit_equal(W, golden.get("turbo", f"t_{n}_W", dtype=dt)), n


def test_wht_self_inverse():
    x = torch.randn(4, 7, 128)
    assert (oracle.wht_along_head_dim(oracle.wht_along_head_dim(x)) - x).abs().max() < 1e-4
    with pytest.raises(ValueError, match="power of 2"):
        oracle.wht_along_head_dim(torch.randn(2, 96))


def test_turbo_quant_against_reference(golden):
    """Bit planes and scales: bit-exact except where the fp32 summation order of the RMS
    moves a value across a codebook midpoint (counted, must stay below 1e-3 of the codes)."""
    total = diff = 0
    for case in golden.meta["turbo"]:
        n = case["name"]
        dt = DTYPES[case["dtype"]]
        D = case["shape"][-1]
        K = golden.get("turbo", f"t_{n}_K", dtype=dt)
        V = golden.get("turbo", f"t_{n}_V", dtype=dt)
        Km, Kl, Kst, Ksr, Kmr = oracle.quantize_k_turbo(K, case["page"])
        Vm, Vl, Vst = oracle.quantize_v_turbo(V)
        assert bit_equal(Ksr, golden.get("turbo", f"t_{n}_Ksr")), n
        assert bit_equal(Kmr, golden.get("turbo", f"t_{n}_Kmr")), n
        for got, key in ((Km, "Kmsb"), (Kl, "Klsb"), (Vm, "Vmsb"), (Vl, "Vlsb")):
            want = golden.get("turbo", f"t_{n}_{key}")
            x = (got ^ want).numpy()
            diff += int(np.unpackbits(x).sum())
            total += got.numel() * 8
        for got, key in ((Kst, "Kst"), (Vst, "Vst")):
            want = golden.get("turbo", f"t_{n}_{key}")
            # bf16 scale: at most one bf16 ulp apart, and only rarely
            d = (got.view(torch.int16).int() - want.view(torch.int16).int()).abs()
            assert d.max() <= 1, n
            assert (d != 0).float().mean() < 0.01, n
    assert diff / total < 1e-3, f"{diff} of {total} plane bits differ"


def test_turbo_dequant_bit_exact(golden):
    for case in golden.meta["turbo"]:
        n = case["name"]
        g = lambda k: golden.get("turbo", f"t_{n}_{k}")  # noqa: E731
        Kd = oracle.dequantize_k_turbo(g("Kmsb"), g("Klsb"), g("Kst"), case["shape"][-1])
        assert bit_equal(Kd, g("Kd")), n


def test_turbo_codebook(golden):
    cb = oracle.turbo_codebook()
    assert torch.allclose(cb, torch.tensor(golden.meta["handwritten"]["turbo_codebook"]))
    assert torch.allclose(cb, -cb.flip(0))


# ---------------------------------------------------------------- scores / selection / compact

def test_scores_close_to_reference(golden):
    for case in golden.meta["chain"]:
        n = case["name"]
        dt = DTYPES[case["dtype"]]
        Q = golden.get("chain", f"{n}_Q", dtype=dt)
        s = oracle.page_scores_int4_fast(Q, golden.get("chain", f"{n}_Ks"), golden.get("chain", f"{n}_Km"))
        want = golden.get("chain", f"{n}_scores")
        assert s.shape == want.shape
        assert torch.allclose(s, want, rtol=1e-4, atol=1e-4), (n, (s - want).abs().max())


def test_selection_matches_reference(golden):
    for case in golden.meta["chain"]:
        n = case["name"]
        scores = golden.get("chain", f"{n}_scores")
        mask = oracle.select_pages_vectorized(scores, case["retention"], case["sinks"], case["window"],
                                              k_max_static=case["k_max_static"])
        assert torch.equal(mask, golden.get("chain", f"{n}_mask", as_bool=True)), n
        r_head = torch.tensor([case["retention"] if h % 2 == 0 else 0.0 for h in range(case["Hq"])])
        mask_ph = oracle.select_pages_vectorized(scores, r_head, case["sinks"], case["window"])
        assert torch.equal(mask_ph, golden.get("chain", f"{n}_mask_ph", as_bool=True)), n
        comp = oracle.build_compact_selection(mask, case["bucket"])
        assert torch.equal(comp, golden.get("chain", f"{n}_comp")), n


def test_selection_handwritten(golden):
    hw = golden.meta["handwritten"]
    c = hw["select_zero_retention"]
    m = oracle.select_pages_vectorized(torch.zeros(1, 1, 1, c["P"]), c["retention"], c["sinks"], c["window"])
    assert m.flatten().int().tolist() == c["mask"]
    for key in ("select_topk", "select_round_up"):
        c = hw[key]
        s = torch.tensor(c["scores"]).reshape(1, 1, 1, -1)
        m = oracle.select_pages_vectorized(s, c["retention"], 0, 0)
        assert m.flatten().int().tolist() == c["mask"], key
    assert oracle.select_pages_vectorized(torch.randn(1, 2, 1, 8), 1.0, 0, 0).all()
    with pytest.raises(ValueError, match="retention"):
        oracle.select_pages_vectorized(torch.zeros(1, 1, 1, 4), 1.5, 0, 0)
    with pytest.raises(ValueError, match="per-head retention"):
        oracle.select_pages_vectorized(torch.zeros(1, 2, 1, 4), torch.tensor([0.5]), 0, 0)


def test_selection_tie_rule_and_static_kmax():
    s = torch.tensor([1.0, 2.0, 2.0, 2.0, 0.0]).reshape(1, 1, 1, 5)
    m = oracle.select_pages_vectorized(s, 0.4, 0, 0)  # k = 2
    assert m.flatten().int().tolist() == [0, 1, 1, 0, 0]
    # static k_max larger than needed changes nothing; smaller caps the count
    sc = torch.randn(2, 3, 1, 40)
    a = oracle.select_pages_vectorized(sc, 0.25, 1, 2)
    b = oracle.select_pages_vectorized(sc, 0.25, 1, 2, k_max_static=33)
    assert torch.equal(a, b)
    c = oracle.select_pages_vectorized(sc, 0.25, 0, 0, k_max_static=3)
    assert (c.sum(-1) == 3).all()
    # sinks / window larger than P clamp
    assert oracle.select_pages_vectorized(torch.randn(1, 1, 1, 3), 0.0, 9, 9).all()


def test_compact_handwritten(golden):
    hw = golden.meta["handwritten"]
    c = hw["compact_basic"]
    mask = torch.zeros(1, 1, 1, c["P"], dtype=torch.bool)
    mask[..., c["selected"]] = True
    for b in c["buckets"]:
        out = oracle.build_compact_selection(mask, b)
        assert out.shape == (1, 1, 1, b) and out.dtype == torch.int32
        assert sorted(out[0, 0, 0, :3].tolist()) == c["selected"]
        assert (out[0, 0, 0, 3:] == -1).all()
    c = hw["compact_small_P"]
    out = oracle.build_compact_selection(torch.tensor(c["mask"]).bool().reshape(1, 1, 1, -1), c["bucket"])
    assert sorted(x for x in out.flatten().tolist() if x != -1) == c["selected"]
    assert (out[0, 0, 0, 3:] == -1).all()
    assert (oracle.build_compact_selection(torch.zeros(1, 1, 1, 8, dtype=torch.bool), 4) == -1).all()
    with pytest.raises(ValueError, match="BUCKET_MAX"):
        oracle.build_compact_selection(mask, 0)
    with pytest.raises(ValueError, match="bool"):
        oracle.build_compact_selection(mask.int(), 4)


# ---------------------------------------------------------------- attention

def test_attention_close_to_reference(golden):
    """fp64-accumulating oracle vs the reference's fp32 chain: tolerance 2e-5 (fp32 noise)."""
    for case in golden.meta["chain"]:
        n = case["name"]
        dt = DTYPES[case["dtype"]]
        g = lambda k, **kw: golden.get("chain", f"{n}_{k}", **kw)  # noqa: E731
        Q = g("Q", dtype=dt)
        args = (Q, g("Kp"), g("Ks"), g("Km"), g("Vp"), g("Vs"), g("Vm"))
        mask = g("mask", as_bool=True)
        O, lse = oracle.sparse_attn_int4(*args, selection_mask=mask, page_size=case["page"])
        assert torch.allclose(O, g("O"), atol=2e-5, rtol=1e-5), (n, (O - g("O")).abs().max())
        assert torch.allclose(lse, g("lse"), atol=2e-5, rtol=1e-6), n
        O2, lse2 = oracle.sparse_attn_int4(*args, selected_page_ids=g("comp"), page_size=case["page"])
        assert torch.equal(O, O2) and torch.equal(lse, lse2), n
        if case["tail"]:
            Kt, Vt = g("Ktail", dtype=dt), g("Vtail", dtype=dt)
            Oa, la = oracle.sparse_attn_int4(*args, selection_mask=mask, page_size=case["page"],
                                             K_partial=Kt, V_partial=Vt)
            assert torch.allclose(Oa, g("Oall"), atol=2e-5, rtol=1e-5), n
            assert torch.allclose(la, g("lse_all"), atol=2e-5, rtol=1e-6), n
            if f"{n}_Omerged" in golden.npz("chain"):
                # the reference's dispatcher rounds both parts to bf16 before merging
                assert (Oa - g("Omerged").float()).abs().max() < 2e-2, n


def test_attention_empty_selection():
    Q = torch.randn(1, 2, 1, 128, dtype=torch.bfloat16)
    K = torch.randn(1, 1, 32, 128, dtype=torch.bfloat16)
    Kp, Ks, Km = oracle.quantize_k_int4(K, 16)
    Vp, Vs, Vm = oracle.quantize_v_int4(K)
    comp = torch.full((1, 2, 1, 4), -1, dtype=torch.int32)
    O, lse = oracle.sparse_attn_int4(Q, Kp, Ks, Km, Vp, Vs, Vm, selected_page_ids=comp, page_size=16)
    assert (O == 0).all() and torch.isinf(lse).all() and (lse < 0).all()


def test_lse_merge_matches_two_way_formula():
    torch.manual_seed(0)
    Oa, Ob = torch.randn(2, 3, 1, 16), torch.randn(2, 3, 1, 16)
    la, lb = torch.randn(2, 3, 1), torch.randn(2, 3, 1)
    m = torch.maximum(la, lb)
    wa, wb = torch.exp(la - m).unsqueeze(-1), torch.exp(lb - m).unsqueeze(-1)
    want = (wa * Oa + wb * Ob) / (wa + wb)
    O, lse = oracle.lse_merge(torch.stack([Oa, Ob]), torch.stack([la, lb]))
    assert torch.allclose(O, want, atol=1e-6)
    assert torch.allclose(lse, torch.logaddexp(la, lb), atol=1e-6)


def test_turbo_attention_close_to_reference(golden):
    if not golden.meta["turbo_attn"]:
        pytest.skip("no turbo attention golden")
    case = golden.meta["turbo_attn"][0]
    g = lambda k, **kw: golden.get("turbo", f"ta_{k}", **kw)  # noqa: E731
    O, lse = oracle.sparse_attn_turbo(g("Q"), g("Kmsb"), g("Klsb"), g("Kst"), g("Vmsb"), g("Vlsb"), g("Vst"),
                                      selection_mask=g("mask", as_bool=True), page_size=case["page"])
    # the reference path dequantises K,V to bf16 first: bf16-level agreement
    assert (O - g("O").float()).abs().max() < 5e-2
    assert (lse - g("lse")).abs().max() < 5e-2


# ---------------------------------------------------------------- config 0 (digests)

@pytest.mark.parametrize("dt_name", ["fp16", "bf16"])
def test_config0_digests(golden, dt_name):
    """BASELINE config 0 end to end on the oracle: packing and metadata digests equal the
    reference's; selection equal; attention within 2e-5."""
    import hashlib
    ref = golden.meta["config0"][dt_name]
    dt = {"fp16": torch.float16, "bf16": torch.bfloat16}[dt_name]
    rng = np.random.default_rng(0)
    K = torch.from_numpy(rng.standard_normal((1, 8, 4096, 128), dtype=np.float32))
    V = torch.from_numpy(rng.standard_normal((1, 8, 4096, 128), dtype=np.float32))
    Q = torch.from_numpy(rng.standard_normal((1, 24, 1, 128), dtype=np.float32))
    for c in (3, 17, 64, 100):
        K[..., c] *= 8.0
    K, V, Q = K.to(dt), V.to(dt), Q.to(dt)

    def sha(t):
        t = t.contiguous()
        if t.dtype in (torch.bfloat16, torch.float16):
            t = t.view(torch.int16)
        if t.dtype == torch.bool:
            t = t.to(torch.uint8)
        return hashlib.sha256(t.numpy().tobytes()).hexdigest()

    if sha(K) != ref["input_sha256"]["K"]:
        pytest.skip("numpy random stream differs from the one the golden was made with")
    Kp, Ks, Km = oracle.quantize_k_int4(K, 16)
    Vp, Vs, Vm = oracle.quantize_v_int4(V)
    for t, key in ((Kp, "K_packed"), (Ks, "K_scale"), (Km, "K_mn"), (Vp, "V_packed"), (Vs, "V_scale"), (Vm, "V_mn")):
        assert sha(t) == ref["sha256"][key], key
    scores = oracle.page_scores_int4_fast(Q, Ks, Km)
    assert np.allclose(scores[0, 0, 0, :8].numpy(), ref["scores_head0_first8"], rtol=1e-5, atol=1e-5)
    mask = oracle.select_pages_vectorized(scores, 0.25, 1, 1, k_max_static=64)
    assert mask.sum(-1).flatten().tolist() == ref["pages_selected_per_head"]
    if ref["min_topk_margin"] > 1e-4:
        assert sha(mask) == ref["sha256"]["mask"]
    O, lse = oracle.sparse_attn_int4(Q, Kp, Ks, Km, Vp, Vs, Vm, selection_mask=mask, page_size=16)
    assert np.abs(O.flatten().numpy() - np.array(ref["O"], dtype=np.float32)).max() < 2e-5
    assert np.abs(lse.flatten().numpy() - np.array(ref["lse"], dtype=np.float32)).max() < 2e-5
