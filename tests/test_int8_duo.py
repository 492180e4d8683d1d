"""INT8 KV variant: the CPU oracle against outputs of the reference itself (tests/golden/int8.npz, made
by tests/golden/make_golden_int8.py), and the DuoAttention pattern loader against the reference's own
test cases (tests/test_duo_pattern.py).  No GPU needed."""
import json
import os

import numpy as np
import pytest
import torch

import oracle
from tests._util import DTYPES, GOLDEN_DIR, bit_equal, from_bits


@pytest.fixture(scope="module")
def int8_golden():
    with open(os.path.join(GOLDEN_DIR, "int8.json")) as f:
        meta = json.load(f)
    return meta["cases"], np.load(os.path.join(GOLDEN_DIR, "int8.npz"))


def _g(npz, name, key, dtype=None):
    return from_bits(npz[f"i8_{name}_{key}"], dtype)


def test_int8_quant_dequant_scores_bit_exact(int8_golden):
    cases, npz = int8_golden
    assert len(cases) >= 4
    for c in cases:
        n, dt, page = c["name"], DTYPES[c["dtype"]], c["page"]
        K, V = _g(npz, n, "K", dt), _g(npz, n, "V", dt)
        Ku, Ks, Km = oracle.quantize_k(K, page)
        Vu, Vs, Vm = oracle.quantize_v(V)
        for got, key in ((Ku, "Ku"), (Ks, "Ks"), (Km, "Km"), (Vu, "Vu"), (Vs, "Vs"), (Vm, "Vm")):
            assert bit_equal(got, _g(npz, n, key)), f"{n}:{key} differs from the reference"
        assert bit_equal(oracle.dequantize_k(Ku, Ks, Km, page), _g(npz, n, "Kd")), n
        assert bit_equal(oracle.dequantize_v(Vu, Vs, Vm), _g(npz, n, "Vd")), n
        Q = _g(npz, n, "Q", DTYPES[c["q_dtype"]])
        got = oracle.page_scores_int8_fast(Q, Ks, Km)
        want, slow = _g(npz, n, "scores"), _g(npz, n, "scores_slow")
        # the reference's fast form runs two fp32 matmuls whose summation order torch does not fix:
        # the restatement's fixed order agrees to fp32 rounding of a D-term sum, and the slow
        # (elementwise-max) form bounds it from the other side
        tol = 4e-6 * (Q.float().abs().sum(-1, keepdim=True) * (Km.float().abs().amax((-1, -2)).max() + 255 * Ks.float().amax()))
        assert ((got - want).abs() <= tol.clamp_min(1e-5)).all(), n
        assert torch.allclose(got, slow, rtol=2e-2, atol=2e-1), n


def test_int8_page_max_identity():
    # mn + 255*scale ~ page max: the upper bound the score uses (reference tests/test_page_scores_int8.py)
    torch.manual_seed(3)
    K = torch.randn(1, 2, 128, 32, dtype=torch.bfloat16)
    _, scale, mn = oracle.quantize_k(K, 64)
    ref = K.float().view(1, 2, 2, 64, 32).max(dim=3).values
    assert torch.allclose(mn.float() + 255.0 * scale.float(), ref, atol=3e-2, rtol=2e-2)


def test_int8_attention_oracle_equals_dense_on_dequantised():
    # all pages selected: the oracle equals softmax attention over code*scale + mn (no bf16 rounding)
    torch.manual_seed(5)
    B, Hq, Hkv, S, D, page = 1, 4, 2, 96, 64, 32
    K = torch.randn(B, Hkv, S, D, dtype=torch.bfloat16)
    V = torch.randn(B, Hkv, S, D, dtype=torch.bfloat16)
    Q = torch.randn(B, Hq, 1, D, dtype=torch.bfloat16)
    Ku, Ks, Km = oracle.quantize_k(K, page)
    Vu, Vs, Vm = oracle.quantize_v(V)
    sel = torch.ones(B, Hq, 1, S // page, dtype=torch.bool)
    O, lse = oracle.sparse_attn_int8(Q, Ku, Ks, Km, Vu, Vs, Vm, selection_mask=sel, page_size=page)
    Kf = Ku.double() * Ks.double().repeat_interleave(page, 2) + Km.double().repeat_interleave(page, 2)
    Vf = Vu.double() * Vs.double() + Vm.double()
    Kf, Vf = Kf.repeat_interleave(Hq // Hkv, 1), Vf.repeat_interleave(Hq // Hkv, 1)
    s = (Q.double() @ Kf.transpose(-1, -2)) / D ** 0.5
    assert torch.allclose(O.double(), torch.softmax(s, -1) @ Vf, atol=1e-5)
    assert torch.allclose(lse.double(), torch.logsumexp(s, -1), atol=1e-5)


# ---------------------------------------------------------------- DuoAttention patterns

def test_duo_threshold_kwarg(tmp_path):
    from flashquest_b200.duo.pattern import load_duo_pattern
    p = tmp_path / "tiny.tsv"
    p.write_text("0.4\t0.6\n0.5\t0.51\n")
    default = load_duo_pattern(p)
    assert default.dtype == torch.bool and default.shape == (2, 2)
    assert default.tolist() == [[False, True], [True, True]]
    assert load_duo_pattern(p, threshold=0.51).tolist() == [[False, True], [False, True]]


def test_duo_llama_shape(tmp_path):
    from flashquest_b200.duo import load_duo_pattern
    rng = np.random.default_rng(0)
    p = tmp_path / "full_attention_heads.tsv"
    p.write_text("\n".join("\t".join(f"{x:.4f}" for x in row) for row in rng.random((32, 8))) + "\n")
    pat = load_duo_pattern(str(p))
    assert pat.shape == (32, 8) and pat.any() and (~pat).any()


def test_duo_errors(tmp_path):
    from flashquest_b200.duo.pattern import load_duo_pattern
    with pytest.raises(FileNotFoundError):
        load_duo_pattern(tmp_path / "nope.tsv")
    p = tmp_path / "empty.tsv"
    p.write_text("")
    with pytest.raises(ValueError, match="empty"):
        load_duo_pattern(p)
    r = tmp_path / "ragged.tsv"
    r.write_text("0.1\t0.2\n0.3\n")
    with pytest.raises(ValueError, match="has 1 cols, expected 2"):
        load_duo_pattern(r)
