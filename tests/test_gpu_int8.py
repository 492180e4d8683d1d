"""INT8 KV variant on the GPU: quantiser, dequantiser and page scores bit-exact against the oracle and
the reference's own outputs (tests/golden/int8.npz); sparse attention within 2e-3 (+ one output ulp) on O
and 1e-3 on the LSE; the persistent cache against the reference's test cases
(tests/test_persistent_cache.py, tests/test_kernel_sparse_edges.py)."""
import json
import os

import numpy as np
import pytest
import torch

import oracle
from tests._util import DTYPES, GOLDEN_DIR, bit_equal, from_bits, make_kv, make_q

pytestmark = pytest.mark.gpu
O_TOL, LSE_TOL = 2e-3, 1e-3


@pytest.fixture(scope="module")
def kq():
    from flashquest_b200.kernel import kv_quant
    return kv_quant


def _close(O, lse, Ow, lw, dtype):
    ulp = 2 ** -8 if dtype == torch.bfloat16 else 2 ** -11
    err = (O.float().cpu() - Ow).abs()
    assert (err <= O_TOL + ulp * Ow.abs()).all(), float(err.max())
    fin = torch.isfinite(lw)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    if fin.any():
        assert ((lse.cpu() - lw)[fin].abs() <= LSE_TOL).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("B,H,S,D,page", [(2, 2, 70, 64, 16), (1, 8, 1024, 128, 64), (1, 1, 33, 32, 8), (3, 2, 16, 256, 16)])
def test_quant_dequant_bit_exact(kq, dtype, B, H, S, D, page):
    K = make_kv(11, (B, H, S, D), dtype)
    V = make_kv(12, (B, H, S, D), dtype, outliers=())
    K[..., 5] = K[0, 0, 0, 5]                                  # a constant channel: the eps clamp
    want = oracle.quantize_k(K, page) + oracle.quantize_v(V)
    got = kq.quantize_k(K.cuda(), page) + kq.quantize_v(V.cuda())
    for g, w, name in zip(got, want, ("K_uint8", "K_scale", "K_mn", "V_uint8", "V_scale", "V_mn")):
        assert bit_equal(g.cpu(), w), name
    assert bit_equal(kq.dequantize_k(got[0], got[1], got[2], page).cpu(), oracle.dequantize_k(*want[:3], page))
    assert bit_equal(kq.dequantize_v(got[3], got[4], got[5]).cpu(), oracle.dequantize_v(*want[3:]))


def test_reference_goldens(kq):
    from flashquest_b200.eager.criticality import page_scores_int8_fast
    with open(os.path.join(GOLDEN_DIR, "int8.json")) as f:
        cases = json.load(f)["cases"]
    npz = np.load(os.path.join(GOLDEN_DIR, "int8.npz"))
    for c in cases:
        n, dt, page = c["name"], DTYPES[c["dtype"]], c["page"]
        g = lambda k, d=None: from_bits(npz[f"i8_{n}_{k}"], d)  # noqa: E731
        Ku, Ks, Km = kq.quantize_k(g("K", dt).cuda(), page)
        Vu, Vs, Vm = kq.quantize_v(g("V", dt).cuda())
        for got, key in ((Ku, "Ku"), (Ks, "Ks"), (Km, "Km"), (Vu, "Vu"), (Vs, "Vs"), (Vm, "Vm")):
            assert bit_equal(got.cpu(), g(key)), f"{n}:{key}"
        assert bit_equal(kq.dequantize_k(Ku, Ks, Km, page).cpu(), g("Kd")), n
        assert bit_equal(kq.dequantize_v(Vu, Vs, Vm).cpu(), g("Vd")), n
        Q = g("Q", DTYPES[c["q_dtype"]])
        sc = page_scores_int8_fast(Q.cuda(), Ks, Km).cpu()
        assert bit_equal(sc, oracle.page_scores_int8_fast(Q, g("Ks"), g("Km"))), n
        assert torch.allclose(sc, g("scores"), rtol=1e-4, atol=1e-3), n       # torch's matmul order is not fixed


def test_empty_and_errors(kq):
    Ku, Ks, Km = kq.quantize_k(torch.empty(1, 2, 0, 64, dtype=torch.bfloat16, device="cuda"), 16)
    assert Ku.shape == (1, 2, 0, 64) and Ks.shape == (1, 2, 0, 64)
    from flashquest_b200.kernel.sparse_fwd import flash_attn_sparse_fwd
    Q = torch.zeros(1, 2, 2, 64, dtype=torch.bfloat16, device="cuda")
    z = torch.zeros(1, 1, 64, 64, dtype=torch.uint8, device="cuda")
    m = torch.zeros(1, 1, 1, 64, dtype=torch.bfloat16, device="cuda")
    t = torch.zeros(1, 1, 64, 1, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NotImplementedError, match="decode-only"):
        flash_attn_sparse_fwd(Q, z, m, m, z, t, t, selection_mask=torch.ones(1, 2, 1, 1, dtype=torch.bool, device="cuda"))
    with pytest.raises(NotImplementedError, match="head_dim"):
        flash_attn_sparse_fwd(torch.zeros(1, 2, 1, 32, dtype=torch.bfloat16, device="cuda"), z[..., :32], m[..., :32], m[..., :32],
                              z[..., :32], t, t, selection_mask=torch.ones(1, 2, 1, 1, dtype=torch.bool, device="cuda"))


def _att_case(seed, B, Hq, Hkv, S, D, page, dtype, retention=0.3):
    K = make_kv(seed, (B, Hkv, S, D), dtype)
    V = make_kv(seed + 1, (B, Hkv, S, D), dtype, outliers=())
    Q = make_q(seed + 2, (B, Hq, 1, D), dtype)
    kv = oracle.quantize_k(K, page) + oracle.quantize_v(V)
    mask = oracle.select_pages_vectorized(oracle.page_scores_int8_fast(Q, kv[1], kv[2]), retention, 1, 1)
    return Q, kv, mask


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,S,D,page", [(1, 24, 8, 4096, 128, 16), (2, 6, 2, 320, 128, 16), (1, 4, 4, 256, 64, 8),
                                               (1, 4, 2, 1024, 128, 64), (2, 8, 2, 512, 64, 32), (1, 3, 3, 256, 128, 128)])
def test_attention_matches_oracle(dtype, B, Hq, Hkv, S, D, page):
    from flashquest_b200.kernel.sparse_fwd import flash_attn_sparse_fwd
    from flashquest_b200 import _lib
    Q, kv, mask = _att_case(21, B, Hq, Hkv, S, D, page, dtype)
    Ow, lw = oracle.sparse_attn_int8(Q, *kv, selection_mask=mask, page_size=page)
    dev = [t.cuda() for t in kv]
    for n_split in (None, 1, 3):
        O, lse = flash_attn_sparse_fwd(Q.cuda(), *dev, selection_mask=mask.cuda(), page_size=page, n_split=n_split)
        assert O.shape == (B, Hq, 1, D) and O.dtype == dtype and lse.shape == (B, Hq, 1)
        _close(O, lse, Ow, lw, dtype)
    O2, none = flash_attn_sparse_fwd(Q.cuda(), *dev, selection_mask=mask.cuda(), page_size=page, return_lse=False)
    assert none is None
    _close(O2, lse, Ow, lw, dtype)
    assert _lib.lib().fq_device_status() == 0


@pytest.mark.parametrize("S_kv", [64, 96, 100, 128, 192, 1023])
def test_partial_last_page(S_kv):
    # the reference's edge grid: S_kv not a multiple of the page size, every page selected
    from flashquest_b200.kernel.sparse_fwd import flash_attn_sparse_fwd
    K = make_kv(S_kv, (1, 1, S_kv, 64), torch.bfloat16)
    V = make_kv(S_kv + 1, (1, 1, S_kv, 64), torch.bfloat16, outliers=())
    Q = make_q(S_kv + 2, (1, 2, 1, 64), torch.bfloat16)
    kv = oracle.quantize_k(K, 64) + oracle.quantize_v(V)
    P = kv[1].shape[2]
    sel = torch.ones(1, 2, 1, P, dtype=torch.bool)
    Ow, lw = oracle.sparse_attn_int8(Q, *kv, selection_mask=sel, page_size=64)
    O, lse = flash_attn_sparse_fwd(Q.cuda(), *[t.cuda() for t in kv], selection_mask=sel.cuda(), page_size=64)
    _close(O, lse, Ow, lw, torch.bfloat16)


@pytest.mark.parametrize("n_rep", [2, 4, 8])
def test_gqa_selection_per_query_head(n_rep):
    from flashquest_b200.kernel.sparse_fwd import flash_attn_sparse_fwd
    H_kv, D, S_kv = 2, 64, 256
    H_q = H_kv * n_rep
    K = make_kv(n_rep, (1, H_kv, S_kv, D), torch.bfloat16)
    V = make_kv(n_rep + 1, (1, H_kv, S_kv, D), torch.bfloat16, outliers=())
    Q = make_q(n_rep + 2, (1, H_q, 1, D), torch.bfloat16)
    kv = oracle.quantize_k(K, 64) + oracle.quantize_v(V)
    sel = torch.zeros(1, H_q, 1, 4, dtype=torch.bool)
    for h in range(H_q):
        sel[0, h, 0, h % 4] = True
    sel[..., 0] = True
    sel[..., -1] = True
    Ow, lw = oracle.sparse_attn_int8(Q, *kv, selection_mask=sel, page_size=64)
    O, lse = flash_attn_sparse_fwd(Q.cuda(), *[t.cuda() for t in kv], selection_mask=sel.cuda(), page_size=64)
    _close(O, lse, Ow, lw, torch.bfloat16)


def test_empty_selection_and_tail():
    from flashquest_b200.kernel.sparse_fwd import flash_attn_sparse_fwd
    Q, kv, mask = _att_case(31, 2, 4, 2, 128, 64, 16, torch.bfloat16)
    dev = [t.cuda() for t in kv]
    none = torch.zeros_like(mask)
    none[1] = mask[1]                                        # batch row 0 attends nothing: O = 0, lse = -inf
    Ow, lw = oracle.sparse_attn_int8(Q, *kv, selection_mask=none, page_size=16)
    O, lse = flash_attn_sparse_fwd(Q.cuda(), *dev, selection_mask=none.cuda(), page_size=16)
    assert (O[0] == 0).all() and torch.isinf(lse[0]).all() and (lse[0] < 0).all()
    _close(O, lse, Ow, lw, torch.bfloat16)
    Kt, Vt = make_kv(41, (2, 2, 5, 64), torch.bfloat16), make_kv(42, (2, 2, 5, 64), torch.bfloat16, outliers=())
    Ow, lw = oracle.sparse_attn_int8(Q, *kv, selection_mask=none, page_size=16, K_partial=Kt, V_partial=Vt)
    O, lse = flash_attn_sparse_fwd(Q.cuda(), *dev, selection_mask=none.cuda(), page_size=16, K_partial=Kt.cuda(), V_partial=Vt.cuda())
    _close(O, lse, Ow, lw, torch.bfloat16)


# ---------------------------------------------------------------- persistent cache

def test_cache_allocation_and_streaming(kq):
    from flashquest_b200.cache.persistent_int8 import PersistentInt8KVCache
    cache = PersistentInt8KVCache(batch_size=1, num_layers=4, num_kv_heads=8, head_dim=128, max_seq_len=2048, page_size=64)
    assert cache.K_uint8.shape == (4, 1, 8, 2048, 128) and cache.K_uint8.dtype == torch.uint8
    assert cache.K_scale.shape == (4, 1, 8, 32, 128) and cache.K_scale.dtype == torch.bfloat16
    assert cache.V_scale.shape == (4, 1, 8, 2048, 1)
    assert cache.K_partial.shape == (4, 1, 8, 64, 128) and cache.K_partial.dtype == torch.bfloat16
    assert cache.get_seq_length(0) == 0 and cache.get_max_length() == 2048 and cache.kv_bits == 8

    cache = PersistentInt8KVCache(batch_size=2, num_layers=2, num_kv_heads=2, head_dim=64, max_seq_len=160, page_size=16)
    K = make_kv(51, (2, 2, 150, 64), torch.bfloat16)
    V = make_kv(52, (2, 2, 150, 64), torch.bfloat16, outliers=())
    # prefill of 37 tokens, then single tokens, then a chunk: every append path
    cuts = [0, 37] + list(range(38, 70)) + [150]
    for a, b in zip(cuts[:-1], cuts[1:]):
        cache.update_quantized(K[:, :, a:b].cuda(), V[:, :, a:b].cuda(), layer_idx=1)
        v = cache.get_views(1)
        assert v["seq_len"] == b and v["completed_len"] == b - b % 16 and v["partial_len"] == b % 16
        assert bit_equal(v["K_partial"].cpu(), K[:, :, b - b % 16:b])
        assert (cache.K_partial[1, :, :, b % 16:] == 0).all()          # stale staging rows are zeroed
    want = oracle.quantize_k(K[:, :, :144], 16) + oracle.quantize_v(V[:, :, :144])
    v = cache.get_views(1)
    for key, w in zip(("K_uint8", "K_scale", "K_mn", "V_uint8", "V_scale", "V_mn"), want):
        assert bit_equal(v[key].cpu(), w), key
    assert cache.get_seq_length(0) == 0
    with pytest.raises(RuntimeError, match="exceeds max_seq_len"):
        cache.update_quantized(K[:, :, :11].cuda(), V[:, :, :11].cuda(), layer_idx=1)
    with pytest.raises(IndexError):
        cache.get_views(2)
    with pytest.raises(NotImplementedError):
        cache.update(None, None, 0)


@pytest.mark.parametrize("D", [128, 64])
def test_attention_with_rows_that_are_not_16_byte_aligned(D):
    """Code rows cut out of a wider tensor (token stride D + 4 bytes) are 4-byte but not 16-byte aligned: the call
    takes the warp-per-token kernel instead of the quarter-warp one; both agree with the oracle."""
    from flashquest_b200.kernel.sparse_fwd import flash_attn_sparse_fwd
    from flashquest_b200 import _lib
    B, Hq, Hkv, S, page, dtype = 1, 4, 2, 640, 16, torch.bfloat16
    Q, kv, mask = _att_case(33, B, Hq, Hkv, S, D, page, dtype)
    Ow, lw = oracle.sparse_attn_int8(Q, *kv, selection_mask=mask, page_size=page)
    dev = [t.cuda() for t in kv]
    wideK = torch.zeros(B, Hkv, S, D + 4, dtype=torch.uint8, device="cuda")
    wideV = torch.zeros_like(wideK)
    wideK[..., :D], wideV[..., :D] = dev[0], dev[3]
    Kc, Vc = wideK[..., :D], wideV[..., :D]
    assert Kc.stride(2) == D + 4 and Kc.stride(3) == 1
    O, lse = flash_attn_sparse_fwd(Q.cuda(), Kc, dev[1], dev[2], Vc, dev[4], dev[5], selection_mask=mask.cuda(), page_size=page)
    _close(O, lse, Ow, lw, dtype)
    O2, lse2 = flash_attn_sparse_fwd(Q.cuda(), *dev, selection_mask=mask.cuda(), page_size=page)
    _close(O2, lse2, Ow, lw, dtype)
    assert _lib.lib().fq_device_status() == 0
