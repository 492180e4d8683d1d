"""TurboQuant K3-V3 path: WHT, plane packing, cache, attention, tail + merge — against the
oracle and the reference goldens."""
import pytest
import torch

import oracle
from tests._util import DTYPES, bit_equal, make_kv, make_q

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    from flashquest_b200.kernel import kv_quant, wht
    from flashquest_b200.kernel.sparse_turbo_fwd import flash_attn_sparse_turbo_fwd
    from flashquest_b200.cache.persistent_turbo import PersistentTurboKVCache
    from flashquest_b200.eager import tail_merge

    class N:
        pass
    n = N()
    n.kvq, n.wht, n.att, n.Cache, n.tm = kv_quant, wht.wht_along_head_dim, flash_attn_sparse_turbo_fwd, PersistentTurboKVCache, tail_merge
    return n


def test_wht_bit_exact(golden, T):
    for case in golden.meta["turbo"]:
        n, dt = case["name"], DTYPES[case["dtype"]]
        K = golden.get("turbo", f"t_{n}_K", dtype=dt)
        assert bit_equal(T.wht(K.cuda()).cpu(), golden.get("turbo", f"t_{n}_W", dtype=dt)), n
    for D in (2, 8, 32, 64, 256, 1024):
        for dt in (torch.float32, torch.float16, torch.bfloat16):
            x = make_q(D, (3, 5, D), dt)
            assert bit_equal(T.wht(x.cuda()).cpu(), oracle.wht_along_head_dim(x)), (D, dt)
    x = torch.randn(4, 7, 128, device="cuda")
    assert (T.wht(T.wht(x)) - x).abs().max() < 1e-4
    with pytest.raises(ValueError, match="power of 2"):
        T.wht(torch.randn(2, 96, device="cuda"))


def test_turbo_quant_matches_reference_and_oracle(golden, T):
    for case in golden.meta["turbo"]:
        n, dt = case["name"], DTYPES[case["dtype"]]
        D = case["shape"][-1]
        K = golden.get("turbo", f"t_{n}_K", dtype=dt)
        V = golden.get("turbo", f"t_{n}_V", dtype=dt)
        got = T.kvq.quantize_k_turbo(K.cuda(), case["page"]) + T.kvq.quantize_v_turbo(V.cuda())
        want = oracle.quantize_k_turbo(K, case["page"]) + oracle.quantize_v_turbo(V)
        for g, w, key in zip(got, want, ("Kmsb", "Klsb", "Kst", "Ksr", "Kmr", "Vmsb", "Vlsb", "Vst")):
            assert bit_equal(g.cpu(), w), f"{n}:{key} vs oracle"
            assert bit_equal(g.cpu(), golden.get("turbo", f"t_{n}_{key}")), f"{n}:{key} vs reference"
        Kd = T.kvq.dequantize_k_turbo(got[0], got[1], got[2], head_dim=D)
        assert bit_equal(Kd.cpu(), golden.get("turbo", f"t_{n}_Kd")), n
    with pytest.raises(ValueError, match="multiple of 8"):
        T.kvq.quantize_k_turbo(torch.randn(1, 1, 16, 12, device="cuda"), 16)


def test_turbo_cache_appends(T):
    B, H, D, page, S_max = 2, 2, 128, 16, 200
    cache = T.Cache(batch_size=B, num_layers=2, num_kv_heads=H, head_dim=D, max_seq_len=S_max, page_size=page,
                    device="cuda", dtype=torch.bfloat16)
    assert cache.kv_bits == 3
    K = make_kv(61, (B, H, S_max, D), torch.bfloat16)
    V = make_kv(62, (B, H, S_max, D), torch.bfloat16, outliers=())
    pos = 0
    for chunk in [2 * page + 3] + [1] * (page + 2) + [page - 1, 2 * page, 5]:
        cache.update_quantized(K[:, :, pos:pos + chunk].cuda(), V[:, :, pos:pos + chunk].cuda(), 1)
        pos += chunk
        v = cache.get_views(1)
        n = v["completed_len"]
        assert v["seq_len"] == pos and v["partial_len"] == pos - n
        if n:
            wk = oracle.quantize_k_turbo(K[:, :, :n], page)
            wv = oracle.quantize_v_turbo(V[:, :, :n])
            for key, w in zip(("K_msb", "K_lsb", "K_scale_turbo", "K_scale_raw", "K_mn_raw"), wk):
                assert bit_equal(v[key].cpu(), w), (key, pos)
            for key, w in zip(("V_msb", "V_lsb", "V_scale_turbo"), wv):
                assert bit_equal(v[key].cpu(), w), (key, pos)
        assert bit_equal(v["K_partial"].cpu(), K[:, :, n:pos].contiguous())
        assert bit_equal(v["V_partial"].cpu(), V[:, :, n:pos].contiguous())
    with pytest.raises(RuntimeError, match="exceeds.*max_seq_len"):
        cache.update_quantized(K[:, :, :150].cuda(), V[:, :, :150].cuda(), 1)
    with pytest.raises(IndexError, match="layer_idx"):
        cache.get_views(2)
    with pytest.raises(ValueError, match="multiple of 8"):
        T.Cache(batch_size=1, num_layers=1, num_kv_heads=1, head_dim=12, max_seq_len=32, device="cuda")
    with pytest.raises(ValueError, match="power of 2"):
        T.Cache(batch_size=1, num_layers=1, num_kv_heads=1, head_dim=24, max_seq_len=32, device="cuda")


@pytest.mark.parametrize("B,Hq,Hkv,S,D,page", [(1, 6, 2, 128, 128, 16), (2, 8, 4, 512, 128, 16), (1, 4, 2, 256, 64, 32),
                                               (1, 24, 8, 4096, 128, 16)])
def test_turbo_attention(golden, T, B, Hq, Hkv, S, D, page):
    K = make_kv(71, (B, Hkv, S, D), torch.bfloat16)
    V = make_kv(72, (B, Hkv, S, D), torch.bfloat16, outliers=())
    Q = make_q(73, (B, Hq, 1, D), torch.bfloat16)
    Km, Kl, Kst, Ksr, Kmr = oracle.quantize_k_turbo(K, page)
    Vm, Vl, Vst = oracle.quantize_v_turbo(V)
    mask = oracle.select_pages_vectorized(oracle.page_scores_int4_fast(Q, Ksr, Kmr), 0.3, 1, 1)
    Ow, lw = oracle.sparse_attn_turbo(Q, Km, Kl, Kst, Vm, Vl, Vst, selection_mask=mask, page_size=page)
    dev = [t.cuda() for t in (Km, Kl, Kst, Vm, Vl, Vst)]
    for n_split in (1, 3, None):
        O, lse = T.att(Q.cuda(), *dev, selection_mask=mask.cuda(), page_size=page, n_split=n_split)
        assert O.shape == (B, Hq, 1, D) and O.dtype == torch.bfloat16 and lse.shape == (B, Hq, 1)
        # Q and O pass through bf16 rotations as in the reference wrapper: bf16-level agreement
        assert (O.float().cpu() - Ow).abs().max() < 2e-2, float((O.float().cpu() - Ow).abs().max())
        assert (lse.cpu() - lw).abs().max() < 2e-2
    if (B, Hq, S) == (1, 6, 128):
        g = lambda k, **kw: golden.get("turbo", f"ta_{k}", **kw)  # noqa: E731
        O, lse = T.att(g("Q").cuda(), g("Kmsb").cuda(), g("Klsb").cuda(), g("Kst").cuda(), g("Vmsb").cuda(), g("Vlsb").cuda(),
                       g("Vst").cuda(), selection_mask=g("mask", as_bool=True).cuda(), page_size=16)
        assert (O.float().cpu() - g("O").float()).abs().max() < 5e-2      # the reference's own test bound
        assert (lse.cpu() - g("lse")).abs().max() < 5e-2
    O0, l0 = T.att(Q.cuda(), *dev, selection_mask=torch.zeros_like(mask).cuda(), page_size=page)
    assert (O0 == 0).all() and torch.isinf(l0).all()


def test_tail_attention_and_merge(golden, T):
    for case in golden.meta["chain"]:
        n = case["name"]
        if f"{n}_Otail" not in golden.npz("chain"):
            continue
        g = lambda k, **kw: golden.get("chain", f"{n}_{k}", **kw)  # noqa: E731
        Q, Kt, Vt = g("Q").cuda(), g("Ktail").cuda(), g("Vtail").cuda()
        Ot, lt = T.tm._bf16_dense_attn_with_lse(Q, Kt, Vt)
        assert (Ot.float().cpu() - g("Otail").float()).abs().max() < 1e-2
        assert (lt.cpu() - g("lsetail")).abs().max() < 1e-3
        Om = T.tm._merge_two_attentions(g("O").to(torch.bfloat16).cuda(), g("lse").cuda(), g("Otail").cuda(), g("lsetail").cuda())
        assert Om.dtype == torch.bfloat16
        assert (Om.float().cpu() - g("Omerged").float()).abs().max() < 8e-3     # one bf16 ulp of the merged values
    torch.manual_seed(0)
    Op, lp = torch.randn(3, 2, 4, 1, 64), torch.randn(3, 2, 4, 1)
    lp[1, 0, 0] = float("-inf")
    Ow, lw = oracle.lse_merge(Op, lp)
    O, lse = T.tm.merge_attentions(Op.cuda(), lp.cuda())
    assert torch.allclose(O.cpu(), Ow, atol=1e-5) and torch.allclose(lse.cpu(), lw, atol=1e-5)
