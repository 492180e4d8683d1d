"""Page scoring, top-k selection and compact index vs the oracle / reference goldens."""
import math

import pytest
import torch

import oracle
from tests._util import DTYPES, bit_equal, make_kv, make_q

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from flashquest_b200.eager import criticality, selection

    class O:
        scores = staticmethod(criticality.page_scores_int4_fast)
        select = staticmethod(selection.select_pages_vectorized)
        select_compact = staticmethod(selection.select_pages_compact)
        compact = staticmethod(selection.build_compact_selection)
    return O


def _meta(seed, B, Hkv, P, D, page=16, dtype=torch.bfloat16):
    K = make_kv(seed, (B, Hkv, P * page, D), dtype)
    _, Ks, Km = oracle.quantize_k_int4(K, page)
    return Ks, Km


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("B,Hq,Hkv,P,D", [(1, 24, 8, 256, 128), (2, 6, 2, 37, 128), (1, 4, 4, 19, 64),
                                          (1, 8, 1, 50, 128), (1, 10, 2, 21, 32), (1, 6, 3, 9, 256)])
def test_scores_bit_exact_vs_oracle(ops, dtype, B, Hq, Hkv, P, D):
    Ks, Km = _meta(1, B, Hkv, P, D)
    Q = make_q(2, (B, Hq, 1, D), dtype)
    want = oracle.page_scores_int4_fast(Q, Ks, Km)
    got = ops.scores(Q.cuda(), Ks.cuda(), Km.cuda())
    assert got.shape == (B, Hq, 1, P) and got.dtype == torch.float32
    assert bit_equal(got.cpu(), want)


def test_scores_reference_goldens_and_views(golden, ops):
    for case in golden.meta["chain"]:
        n, dt = case["name"], DTYPES[case["dtype"]]
        Q = golden.get("chain", f"{n}_Q", dtype=dt).cuda()
        Ks, Km = golden.get("chain", f"{n}_Ks").cuda(), golden.get("chain", f"{n}_Km").cuda()
        want = golden.get("chain", f"{n}_scores")
        got = ops.scores(Q, Ks, Km).cpu()
        assert torch.allclose(got, want, rtol=1e-4, atol=1e-4), n
        # metadata living in a larger preallocated cache (strided view)
        big_s = torch.zeros(Ks.shape[0], Ks.shape[1], Ks.shape[2] + 5, Ks.shape[3], dtype=Ks.dtype, device="cuda")
        big_m = torch.zeros_like(big_s)
        big_s[:, :, : Ks.shape[2]], big_m[:, :, : Ks.shape[2]] = Ks, Km
        got2 = ops.scores(Q, big_s[:, :, : Ks.shape[2]], big_m[:, :, : Ks.shape[2]]).cpu()
        assert bit_equal(got, got2), n
    with pytest.raises(ValueError, match="divisible"):
        ops.scores(torch.zeros(1, 5, 1, 128, device="cuda"), torch.zeros(1, 2, 4, 128, dtype=torch.bfloat16, device="cuda"),
                   torch.zeros(1, 2, 4, 128, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("P", [1, 5, 31, 32, 33, 256, 1000, 2048, 5000, 32768, 60000])
@pytest.mark.parametrize("retention", [0.0, 0.1, 0.25, 1.0])
def test_select_matches_oracle(ops, P, retention):
    torch.manual_seed(P)
    B, H = 2, 3
    scores = torch.randn(B, H, 1, P)
    scores[0, 0, 0, ::7] = 0.5            # many exact ties
    scores[1, 1, 0, :] = -0.0             # a whole row of equal scores
    if P > 3:
        scores[1, 2, 0, 1] = float("inf")
        scores[1, 2, 0, 2] = float("-inf")
    for sinks, window, kms in ((0, 0, None), (1, 1, None), (4, 2, math.ceil(retention * (P + 8))), (3, 50000, 3)):
        want = oracle.select_pages_vectorized(scores, retention, sinks, window, k_max_static=kms)
        got = ops.select(scores.cuda(), retention, sinks, window, k_max_static=kms)
        assert got.dtype == torch.bool and got.shape == (B, H, 1, P)
        assert torch.equal(got.cpu(), want), (P, retention, sinks, window, kms)
        bucket = max(1, (kms if kms is not None else math.ceil(retention * P)) + sinks + min(window, P))
        for bk in (bucket, 7):
            wc = oracle.build_compact_selection(want, bk)
            gc, gcount = ops.select_compact(scores.cuda(), retention, sinks, window, k_max_static=kms,
                                            BUCKET_MAX=bk, return_count=True)
            assert torch.equal(gc.cpu(), wc)
            assert torch.equal(gcount.cpu().long(), want.sum(-1).squeeze(-1))
            assert torch.equal(ops.compact(got, bk).cpu(), wc)


def test_select_per_head_retention_and_errors(ops):
    torch.manual_seed(0)
    scores = torch.randn(2, 6, 1, 300)
    r = torch.tensor([0.25, 0.0, 0.5, 1.0, 0.01, 0.2])
    want = oracle.select_pages_vectorized(scores, r, 2, 1)
    assert torch.equal(ops.select(scores.cuda(), r.cuda(), 2, 1).cpu(), want)
    assert torch.equal(ops.select(scores.cuda(), r, 2, 1, k_max_static=150).cpu(),
                       oracle.select_pages_vectorized(scores, r, 2, 1, k_max_static=150))
    with pytest.raises(ValueError, match="retention"):
        ops.select(scores.cuda(), 1.5, 0, 0)
    with pytest.raises(ValueError, match="per-head retention"):
        ops.select(scores.cuda(), torch.tensor([0.5]), 0, 0)
    with pytest.raises(ValueError, match="BUCKET_MAX"):
        ops.compact(torch.zeros(1, 1, 1, 4, dtype=torch.bool, device="cuda"), 0)
    with pytest.raises(ValueError, match="bool"):
        ops.compact(torch.zeros(1, 1, 1, 4, dtype=torch.int32, device="cuda"), 4)


def test_select_reference_goldens(golden, ops):
    hw = golden.meta["handwritten"]
    c = hw["select_zero_retention"]
    m = ops.select(torch.zeros(1, 1, 1, c["P"], device="cuda"), c["retention"], c["sinks"], c["window"])
    assert m.flatten().int().tolist() == c["mask"]
    for key in ("select_topk", "select_round_up"):
        c = hw[key]
        m = ops.select(torch.tensor(c["scores"], device="cuda").reshape(1, 1, 1, -1), c["retention"], 0, 0)
        assert m.flatten().int().tolist() == c["mask"], key
    for case in golden.meta["chain"]:
        n = case["name"]
        scores = golden.get("chain", f"{n}_scores").cuda()
        mask = ops.select(scores, case["retention"], case["sinks"], case["window"], k_max_static=case["k_max_static"])
        assert torch.equal(mask.cpu(), golden.get("chain", f"{n}_mask", as_bool=True)), n
        comp = ops.compact(mask, case["bucket"])
        assert torch.equal(comp.cpu(), golden.get("chain", f"{n}_comp")), n
        r_head = torch.tensor([case["retention"] if h % 2 == 0 else 0.0 for h in range(case["Hq"])])
        assert torch.equal(ops.select(scores, r_head, case["sinks"], case["window"]).cpu(),
                           golden.get("chain", f"{n}_mask_ph", as_bool=True)), n


def test_compact_sentinels_and_truncation(ops, golden):
    c = golden.meta["handwritten"]["compact_basic"]
    mask = torch.zeros(1, 1, 1, c["P"], dtype=torch.bool, device="cuda")
    mask[..., c["selected"]] = True
    for b in c["buckets"]:
        out = ops.compact(mask, b)
        assert out.shape == (1, 1, 1, b) and out.dtype == torch.int32
        assert sorted(out[0, 0, 0, :3].tolist()) == c["selected"] and (out[0, 0, 0, 3:] == -1).all()
    assert (ops.compact(torch.zeros(1, 1, 1, 8, dtype=torch.bool, device="cuda"), 4) == -1).all()
    full = ops.compact(torch.ones(1, 1, 1, 4, dtype=torch.bool, device="cuda"), 2)   # keeps the highest ids
    assert full.flatten().tolist() == [3, 2]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,Hq,Hkv,P,D", [(1, 24, 8, 2048, 128), (2, 6, 2, 37, 128), (1, 4, 4, 19, 64), (1, 8, 2, 257, 128),
                                          (1, 2, 1, 1, 128), (1, 10, 5, 21, 32), (1, 6, 3, 300, 256), (1, 3, 1, 4100, 128)])
def test_fused_score_select_equals_separate_calls(ops, dtype, B, Hq, Hkv, P, D):
    """fq_score_select against the oracle and against the two separate launches: the same bits in the
    scores, the same compact list, with and without the early metadata request."""
    from flashquest_b200.eager.selection import score_select_compact
    Ks, Km = _meta(3, B, Hkv, P, D)
    Ks[:, :, P // 2] = Ks[:, :, 0]             # two pages with identical metadata: an exact score tie
    Km[:, :, P // 2] = Km[:, :, 0]
    Q = make_q(4, (B, Hq, 1, D), dtype)
    want_s = oracle.page_scores_int4_fast(Q, Ks, Km)
    r_head = torch.tensor([0.25 if h % 3 else 0.0 for h in range(Hq)])
    for retention, sinks, window in ((0.25, 1, 1), (r_head, 4, 2), (1.0, 0, 0), (0.0, 0, 3)):
        rmax = float(retention.max()) if isinstance(retention, torch.Tensor) else retention
        kms = math.ceil(rmax * P)
        bucket = max(1, kms + sinks + window)
        want_m = oracle.select_pages_vectorized(want_s, retention, sinks, window, k_max_static=kms)
        want_c = oracle.build_compact_selection(want_m, bucket)
        r_dev = retention.cuda() if isinstance(retention, torch.Tensor) else retention
        for fresh in (0, P, max(P - 1, 0), P // 2):
            s, c = score_select_compact(Q.cuda(), Ks.cuda(), Km.cuda(), r_dev, sinks, window, k_max_static=kms,
                                        BUCKET_MAX=bucket, first_fresh_page=fresh)
            assert s.shape == (B, Hq, 1, P) and c.shape == (B, Hq, 1, bucket)
            assert bit_equal(s.cpu(), want_s), (retention, fresh)
            assert torch.equal(c.cpu(), want_c), (retention, fresh)
    s2 = ops.scores(Q.cuda(), Ks.cuda(), Km.cuda())
    assert bit_equal(s2.cpu(), want_s)


def test_fused_score_select_int8_levels_and_errors():
    from flashquest_b200.eager.selection import score_select_compact
    K = make_kv(9, (1, 2, 40 * 16, 128), torch.bfloat16)
    _, Ks, Km = oracle.quantize_k(K, 16)
    Q = make_q(10, (1, 4, 1, 128), torch.bfloat16)
    want_s = oracle.page_scores_int8_fast(Q, Ks, Km)
    want_c = oracle.build_compact_selection(oracle.select_pages_vectorized(want_s, 0.3, 1, 1, k_max_static=12), 14)
    s, c = score_select_compact(Q.cuda(), Ks.cuda(), Km.cuda(), 0.3, 1, 1, k_max_static=12, BUCKET_MAX=14, levels=255)
    assert bit_equal(s.cpu(), want_s) and torch.equal(c.cpu(), want_c)
    with pytest.raises(ValueError, match="levels"):
        score_select_compact(Q.cuda(), Ks.cuda(), Km.cuda(), 0.3, 1, 1, k_max_static=12, BUCKET_MAX=14, levels=16)
    with pytest.raises(NotImplementedError):      # 8 query heads per KV head: outside the fused launch
        score_select_compact(make_q(1, (1, 16, 1, 128), torch.bfloat16).cuda(), Ks.cuda(), Km.cuda(), 0.3, 1, 1,
                             k_max_static=12, BUCKET_MAX=14)
