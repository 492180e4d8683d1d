"""Sparse INT4 decode attention (split-K, tail, LSE merge) vs the oracle and the goldens.

Tolerance: north-star bound max-abs 2e-3 on O (fp16 / bf16 output rounding included where
|O| < 1, plus one output ulp) and 1e-3 on the LSE."""
import math

import pytest
import torch

import oracle
from tests._util import DTYPES, make_kv, make_q

pytestmark = pytest.mark.gpu
O_TOL, LSE_TOL = 2e-3, 1e-3


@pytest.fixture(scope="module")
def att():
    from flashquest_b200.kernel.sparse_int4_fwd import flash_attn_sparse_int4_fwd
    from flashquest_b200.kernel.sparse_int4_fwd_compact import flash_attn_sparse_int4_fwd_compact
    from flashquest_b200 import _lib

    class A:
        mask = staticmethod(flash_attn_sparse_int4_fwd)
        compact = staticmethod(flash_attn_sparse_int4_fwd_compact)
        status = staticmethod(lambda: _lib.lib().fq_device_status())
    return A


def _close(O, lse, Ow, lw, dtype):
    ulp = 2 ** -8 if dtype == torch.bfloat16 else 2 ** -11
    tol = O_TOL + ulp * Ow.abs()
    assert ((O.float().cpu() - Ow).abs() <= tol).all(), float((O.float().cpu() - Ow).abs().max())
    fin = torch.isfinite(lw)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    assert ((lse.cpu() - lw)[fin].abs() <= LSE_TOL).all() if fin.any() else True


def _case(seed, B, Hq, Hkv, S, D, page, dtype, retention=0.25, sinks=1, window=1):
    K = make_kv(seed, (B, Hkv, S, D), dtype)
    V = make_kv(seed + 1, (B, Hkv, S, D), dtype, outliers=())
    Q = make_q(seed + 2, (B, Hq, 1, D), dtype)
    kv = oracle.quantize_k_int4(K, page) + oracle.quantize_v_int4(V)
    scores = oracle.page_scores_int4_fast(Q, kv[1], kv[2])
    mask = oracle.select_pages_vectorized(scores, retention, sinks, window)
    return Q, kv, mask


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,S,D,page", [(1, 24, 8, 4096, 128, 16), (2, 6, 2, 320, 128, 16), (1, 4, 4, 256, 64, 8),
                                               (1, 4, 2, 1024, 128, 64), (2, 8, 2, 512, 64, 32), (1, 2, 1, 128, 128, 8),
                                               (1, 3, 3, 256, 128, 128)])
def test_attention_matches_oracle(att, dtype, B, Hq, Hkv, S, D, page):
    Q, kv, mask = _case(7, B, Hq, Hkv, S, D, page, dtype)
    Ow, lw = oracle.sparse_attn_int4(Q, *kv, selection_mask=mask, page_size=page)
    dev = [t.cuda() for t in kv]
    O, lse = att.mask(Q.cuda(), *dev, selection_mask=mask.cuda(), page_size=page)
    assert O.shape == (B, Hq, 1, D) and O.dtype == dtype and lse.shape == (B, Hq, 1)
    _close(O, lse, Ow, lw, dtype)
    comp = oracle.build_compact_selection(mask, int(mask.sum(-1).max()) + 3).cuda()
    for n_split in (1, 2, 5, None):
        O2, lse2 = att.compact(Q.cuda(), *dev, selected_page_ids=comp, page_size=page, n_split=n_split)
        _close(O2, lse2, Ow, lw, dtype)
    O3, none = att.compact(Q.cuda(), *dev, selected_page_ids=comp.squeeze(2), page_size=page, return_lse=False)
    assert none is None
    _close(O3, lse, Ow, lw, dtype)
    assert att.status() == 0


def test_attention_reference_goldens(golden, att):
    for case in golden.meta["chain"]:
        n, dt = case["name"], DTYPES[case["dtype"]]
        g = lambda k, **kw: golden.get("chain", f"{n}_{k}", **kw)  # noqa: E731
        Q = g("Q", dtype=dt).cuda()
        dev = [g(k).cuda() for k in ("Kp", "Ks", "Km", "Vp", "Vs", "Vm")]
        O, lse = att.mask(Q, *dev, selection_mask=g("mask", as_bool=True).cuda(), page_size=case["page"])
        _close(O, lse, g("O"), g("lse"), dt)
        O2, lse2 = att.compact(Q, *dev, selected_page_ids=g("comp").cuda(), page_size=case["page"])
        _close(O2, lse2, g("O"), g("lse"), dt)
        if case["tail"]:
            Kt, Vt = g("Ktail", dtype=dt).cuda(), g("Vtail", dtype=dt).cuda()
            O3, lse3 = att.compact(Q, *dev, selected_page_ids=g("comp").cuda(), page_size=case["page"],
                                   K_partial=Kt, V_partial=Vt)
            _close(O3, lse3, g("Oall"), g("lse_all"), dt)
            if f"{n}_Omerged" in golden.npz("chain"):
                # the reference dispatcher's own result (parts rounded to bf16 before the merge)
                assert (O3.float().cpu() - g("Omerged").float()).abs().max() < 2e-2


def test_sentinels_order_and_empty(att):
    B, Hq, Hkv, S, D, page = 1, 6, 2, 512, 128, 16
    Q, kv, mask = _case(21, B, Hq, Hkv, S, D, page, torch.bfloat16)
    dev = [t.cuda() for t in kv]
    Ow, lw = oracle.sparse_attn_int4(Q, *kv, selection_mask=mask, page_size=page)
    comp = oracle.build_compact_selection(mask, 64)
    # shuffle the list and scatter sentinels / out-of-range ids through it: result unchanged
    gen = torch.Generator().manual_seed(0)
    perm = torch.stack([torch.randperm(64, generator=gen) for _ in range(B * Hq)]).reshape(B, Hq, 1, 64)
    shuffled = torch.gather(comp, -1, perm)
    padded = torch.full((B, Hq, 1, 100), -1, dtype=torch.int32)
    padded[..., 10:74] = shuffled
    padded[..., 3] = -7
    padded[..., 90] = S // page + 5      # beyond the last page: ignored
    O, lse = att.compact(Q.cuda(), *dev, selected_page_ids=padded.cuda(), page_size=page, n_split=3)
    _close(O, lse, Ow, lw, torch.bfloat16)
    # nothing selected: O == 0, lse == -inf
    none = torch.full((B, Hq, 1, 8), -1, dtype=torch.int32, device="cuda")
    O0, l0 = att.compact(Q.cuda(), *dev, selected_page_ids=none, page_size=page)
    assert (O0 == 0).all() and torch.isinf(l0).all() and (l0 < 0).all()
    O0, l0 = att.mask(Q.cuda(), *dev, selection_mask=torch.zeros_like(mask).cuda(), page_size=page)
    assert (O0 == 0).all() and torch.isinf(l0).all()
    # one head with an empty list, others not
    some = comp.clone()
    some[0, 2] = -1
    O1, l1 = att.compact(Q.cuda(), *dev, selected_page_ids=some.cuda(), page_size=page, n_split=4)
    assert (O1[0, 2] == 0).all() and torch.isinf(l1[0, 2]).all()
    _close(O1[:, :2], l1[:, :2], Ow[:, :2], lw[:, :2], torch.bfloat16)
    assert att.status() == 0


def test_ragged_last_page_tail_and_views(att):
    B, Hq, Hkv, D, page = 2, 6, 2, 128, 16
    S_alloc, S_kv = 400, 296 + 5          # last page holds 5 valid tokens
    K = make_kv(31, (B, Hkv, S_kv, D), torch.float16)
    V = make_kv(32, (B, Hkv, S_kv, D), torch.float16, outliers=())
    Q = make_q(33, (B, Hq, 1, D), torch.float16)
    kv = oracle.quantize_k_int4(K, page) + oracle.quantize_v_int4(V)
    P = kv[1].shape[2]
    mask = oracle.select_pages_vectorized(oracle.page_scores_int4_fast(Q, kv[1], kv[2]), 0.3, 1, 2)
    Kt, Vt = make_kv(34, (B, Hkv, 11, D), torch.float16), make_kv(35, (B, Hkv, 11, D), torch.float16, outliers=())
    Ow, lw = oracle.sparse_attn_int4(Q, *kv, selection_mask=mask, page_size=page, K_partial=Kt, V_partial=Vt)
    # cache-like storage: (L,B,H,S_alloc,...) with the layer's view sliced out
    def store(t, rows):
        big = torch.zeros(2, B, Hkv, rows, *t.shape[3:], dtype=t.dtype, device="cuda")
        big[1, :, :, : t.shape[2]] = t.cuda()
        return big[1, :, :, : t.shape[2]]
    dev = [store(kv[0], S_alloc), store(kv[1], S_alloc // page), store(kv[2], S_alloc // page),
           store(kv[3], S_alloc), store(kv[4], S_alloc), store(kv[5], S_alloc)]
    part = torch.zeros(B, Hkv, page, D, dtype=torch.float16, device="cuda")
    part2 = torch.zeros_like(part)
    part[:, :, :11], part2[:, :, :11] = Kt.cuda(), Vt.cuda()
    for n_split in (1, 3):
        O, lse = att.mask(Q.cuda(), *dev, selection_mask=mask.cuda(), page_size=page,
                          K_partial=part[:, :, :11], V_partial=part2[:, :, :11], n_split=n_split)
        _close(O, lse, Ow, lw, torch.float16)
    # tail only (no completed page yet)
    Oo, lo = oracle.sparse_attn_int4(Q, *kv, selected_page_ids=torch.full((B, Hq, 1, 1), -1, dtype=torch.int32),
                                     page_size=page, K_partial=Kt, V_partial=Vt)
    O, lse = att.compact(Q.cuda(), *dev, selected_page_ids=torch.full((B, Hq, 1, 1), -1, dtype=torch.int32, device="cuda"),
                         page_size=page, K_partial=Kt.cuda(), V_partial=Vt.cuda())
    _close(O, lse, Oo, lo, torch.float16)
    assert att.status() == 0


def test_argument_errors(att):
    Q = torch.zeros(1, 4, 1, 128, dtype=torch.bfloat16, device="cuda")
    Kp = torch.zeros(1, 2, 32, 64, dtype=torch.uint8, device="cuda")
    Ks = torch.zeros(1, 2, 2, 128, dtype=torch.bfloat16, device="cuda")
    Vs = torch.zeros(1, 2, 32, 1, dtype=torch.bfloat16, device="cuda")
    m = torch.ones(1, 4, 1, 2, dtype=torch.bool, device="cuda")
    with pytest.raises(NotImplementedError, match="decode-only"):
        att.mask(Q.expand(1, 4, 2, 128), Kp, Ks, Ks, Kp, Vs, Vs, selection_mask=m, page_size=16)
    with pytest.raises(NotImplementedError, match="head_dim"):
        att.mask(torch.zeros(1, 4, 1, 32, dtype=torch.bfloat16, device="cuda"), Kp[..., :16], Ks[..., :32], Ks[..., :32],
                 Kp[..., :16], Vs, Vs, selection_mask=m, page_size=16)
    with pytest.raises(AssertionError):
        att.mask(Q.float(), Kp, Ks, Ks, Kp, Vs, Vs, selection_mask=m, page_size=16)
    with pytest.raises(ValueError, match="3D or 4D"):
        att.compact(Q, Kp, Ks, Ks, Kp, Vs, Vs, selected_page_ids=torch.zeros(4, dtype=torch.int32, device="cuda"), page_size=16)


def test_full_size_invariances(att):
    """BASELINE config 1 size (one layer, 32k, page 16): split-count invariance, mask ==
    compact, and agreement with the oracle on a subset of heads."""
    from flashquest_b200.eager.criticality import page_scores_int4_fast
    from flashquest_b200.eager.selection import select_pages_compact
    from flashquest_b200.kernel.kv_quant import quantize_k_int4, quantize_v_int4
    B, Hq, Hkv, S, D, page = 1, 24, 8, 32768, 128, 16
    g = torch.Generator(device="cuda").manual_seed(5)
    K = torch.randn(B, Hkv, S, D, device="cuda", generator=g)
    K[..., [3, 17, 64, 100]] *= 8
    K, V = K.half(), torch.randn(B, Hkv, S, D, device="cuda", generator=g).half()
    Q = torch.randn(B, Hq, 1, D, device="cuda", generator=g).half()
    kv = quantize_k_int4(K, page) + quantize_v_int4(V)
    scores = page_scores_int4_fast(Q, kv[1], kv[2])
    comp, mask = select_pages_compact(scores, 0.25, 1, 1, k_max_static=512, BUCKET_MAX=514, return_mask=True)
    assert int(mask.sum(-1).max()) <= 514 and int(mask.sum(-1).min()) >= 512
    base, lbase = att.compact(Q, *kv, selected_page_ids=comp, page_size=page, n_split=1)
    for n_split in (2, 7, 12, 33):
        O, lse = att.compact(Q, *kv, selected_page_ids=comp, page_size=page, n_split=n_split)
        assert (O.float() - base.float()).abs().max() <= 1e-3 and (lse - lbase).abs().max() <= 1e-4
    Om, lm = att.mask(Q, *kv, selection_mask=mask, page_size=page)
    assert (Om.float() - base.float()).abs().max() <= 1e-3
    cpu = [t.cpu() for t in kv]
    heads = slice(0, 3)   # one GQA group on the CPU oracle
    Ow, lw = oracle.sparse_attn_int4(Q.cpu()[:, heads], *[t[:, :1] for t in cpu], selection_mask=mask.cpu()[:, heads], page_size=page)
    _close(base[:, heads], lbase[:, heads], Ow, lw, torch.float16)
    assert att.status() == 0


@pytest.mark.parametrize("S,k_max", [(131072, 1024), (524288, 4096)])
def test_config4_shapes(att, S, k_max):
    """BASELINE config 4's two shapes (retention 0.125, page 16, 24/8 heads): 128k context
    (8192 pages, bucket 1026) and 512k context (32 768 pages, bucket 4098).  Whole chain on the GPU
    for one sequence; scores, page set, compact list and attention of one GQA group against the
    oracle on the same packed bytes."""
    from flashquest_b200.eager.criticality import page_scores_int4_fast
    from flashquest_b200.eager.selection import select_pages_compact
    from flashquest_b200.kernel.kv_quant import quantize_k_int4, quantize_v_int4
    B, Hq, Hkv, D, page = 1, 24, 8, 128, 16
    P, bucket = S // page, k_max + 2
    g = torch.Generator(device="cuda").manual_seed(S % 1000 + 11)
    K = torch.randn(B, Hkv, S, D, device="cuda", generator=g)
    K[..., [3, 17, 64, 100]] *= 8
    K, V = K.half(), torch.randn(B, Hkv, S, D, device="cuda", generator=g).half()
    Q = torch.randn(B, Hq, 1, D, device="cuda", generator=g).half()
    kv = quantize_k_int4(K, page) + quantize_v_int4(V)
    del K, V
    scores = page_scores_int4_fast(Q, kv[1], kv[2])
    comp, mask = select_pages_compact(scores, 0.125, 1, 1, k_max_static=k_max, BUCKET_MAX=bucket, return_mask=True)
    assert comp.shape[-1] == bucket and int(mask.sum(-1).min()) >= k_max and int(mask.sum(-1).max()) <= bucket
    O, lse = att.compact(Q, *kv, selected_page_ids=comp, page_size=page)
    for n_split in (1, 9):
        O2, lse2 = att.compact(Q, *kv, selected_page_ids=comp, page_size=page, n_split=n_split)
        assert (O2.float() - O.float()).abs().max() <= 1e-3 and (lse2 - lse).abs().max() <= 1e-4
    hkv, heads = 5, slice(15, 18)
    cpu = [t[:, hkv:hkv + 1].cpu() for t in kv]
    s_ref = oracle.page_scores_int4_fast(Q.cpu()[:, heads], cpu[1], cpu[2])
    assert torch.equal(scores.cpu()[:, heads], s_ref)
    m_ref = oracle.select_pages_vectorized(s_ref, 0.125, 1, 1, k_max_static=k_max)
    assert torch.equal(mask.cpu()[:, heads], m_ref)
    assert torch.equal(comp.cpu()[:, heads], oracle.build_compact_selection(m_ref, bucket))
    Ow, lw = oracle.sparse_attn_int4(Q.cpu()[:, heads], *cpu, selection_mask=m_ref, page_size=page)
    _close(O[:, heads], lse[:, heads], Ow, lw, torch.float16)
    assert att.status() == 0


def test_many_ctas_with_refills_and_empty_trailing_units(att):
    """A grid larger than the GPU, several pipeline refills per CTA and last iterations whose
    units are partly empty (regression: an empty unit must not let a copy-issuing lane fall two
    barrier phases behind the consumers)."""
    from flashquest_b200.kernel.kv_quant import quantize_k_int4, quantize_v_int4
    B, Hq, Hkv, S, D, page = 16, 24, 8, 4096, 128, 16
    g = torch.Generator(device="cuda").manual_seed(9)
    K = torch.randn(B, Hkv, S, D, device="cuda", generator=g).half()
    V = torch.randn(B, Hkv, S, D, device="cuda", generator=g).half()
    Q = torch.randn(B, Hq, 1, D, device="cuda", generator=g).half()
    kv = quantize_k_int4(K, page) + quantize_v_int4(V)
    cpu = [t[:1, :1].cpu() for t in kv]
    for bucket in (77, 130, 200):
        comp = torch.stack([torch.randperm(S // page, device="cuda", generator=g)[:bucket]
                            for _ in range(B * Hq)]).reshape(B, Hq, 1, bucket).int()
        outs = []
        for n_split in (1, 2, 5):
            for _ in range(3):
                O, lse = att.compact(Q, *kv, selected_page_ids=comp, page_size=page, n_split=n_split)
            torch.cuda.synchronize()
            assert att.status() == 0, (bucket, n_split)
            outs.append((O, lse))
        for O, lse in outs[1:]:
            assert (O.float() - outs[0][0].float()).abs().max() <= 1e-3
            assert (lse - outs[0][1]).abs().max() <= 1e-4
        Ow, lw = oracle.sparse_attn_int4(Q[:1, :3].cpu(), *cpu, selected_page_ids=comp[:1, :3].cpu(), page_size=page)
        _close(outs[0][0][:1, :3], outs[0][1][:1, :3], Ow, lw, torch.float16)


def test_counted_list_walks_only_the_front(att):
    """The mask form builds a list as wide as the page count plus the number of real entries per row; the
    attention call walks only that many.  The count equals the row's selected pages, the result equals the
    tight-list result bit for bit at one split, and a smaller count drops exactly the entries behind it
    (checked against the oracle with those pages removed from the mask)."""
    from flashquest_b200.eager.selection import build_compact_selection
    from flashquest_b200.kernel.sparse_int4_fwd_compact import sparse_decode_int4
    B, Hq, Hkv, S, D, page, dtype = 2, 6, 2, 2048, 128, 16, torch.float16
    Q, kv, mask = _case(41, B, Hq, Hkv, S, D, page, dtype, retention=0.2)
    mask[1, 3] = False                                     # a row with nothing selected
    dev = [t.cuda() for t in kv]
    wide, count = build_compact_selection(mask.cuda(), S // page, return_count=True)
    assert torch.equal(count.cpu().long(), mask.sum(-1))
    assert torch.equal(wide.cpu(), oracle.build_compact_selection(mask, S // page))
    tight = oracle.build_compact_selection(mask, int(mask.sum(-1).max())).cuda()
    O1, l1 = att.compact(Q.cuda(), *dev, selected_page_ids=tight, page_size=page, n_split=1)
    O2, l2 = sparse_decode_int4(Q.cuda(), *dev, wide.squeeze(2), page_size=page, sm_scale=None, return_lse=True,
                                n_split=1, list_count=count)
    assert torch.equal(O1, O2) and torch.equal(l1, l2)
    O3, l3 = att.mask(Q.cuda(), *dev, selection_mask=mask.cuda(), page_size=page)          # default split count
    Ow, lw = oracle.sparse_attn_int4(Q, *kv, selection_mask=mask, page_size=page)
    _close(O3, l3, Ow, lw, dtype)
    # half the count: the list is descending, so the lowest page ids of every row fall away
    half = (count // 2).contiguous()
    m2 = torch.zeros_like(mask)
    ids = wide.cpu().long()
    for b in range(B):
        for h in range(Hq):
            keep = ids[b, h, 0, :int(half[b, h, 0])]
            m2[b, h, 0, keep] = True
    O4, l4 = sparse_decode_int4(Q.cuda(), *dev, wide.squeeze(2), page_size=page, sm_scale=None, return_lse=True,
                                list_count=half)
    Ow2, lw2 = oracle.sparse_attn_int4(Q, *kv, selection_mask=m2, page_size=page)
    _close(O4, l4, Ow2, lw2, dtype)
    assert att.status() == 0
