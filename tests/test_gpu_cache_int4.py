"""PersistentInt4KVCache: prefill / decode / page-completing appends equal a fresh quantise
of the same tokens (reference tests/test_persistent_int4.py:19-75, test_persistent_cache.py)."""
import pytest
import torch

import oracle
from tests._util import bit_equal, make_kv, make_q

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def Cache():
    from flashquest_b200.cache.persistent_int4 import PersistentInt4KVCache
    return PersistentInt4KVCache


def _check_against_oracle(cache, K, V, layer, page):
    v = cache.get_views(layer)
    seen = v["seq_len"]
    n = v["completed_len"]
    assert v["partial_len"] == seen - n and n % page == 0
    if n:
        Kp, Ks, Km = oracle.quantize_k_int4(K[:, :, :n], page)
        Vp, Vs, Vm = oracle.quantize_v_int4(V[:, :, :n])
        for key, want in (("K_packed", Kp), ("K_scale", Ks), ("K_mn", Km), ("V_packed", Vp), ("V_scale", Vs), ("V_mn", Vm)):
            assert bit_equal(v[key].cpu(), want), key
    else:
        assert v["K_packed"].shape[2] == 0 and v["K_scale"].shape[2] == 0
    assert bit_equal(v["K_partial"].cpu(), K[:, :, n:seen].contiguous())
    assert bit_equal(v["V_partial"].cpu(), V[:, :, n:seen].contiguous())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("page", [8, 16, 64])
def test_append_patterns_equal_fresh_quantize(Cache, dtype, page):
    B, H, D, S_max = 2, 2, 128, 400
    cache = Cache(batch_size=B, num_layers=2, num_kv_heads=H, head_dim=D, max_seq_len=S_max, page_size=page,
                  device="cuda", dtype=dtype)
    assert cache.kv_bits == 4 and cache.get_max_length() == S_max
    assert cache.K_packed.shape == (2, B, H, S_max, D // 2) and cache.K_packed.dtype == torch.uint8
    assert cache.K_scale.shape == (2, B, H, (S_max + page - 1) // page, D) and cache.K_scale.dtype == torch.bfloat16
    assert cache.V_scale.shape == (2, B, H, S_max, 1) and cache.K_partial.shape == (2, B, H, page, D)
    K = make_kv(41, (B, H, S_max, D), dtype)
    V = make_kv(42, (B, H, S_max, D), dtype, outliers=())
    # prefill that ends inside a page, then single-token decode appends across several page
    # boundaries, then chunks that complete pages in the middle of the chunk
    pos = 0
    for chunk in [3 * page + 5] + [1] * (2 * page + 3) + [page - 1, 2 * page, 1, page + 7, 2]:
        if pos + chunk > S_max:
            break
        cache.update_quantized(K[:, :, pos:pos + chunk].cuda(), V[:, :, pos:pos + chunk].cuda(), 1)
        pos += chunk
        assert cache.get_seq_length(1) == pos and cache.get_seq_length(0) == 0
        _check_against_oracle(cache, K, V, 1, page)
    # layer 0 untouched
    assert (cache.K_packed[0] == 0).all() and (cache.K_partial[0] == 0).all()
    # reset by assignment (how the reference's runtime reuses a cache) and refill
    cache._seen_tokens = [0] * 2
    cache.update_quantized(K[:, :, :page].cuda(), V[:, :, :page].cuda(), 0)
    _check_against_oracle(cache, K, V, 0, page)


def test_partial_only_views_overflow_and_bad_layer(Cache):
    cache = Cache(batch_size=1, num_layers=1, num_kv_heads=2, head_dim=64, max_seq_len=32, page_size=16, device="cuda")
    K = make_kv(1, (1, 2, 40, 64), torch.bfloat16)
    cache.update_quantized(K[:, :, :5].cuda(), K[:, :, :5].cuda(), 0)
    v = cache.get_views(0)
    assert v["completed_len"] == 0 and v["partial_len"] == 5 and v["K_packed"].shape[2] == 0
    assert bit_equal(v["K_partial"].cpu(), K[:, :, :5].contiguous())
    with pytest.raises(RuntimeError, match="exceeds.*max_seq_len"):
        cache.update_quantized(K[:, :, :28].cuda(), K[:, :, :28].cuda(), 0)
    with pytest.raises(IndexError, match="layer_idx"):
        cache.update_quantized(K[:, :, :1].cuda(), K[:, :, :1].cuda(), 1)
    with pytest.raises(IndexError, match="layer_idx"):
        cache.get_views(-1)
    with pytest.raises(NotImplementedError):
        cache.update()
    with pytest.raises(ValueError, match="even head_dim"):
        Cache(batch_size=1, num_layers=1, num_kv_heads=1, head_dim=65, max_seq_len=32, page_size=16, device="cuda")
    # fp32 input is cast to the cache dtype like the reference's patched forward does
    cache.update_quantized(K[:, :, 5:27].float().cuda(), K[:, :, 5:27].float().cuda(), 0)
    _check_against_oracle(cache, K, K, 0, 16)


def test_decode_step_dispatcher_matches_oracle(Cache):
    """QuestDecodeInt4.attend == oracle chain, while the cache grows token by token."""
    from flashquest_b200.eager.decode_step import QuestDecodeInt4
    B, Hq, Hkv, D, page, S0 = 2, 6, 2, 128, 16, 300
    cache = Cache(batch_size=B, num_layers=2, num_kv_heads=Hkv, head_dim=D, max_seq_len=512, page_size=page,
                  device="cuda", dtype=torch.float16)
    K = make_kv(51, (B, Hkv, 512, D), torch.float16)
    V = make_kv(52, (B, Hkv, 512, D), torch.float16, outliers=())
    pattern = torch.tensor([True, False])      # second KV head is a streaming head
    step = QuestDecodeInt4(cache, num_q_heads=Hq, retention=0.25, num_sinks=2, window_pages=1,
                           head_pattern_layer=pattern, q_dtype=torch.float16)
    cache.update_quantized(K[:, :, :S0].cuda(), V[:, :, :S0].cuda(), 1)
    for t in range(S0, S0 + 2 * page + 2):
        Q = torch.randn(B, Hq, 1, D, generator=torch.Generator().manual_seed(t)).half()
        if t % 2 == 0:      # two equivalent routes: separate calls, or the one-call layer step
            cache.update_quantized(K[:, :, t:t + 1].cuda(), V[:, :, t:t + 1].cuda(), 1)
            O, lse = step.attend(Q.cuda(), 1)
        else:
            O, lse = step.step(K[:, :, t:t + 1].cuda(), V[:, :, t:t + 1].cuda(), Q.cuda(), 1)
        assert cache.get_seq_length(1) == t + 1
        seen = t + 1
        n = seen - seen % page
        kv = oracle.quantize_k_int4(K[:, :, :n], page) + oracle.quantize_v_int4(V[:, :, :n])
        s = oracle.page_scores_int4_fast(Q, kv[1], kv[2])
        r = torch.tensor([0.25] * 3 + [0.0] * 3)
        m = oracle.select_pages_vectorized(s, r, 2, 1, k_max_static=step.k_max_static)
        Ow, lw = oracle.sparse_attn_int4(Q, *kv, selection_mask=m, page_size=page,
                                         K_partial=K[:, :, n:seen], V_partial=V[:, :, n:seen])
        assert (O.float().cpu() - Ow).abs().max() < 2e-3, t
        assert (lse.cpu() - lw).abs().max() < 1e-3, t
    # empty cache: tail-only attention
    Q = torch.randn(B, Hq, 1, D, generator=torch.Generator().manual_seed(1)).half()
    O, lse = step.step(K[:, :, :3].cuda(), V[:, :, :3].cuda(), Q.cuda(), 0)
    Ow, lw = oracle.sparse_attn_int4(Q, *kv, selected_page_ids=torch.full((B, Hq, 1, 1), -1, dtype=torch.int32),
                                     page_size=page, K_partial=K[:, :, :3], V_partial=V[:, :, :3])
    assert (O.float().cpu() - Ow).abs().max() < 2e-3 and (lse.cpu() - lw).abs().max() < 1e-3
    with pytest.raises(IndexError, match="layer_idx"):
        step.step(K[:, :, :1].cuda(), V[:, :, :1].cuda(), Q.cuda(), 5)
    with pytest.raises(RuntimeError, match="exceeds.*max_seq_len"):
        step.step(K[:, :, :512].cuda(), V[:, :, :512].cuda(), Q.cuda(), 0)


def test_step_all_equals_per_layer_steps():
    """fq_decode_step_int4 (all layers in one call) == fq_decode_layer_int4 layer by layer, bit for bit,
    with layers at different lengths (one of them crossing a page boundary)."""
    from flashquest_b200.cache.persistent_int4 import PersistentInt4KVCache
    from flashquest_b200.eager.decode_step import QuestDecodeInt4
    B, Hq, Hkv, D, page, Ln = 1, 6, 2, 128, 16, 3
    outs = []
    for mode in ("all", "each"):
        cache = PersistentInt4KVCache(batch_size=B, num_layers=Ln, num_kv_heads=Hkv, head_dim=D, max_seq_len=256,
                                      page_size=page, device="cuda", dtype=torch.float16)
        step = QuestDecodeInt4(cache, num_q_heads=Hq, retention=0.5, num_sinks=1, window_pages=1, q_dtype=torch.float16)
        for li, s0 in enumerate((95, 64, 130)):
            cache.update_quantized(make_kv(60 + li, (B, Hkv, s0, D), torch.float16).cuda(),
                                   make_kv(70 + li, (B, Hkv, s0, D), torch.float16, outliers=()).cuda(), li)
        res = []
        for t in range(3):
            k = make_kv(80 + t, (Ln, B, Hkv, 1, D), torch.float16).cuda()
            v = make_kv(90 + t, (Ln, B, Hkv, 1, D), torch.float16, outliers=()).cuda()
            q = make_q(100 + t, (Ln, B, Hq, 1, D), torch.float16).cuda()
            if mode == "all":
                O, lse = step.step_all(k, v, q)
                res.append((O.clone(), lse.clone()))
            else:
                Os, ls = zip(*[tuple(x.clone() for x in step.step(k[li], v[li], q[li], li)) for li in range(Ln)])
                res.append((torch.stack(Os), torch.stack(ls)))
        assert [cache.get_seq_length(li) for li in range(Ln)] == [98, 67, 133]
        outs.append(res)
    for (Oa, la), (Oe, le) in zip(*outs):
        assert torch.equal(Oa, Oe) and torch.equal(la, le)


@pytest.mark.parametrize("start,n_new", [((0, 0), 1), ((95, 300), 1), ((7, 130), 5)])
def test_graph_replayed_steps_equal_stream_steps(start, n_new):
    """fq_decode_step_int4_dev (sequence length read on the device, one captured graph replayed
    for every token) == fq_decode_step_int4 bit for bit, from an empty cache and across page boundaries."""
    from flashquest_b200.cache.persistent_int4 import PersistentInt4KVCache
    from flashquest_b200.eager.decode_step import QuestDecodeInt4
    B, Hq, Hkv, D, page, Ln, steps = 2, 6, 2, 128, 16, 2, 40 if n_new == 1 else 12
    outs = []
    for mode in ("graph", "stream"):
        cache = PersistentInt4KVCache(batch_size=B, num_layers=Ln, num_kv_heads=Hkv, head_dim=D, max_seq_len=512,
                                      page_size=page, device="cuda", dtype=torch.float16)
        step = QuestDecodeInt4(cache, num_q_heads=Hq, retention=0.5, num_sinks=1, window_pages=1, q_dtype=torch.float16)
        for li, s0 in enumerate(start):
            if s0:
                cache.update_quantized(make_kv(60 + li, (B, Hkv, s0, D), torch.float16).cuda(),
                                       make_kv(70 + li, (B, Hkv, s0, D), torch.float16, outliers=()).cuda(), li)
        kb = torch.empty(Ln, B, Hkv, n_new, D, dtype=torch.float16, device="cuda")
        vb, qb = torch.empty_like(kb), torch.empty(Ln, B, Hq, 1, D, dtype=torch.float16, device="cuda")
        replay = step.capture_step_graph(kb, vb, qb) if mode == "graph" else None
        res = []
        for t in range(steps):
            kb.copy_(make_kv(800 + t, (Ln, B, Hkv, n_new, D), torch.float16))
            vb.copy_(make_kv(900 + t, (Ln, B, Hkv, n_new, D), torch.float16, outliers=()))
            qb.copy_(make_q(1000 + t, (Ln, B, Hq, 1, D), torch.float16))
            O, lse = replay() if mode == "graph" else step.step_all(kb, vb, qb)
            res.append((O.clone(), lse.clone()))
        assert [cache.get_seq_length(li) for li in range(Ln)] == [s + steps * n_new for s in start]
        outs.append((res, [t.clone() for t in (cache.K_packed, cache.V_packed, cache.K_scale, cache.K_mn, cache.V_scale, cache.V_mn)]))
    (ra, ca), (rb, cb) = outs
    for t, ((Oa, la), (Ob, lb)) in enumerate(zip(ra, rb)):
        assert torch.equal(Oa, Ob) and torch.equal(la, lb), t
    n_tok = [s + steps * n_new for s in start]
    for li in range(Ln):                     # cache contents of the filled part
        nq = n_tok[li] - n_tok[li] % page
        assert torch.equal(ca[0][li][:, :, :nq], cb[0][li][:, :, :nq]) and torch.equal(ca[1][li][:, :, :nq], cb[1][li][:, :, :nq])
        assert bit_equal(ca[2][li][:, :, : nq // page], cb[2][li][:, :, : nq // page])
        assert bit_equal(ca[4][li][:, :, :nq], cb[4][li][:, :, :nq])
