"""patch_llama_for_quest_persistent on a random-init tiny Hugging Face LlamaModel: prefill, then
teacher-forced decode steps across page boundaries, for the INT4 cache (bool-mask path against
compact path) and the TurboQuant cache, every attention call checked against the oracle chain on the
very q / k / v that went into it (reference test: tests/test_persistent_patch_compact.py:10-66)."""
import math

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _tiny_llama():
    from transformers import AutoConfig
    from transformers.models.llama.modeling_llama import LlamaModel
    cfg = AutoConfig.for_model("llama", hidden_size=256, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2,
                               intermediate_size=256, max_position_embeddings=512, vocab_size=128)
    cfg.head_dim = 64
    torch.manual_seed(42)
    return cfg, LlamaModel(cfg).cuda().to(torch.bfloat16).eval()


def _dense_causal(q, K, V):
    """fp32 reference of the prefill branch: query i sees keys 0..i, grouped-query heads."""
    B, Hq, Sq, D = q.shape
    n_rep = Hq // K.shape[1]
    Kf, Vf = K.float().repeat_interleave(n_rep, 1), V.float().repeat_interleave(n_rep, 1)
    s = q.float() @ Kf.transpose(-1, -2) / math.sqrt(D)
    i, j = torch.arange(Sq)[:, None], torch.arange(K.shape[2])[None, :]
    s = s.masked_fill(j > i, float("-inf"))
    return torch.softmax(s, -1) @ Vf


class _OracleCheck:
    """Replays every traced attention call on the CPU oracle."""

    def __init__(self, kv_bits, page, n_layers, H_q, retention_rows, sinks, window, k_max_static, fused_tail):
        self.bits, self.page, self.sinks, self.window, self.kms, self.fused = kv_bits, page, sinks, window, k_max_static, fused_tail
        self.K, self.V = [None] * n_layers, [None] * n_layers
        self.ret = retention_rows                       # per layer: (H_q,) fp32 retention per query head
        self.worst = {"prefill": 0.0, "decode": 0.0}
        self.calls = 0

    def __call__(self, li, q, k, v, attn):
        q, k, v, attn = q.cpu(), k.cpu(), v.cpu(), attn.float().cpu()
        self.K[li] = k if self.K[li] is None else torch.cat([self.K[li], k], 2)
        self.V[li] = v if self.V[li] is None else torch.cat([self.V[li], v], 2)
        K, V, page = self.K[li], self.V[li], self.page
        S = K.shape[2]
        nq = S - S % page
        self.calls += 1
        if q.shape[2] > 1:
            if self.bits == 4:
                kq, vq = oracle.quantize_k_int4(K[:, :, :nq], page), oracle.quantize_v_int4(V[:, :, :nq])
                Kd, Vd = oracle.dequantize_k_int4(*kq, page), oracle.dequantize_v_int4(*vq)
            elif self.bits == 8:
                kq, vq = oracle.quantize_k(K[:, :, :nq], page), oracle.quantize_v(V[:, :, :nq])
                Kd, Vd = oracle.dequantize_k(*kq, page), oracle.dequantize_v(*vq)
            else:
                kq, vq = oracle.quantize_k_turbo(K[:, :, :nq], page), oracle.quantize_v_turbo(V[:, :, :nq])
                Kd = oracle.dequantize_k_turbo(kq[0], kq[1], kq[2], head_dim=K.shape[-1])
                Vd = oracle.dequantize_v_turbo(vq[0], vq[1], vq[2], head_dim=K.shape[-1])
            want = _dense_causal(q, torch.cat([Kd.to(K.dtype), K[:, :, nq:]], 2), torch.cat([Vd.to(V.dtype), V[:, :, nq:]], 2))
            err = (attn - want).abs().max().item()
            self.worst["prefill"] = max(self.worst["prefill"], err)
            assert err <= 8e-3, ("prefill", li, err)          # bf16 probabilities and output: two bf16 ulps at |O| ~ 1
            return
        Kt, Vt = K[:, :, nq:], V[:, :, nq:]
        r = self.ret[li]
        if self.bits in (4, 8):
            qk, qv, sc, at = ((oracle.quantize_k_int4, oracle.quantize_v_int4, oracle.page_scores_int4_fast, oracle.sparse_attn_int4)
                              if self.bits == 4 else
                              (oracle.quantize_k, oracle.quantize_v, oracle.page_scores_int8_fast, oracle.sparse_attn_int8))
            kv = qk(K[:, :, :nq], page) + qv(V[:, :, :nq])
            if nq:
                mask = oracle.select_pages_vectorized(sc(q, kv[1], kv[2]), r, self.sinks, self.window, k_max_static=self.kms)
            else:
                mask = torch.zeros(q.shape[0], q.shape[1], 1, 0, dtype=torch.bool)
            want, _ = at(q, *kv, selection_mask=mask, page_size=page, K_partial=Kt, V_partial=Vt)
            tol = 2e-3 + 2 ** -8 * want.abs() * (1 if self.fused else 3)   # separate bf16 partials + merge: two more roundings
        else:
            kq, vq = oracle.quantize_k_turbo(K[:, :, :nq], page), oracle.quantize_v_turbo(V[:, :, :nq])
            parts_O, parts_l = [], []
            if nq:
                mask = oracle.select_pages_vectorized(oracle.page_scores_int4_fast(q, kq[3], kq[4]), r, self.sinks, self.window,
                                                      k_max_static=self.kms)
                O1, l1 = oracle.sparse_attn_turbo(q, kq[0], kq[1], kq[2], vq[0], vq[1], vq[2], selection_mask=mask, page_size=page)
                parts_O.append(O1); parts_l.append(l1)
            if S > nq or not nq:
                e8 = torch.empty(q.shape[0], K.shape[1], 0, K.shape[-1] // 2, dtype=torch.uint8)
                em = torch.empty(q.shape[0], K.shape[1], 0, K.shape[-1], dtype=torch.bfloat16)
                ev = torch.empty(q.shape[0], K.shape[1], 0, 1, dtype=torch.bfloat16)
                O2, l2 = oracle.sparse_attn_int4(q, e8, em, em, e8, ev, ev, selected_page_ids=torch.full((q.shape[0], q.shape[1], 1, 1), -1, dtype=torch.int32),
                                                 page_size=page, K_partial=Kt, V_partial=Vt)
                parts_O.append(O2); parts_l.append(l2)
            want, _ = oracle.lse_merge(torch.stack(parts_O), torch.stack(parts_l))
            tol = 2e-2 + 0 * want                   # q and O pass through bf16 rotations (the reference's own test bound is 5e-2)
        err = (attn - want).abs()
        self.worst["decode"] = max(self.worst["decode"], float((err / tol).max()))
        assert (err <= tol).all(), ("decode", li, S, float(err.max()))


def _run(model, cache, ids_prompt, ids_steps):
    outs = []
    with torch.no_grad():
        outs.append(model(ids_prompt, past_key_values=cache).last_hidden_state)
        for t in range(ids_steps.shape[1]):
            outs.append(model(ids_steps[:, t:t + 1], past_key_values=cache).last_hidden_state)
    return torch.cat(outs, 1)


@pytest.mark.parametrize("kv_bits,page", [(4, 8), (4, 16), (3, 16), (8, 16)])
def test_patched_forward_paths_and_oracle(kv_bits, page):
    from flashquest_b200.cache.persistent_int4 import PersistentInt4KVCache
    from flashquest_b200.cache.persistent_int8 import PersistentInt8KVCache
    from flashquest_b200.cache.persistent_turbo import PersistentTurboKVCache
    from flashquest_b200.eager import llama_persistent_patch as lpp
    from transformers.cache_utils import Cache
    cfg, model_a = _tiny_llama()
    Cls = {4: PersistentInt4KVCache, 8: PersistentInt8KVCache, 3: PersistentTurboKVCache}[kv_bits]
    mk = lambda: Cls(num_layers=2, batch_size=1, num_kv_heads=2, head_dim=64, page_size=page, max_seq_len=128)
    cache_a = mk()
    assert isinstance(cache_a, Cache) and cache_a.kv_bits == kv_bits
    head_pattern = torch.tensor([[True, True], [True, False]])          # one streaming KV head in layer 1
    retention, sinks, window = 0.5, 2, 1
    kw = dict(head_pattern=head_pattern, retention=retention, num_sinks=sinks, window_pages=window, page_size=page)
    torch.manual_seed(0)
    prompt = torch.randint(0, 128, (1, 37), device="cuda")
    steps = torch.randint(0, 128, (1, 30), device="cuda")            # crosses page boundaries at either page size
    k_max_static = math.ceil(retention * (128 // page))
    rows = [torch.where(head_pattern[l].repeat_interleave(2), torch.tensor(retention), torch.tensor(0.0)).float() for l in range(2)]

    lpp.patch_llama_for_quest_persistent(model_a, cache=cache_a, use_compact_kernel=False, **kw)
    chk_a = _OracleCheck(kv_bits, page, 2, 4, rows, sinks, window, k_max_static, fused_tail=False)
    lpp.TRACE = chk_a
    try:
        out_a = _run(model_a, cache_a, prompt, steps)
    finally:
        lpp.TRACE = None
    assert chk_a.calls == 2 * 31 and cache_a.get_seq_length() == 67
    print(f"kv_bits={kv_bits} page={page} worst prefill error {chk_a.worst['prefill']:.2e}, decode {chk_a.worst['decode']:.2f} of the bound")
    if kv_bits != 4:
        with pytest.raises(NotImplementedError, match="kv_bits=4"):
            lpp.make_quest_persistent_forward(cache=cache_a, head_pattern_layer=head_pattern[0], retention=0.5, num_sinks=2,
                                              window_pages=1, page_size=page, use_compact_kernel=True)
        return
    # path B: compact kernel, same weights (reference test: both paths agree within 5e-2)
    _, model_b = _tiny_llama()
    model_b.load_state_dict(model_a.state_dict())
    cache_b = mk()
    lpp.patch_llama_for_quest_persistent(model_b, cache=cache_b, use_compact_kernel=True, **kw)
    chk_b = _OracleCheck(kv_bits, page, 2, 4, rows, sinks, window, k_max_static, fused_tail=True)
    lpp.TRACE = chk_b
    try:
        out_b = _run(model_b, cache_b, prompt, steps)
    finally:
        lpp.TRACE = None
    # The reference's own test compares the two paths after a prefill only, at 5e-2.  Here 30 free-running
    # decode steps follow: a last-bit difference in one layer's output can move a 4-bit code of the next
    # layer's k / v by one step, so a few elements drift further; both paths are held to the oracle call by
    # call above, here the prefill must agree at the reference's bound and the decode steps in bulk.
    torch.testing.assert_close(out_b[:, :37], out_a[:, :37], atol=5e-2, rtol=5e-2)
    diff = (out_b.float() - out_a.float()).abs()
    assert (diff > 5e-2 + 5e-2 * out_a.float().abs()).float().mean().item() < 0.02 and diff.max().item() < 1.0, diff.max().item()
    for name in ("K_packed", "V_packed", "K_scale", "K_mn", "V_scale", "V_mn"):
        va, vb = cache_a.get_views(1)[name], cache_b.get_views(1)[name]
        assert va.shape == vb.shape


def test_patch_argument_errors():
    from flashquest_b200.cache.persistent_int4 import PersistentInt4KVCache
    from flashquest_b200.eager import llama_persistent_patch as lpp
    cfg, model = _tiny_llama()
    cache = PersistentInt4KVCache(num_layers=2, batch_size=1, num_kv_heads=2, head_dim=64, page_size=16, max_seq_len=64)
    with pytest.raises(ValueError, match="2D"):
        lpp.patch_llama_for_quest_persistent(model, cache=cache, head_pattern=torch.ones(2, dtype=torch.bool))
    with pytest.raises(ValueError, match="head_pattern has 1 layers"):
        lpp.patch_llama_for_quest_persistent(model, cache=cache, head_pattern=torch.ones(1, 2, dtype=torch.bool), page_size=16)
    with pytest.raises(RuntimeError, match="no LlamaAttention"):
        lpp.patch_llama_for_quest_persistent(torch.nn.Linear(2, 2), cache=cache, head_pattern=torch.ones(2, 2, dtype=torch.bool))

    class Fake:
        kv_bits, head_dim, max_seq_len, page_size = 8, 64, 64, 16
    with pytest.raises(NotImplementedError, match="kv_bits=4"):
        lpp.make_quest_persistent_forward(cache=Fake(), head_pattern_layer=torch.ones(2, dtype=torch.bool), retention=0.5,
                                          num_sinks=2, window_pages=1, page_size=16, use_compact_kernel=True)
