"""The Llama-shaped decode step (norms, rotary embedding, AWQ projections, sparse INT4 attention,
SwiGLU, lm_head, argmax) against a CPU restatement with Hugging Face's fp16 roundings, built
from the oracle's AWQ GEMV and attention chain, token by token from an empty cache."""
import math

import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def _rms(x, w, eps):
    xf = x.float()
    xh = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).half()
    return w * xh


def _awq(x, lin):
    return oracle.awq_gemv(x, lin.qweight.cpu(), lin.scales.cpu(), lin.qzeros.cpu(), group_size=lin.group_size).half()


def _rope(x, pos, theta):
    # x (B, H, D) fp16; Hugging Face rotate_half convention with fp16 cos / sin
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2).float() / D))
    ang = pos * inv
    cos = torch.cat([ang, ang]).cos().half()
    sin = torch.cat([ang, ang]).sin().half()
    rot = torch.cat([-x[..., D // 2:], x[..., : D // 2]], dim=-1)
    return x * cos + rot * sin


class _Ref:
    def __init__(self, cfg, w, page, retention, sinks, window, k_max_static):
        self.cfg, self.w, self.page = cfg, w, page
        self.sel = (retention, sinks, window, k_max_static)
        self.K = [None] * cfg.layers
        self.V = [None] * cfg.layers

    def step(self, ids, trace=None, views_fn=None, kv_err=None):
        """views_fn(layer) -> the GPU cache's views AFTER the GPU ran the same step: the attention then
        reads the GPU's packed bytes and staged tokens (teacher-forced cache), so that a last-bit
        difference in k or v cannot move a 4-bit code and with it every later result; the k / v this
        restatement computes itself are compared with the GPU's staged ones into kv_err instead."""
        c, w = self.cfg, self.w
        B = ids.shape[0]
        pos = 0 if self.K[0] is None else self.K[0].shape[2]
        x = w.embed.cpu()[ids.long()]
        delta = None
        for li, lw in enumerate(w.layers):
            if delta is not None:
                x = x + delta
                if trace is not None:
                    trace.append(x)
            n = _rms(x, lw.input_norm.cpu(), c.rms_eps)
            q = _awq(n, lw.q_proj).view(B, c.q_heads, c.head_dim)
            k = _awq(n, lw.k_proj).view(B, c.kv_heads, c.head_dim)
            v = _awq(n, lw.v_proj).view(B, c.kv_heads, c.head_dim)
            q, k = _rope(q, pos, c.rope_theta), _rope(k, pos, c.rope_theta)
            self.K[li] = k.unsqueeze(2) if self.K[li] is None else torch.cat([self.K[li], k.unsqueeze(2)], 2)
            self.V[li] = v.unsqueeze(2) if self.V[li] is None else torch.cat([self.V[li], v.unsqueeze(2)], 2)
            seen = self.K[li].shape[2]
            nq = seen - seen % self.page
            K_tail, V_tail = self.K[li][:, :, nq:], self.V[li][:, :, nq:]
            if views_fn is None:
                Kc, Vc = self.K[li][:, :, :nq], self.V[li][:, :, :nq]
                kv = oracle.quantize_k_int4(Kc, self.page) + oracle.quantize_v_int4(Vc)
            else:
                vw = views_fn(li)
                assert vw["seq_len"] == seen and vw["completed_len"] == nq
                kv = tuple(vw[n].cpu() for n in ("K_packed", "K_scale", "K_mn", "V_packed", "V_scale", "V_mn"))
                gk, gv = vw["K_partial"].cpu(), vw["V_partial"].cpu()
                if seen > nq and kv_err is not None:      # the newest token is still staged unquantised: compare it
                    for mine, theirs in ((k, gk[:, :, -1]), (v, gv[:, :, -1])):
                        kv_err.append(float((mine.float() - theirs.float()).abs().max() / (2e-3 * mine.float().abs().max() + 1e-3)))
                K_tail, V_tail = gk, gv
            r, s, wn, kms = self.sel
            if nq > 0:
                sc = oracle.page_scores_int4_fast(q.unsqueeze(2), kv[1], kv[2])
                mask = oracle.select_pages_vectorized(sc, r, s, wn, k_max_static=kms)
            else:
                mask = torch.zeros(B, c.q_heads, 1, 0, dtype=torch.bool)
            O, _ = oracle.sparse_attn_int4(q.unsqueeze(2), *kv, selection_mask=mask, page_size=self.page,
                                           K_partial=K_tail, V_partial=V_tail)
            attn = _awq(O.half().reshape(B, -1), lw.o_proj)
            x = x + attn
            if trace is not None:
                trace.append(x)
            n = _rms(x, lw.post_norm.cpu(), c.rms_eps)
            gate, up = _awq(n, lw.gate_proj), _awq(n, lw.up_proj)
            act = torch.nn.functional.silu(gate.float()).half() * up
            delta = _awq(act, lw.down_proj)
        x = x + delta
        if trace is not None:
            trace.append(x)
        n = _rms(x, w.final_norm.cpu(), c.rms_eps)
        return (n.float() @ w.lm_head.cpu().float().T).half()


def test_small_ops_match_torch():
    from flashquest_b200._lib import check, lib, ptr, stream_ptr
    L = lib()
    g = torch.Generator().manual_seed(3)
    dev = torch.device("cuda")
    st = lambda: stream_ptr(dev)
    # add + RMSNorm
    a, b = torch.randn(3, 3072, generator=g).half(), torch.randn(3, 3072, generator=g).half()
    wt = (1 + 0.1 * torch.randn(3072, generator=g)).half()
    s_out, y = torch.empty(3, 3072, dtype=torch.float16, device=dev), torch.empty(3, 3072, dtype=torch.float16, device=dev)
    ad, bd, wd = a.cuda(), b.cuda(), wt.cuda()             # keep the device copies alive across the launch
    check(L.fq_add_rmsnorm(ptr(ad), ptr(bd), ptr(wd), 1e-5, 3, 3072, ptr(s_out), ptr(y), st()))
    h = a + b
    assert torch.equal(s_out.cpu(), h)
    assert (y.cpu().float() - _rms(h, wt, 1e-5).float()).abs().max() <= 2e-3      # one fp16 ulp at |y| ~ 4
    # RoPE
    q, k = torch.randn(2, 6, 128, generator=g).half(), torch.randn(2, 2, 128, generator=g).half()
    qd, kd = q.cuda(), k.cuda()
    check(L.fq_rope(ptr(qd), qd.stride(0), qd.stride(1), 6, ptr(kd), kd.stride(0), kd.stride(1), 2, 2, 128, 32767, 500000.0, st()))
    assert (qd.cpu().float() - _rope(q, 32767, 500000.0).float()).abs().max() <= 6e-3   # sin/cos of a large angle in fp32
    assert (kd.cpu().float() - _rope(k, 32767, 500000.0).float()).abs().max() <= 6e-3
    # SwiGLU
    gt, up = torch.randn(2, 8192, generator=g).half() * 3, torch.randn(2, 8192, generator=g).half()
    out = torch.empty(2, 8192, dtype=torch.float16, device=dev)
    gd, ud = gt.cuda(), up.cuda()
    check(L.fq_swiglu(ptr(gd), ptr(ud), gt.numel(), ptr(out), st()))
    want = torch.nn.functional.silu(gt.float()).half() * up
    assert (out.cpu().float() - want.float()).abs().max() <= 4e-3
    # fp16 GEMV + argmax
    x, W = torch.randn(3, 512, generator=g).half(), (torch.randn(1000, 512, generator=g) * 0.05).half()
    yv = torch.empty(3, 1000, dtype=torch.float16, device=dev)
    xd, Wd = x.cuda(), W.cuda()
    check(L.fq_gemv_f16(ptr(xd), ptr(Wd), 3, 512, 1000, ptr(yv), st()))
    ref = (x.float() @ W.float().T)
    assert (yv.cpu().float() - ref).abs().max() <= 2e-3 * ref.abs().max() + 1e-3
    # one row on the CUDA cores, 2..8 rows on the tensor cores, ragged N, a K the tensor-core path does not take
    for Mr, Kr, Nr in ((1, 512, 1000), (2, 1024, 130), (8, 3072, 2056), (5, 520, 64), (8, 256, 7)):
        xr, Wr = torch.randn(Mr, Kr, generator=g).half(), (torch.randn(Nr, Kr, generator=g) * 0.05).half()
        yr = torch.full((Mr, Nr), float("nan"), dtype=torch.float16, device=dev)
        xrd, Wrd = xr.cuda(), Wr.cuda()
        check(L.fq_gemv_f16(ptr(xrd), ptr(Wrd), Mr, Kr, Nr, ptr(yr), st()))
        rr = xr.float() @ Wr.float().T
        assert (yr.cpu().float() - rr).abs().max() <= 2e-3 * rr.abs().max() + 1e-3, (Mr, Kr, Nr)
    idx = torch.empty(3, dtype=torch.int32, device=dev)
    yv[1, 7] = yv[1].max() ; yv[1, 500] = yv[1, 7]               # a tie: the first index wins
    check(L.fq_argmax_f16(ptr(yv), 3, 1000, ptr(idx), st()))
    assert idx.cpu().tolist() == yv.float().argmax(-1).cpu().tolist()
    assert idx[1].item() == int((yv[1] == yv[1].max()).nonzero()[0])


def test_decode_steps_match_cpu_restatement():
    from flashquest_b200.eager.llama_decode import LlamaConfig, LlamaInt4Decoder, random_llama_weights
    cfg = LlamaConfig(hidden=256, layers=2, q_heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=512)
    w = random_llama_weights(cfg, "cuda", seed=1)
    page, B = 16, 2
    dec = LlamaInt4Decoder(cfg, w, batch_size=B, max_seq_len=64, page_size=page, retention=0.5, num_sinks=1, window_pages=1)
    ref = _Ref(cfg, w, page, 0.5, 1, 1, dec.attn.k_max_static)
    ids = torch.tensor([5, 300], dtype=torch.int32)
    worst = 0.0
    for t in range(36):                                   # crosses two page boundaries
        nxt = dec.decode_step(ids.cuda()) if t % 3 else dec.decode_step_per_op(ids.cuda())   # one-call step and per-operator route
        got = dec.logits.float().cpu()
        want = ref.step(ids).float()
        tol = 3e-2 * want.abs().max().item() + 1e-2
        err = (got - want).abs().max().item()
        worst = max(worst, err / tol)
        assert err <= tol, (t, err, tol)
        top2 = want.topk(2, dim=-1).values
        for b in range(B):
            if (top2[b, 0] - top2[b, 1]).item() > 2 * tol:
                assert nxt[b].item() == int(want[b].argmax())
        ids = want.argmax(-1).to(torch.int32)             # both sides continue from the reference's choice
    assert dec.cache.get_seq_length(0) == 36


@pytest.mark.parametrize("layers", [1, 2])
def test_decode_steps_at_config3_widths(layers):
    """One and two layers at BASELINE config 3's widths (hidden 3072, 24/8 heads x 128, FFN 8192,
    vocab 128 256), teacher-forced token ids AND cache contents, from an empty cache across a page
    boundary: the residual stream after every block and the logits against the CPU restatement.

    Bound: 2e-3 * max|reference| + one fp16 ulp of the value.  The restatement attends over the GPU
    cache's own bytes (a 4-bit code is a discontinuous function of k: one fp16 ulp in k can move a
    code by one step, which is 1/15 of the page's range; with free-running caches the logits drift
    to 6e-3 * max within one page) and its own k / v are compared with the staged ones at the same
    bound.  Every page is kept (retention 1) so that a last-bit difference in q cannot change the
    page set, which is checked exactly elsewhere."""
    from flashquest_b200.eager.llama_decode import LlamaConfig, LlamaInt4Decoder, random_llama_weights
    cfg = LlamaConfig(layers=layers)
    w = random_llama_weights(cfg, "cuda", seed=4, scale_down=0.25)
    page, B = 16, 1
    dec = LlamaInt4Decoder(cfg, w, batch_size=B, max_seq_len=64, page_size=page, retention=1.0, num_sinks=1, window_pages=1)
    ref = _Ref(cfg, w, page, 1.0, 1, 1, dec.attn.k_max_static)
    ids = torch.tensor([4711], dtype=torch.int32)
    worst_h = worst_l = 0.0
    kv_err = []
    for t in range(19):
        tr_g, tr_r = [], []
        if t % 2:
            dec.decode_step(ids.cuda())
        else:
            dec.decode_step_per_op(ids.cuda(), trace=tr_g)
        got = dec.logits.float().cpu()
        want = ref.step(ids, trace=tr_r, views_fn=dec.cache.get_views, kv_err=kv_err).float()
        for hg, hr in zip(tr_g, tr_r):
            hr = hr.float()
            tol = 2e-3 * hr.abs().max() + 2 ** -11 * hr.abs()
            err = (hg.float().cpu() - hr).abs()
            worst_h = max(worst_h, float((err / tol).max()))
            assert (err <= tol).all(), (t, float(err.max()), float(hr.abs().max()))
        assert len(tr_g) == (len(tr_r) if tr_g else 0)
        tol = 2e-3 * want.abs().max() + 2 ** -11 * want.abs()
        err = (got - want).abs()
        worst_l = max(worst_l, float((err / tol).max()))
        assert (err <= tol).all(), (t, float(err.max()), float(want.abs().max()))
        ids = want.argmax(-1).to(torch.int32)
    assert kv_err and max(kv_err) <= 1.0, max(kv_err)
    print(f"config-3 widths, {layers} layer(s): worst hidden error {worst_h:.2f} of the bound, logits {worst_l:.2f}, "
          f"k/v {max(kv_err):.2f}")


def _ref_prefill(cfg, w, ids, page):
    """CPU restatement of the prefill branch: all tokens at once, attention over the dequantised completed
    pages followed by the staged tail, causal; returns (last-token logits, per-layer K, V as appended)."""
    S = ids.numel()
    x = w.embed.cpu()[ids.long()]
    Ks, Vs = [], []
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2).float() / cfg.head_dim))

    def rope_all(t):                       # t (S, H, D)
        ang = torch.arange(S).float()[:, None] * inv[None, :]
        cos = torch.cat([ang, ang], -1).cos().half()[:, None, :]
        sin = torch.cat([ang, ang], -1).sin().half()[:, None, :]
        D = t.shape[-1]
        rot = torch.cat([-t[..., D // 2:], t[..., : D // 2]], dim=-1)
        return t * cos + rot * sin
    delta = None
    for lw in w.layers:
        if delta is not None:
            x = x + delta
        n = _rms(x, lw.input_norm.cpu(), cfg.rms_eps)
        q = rope_all(_awq(n, lw.q_proj).view(S, cfg.q_heads, cfg.head_dim))
        k = rope_all(_awq(n, lw.k_proj).view(S, cfg.kv_heads, cfg.head_dim))
        v = _awq(n, lw.v_proj).view(S, cfg.kv_heads, cfg.head_dim)
        K4, V4 = k.transpose(0, 1).unsqueeze(0).contiguous(), v.transpose(0, 1).unsqueeze(0).contiguous()
        Ks.append(K4); Vs.append(V4)
        nq = S - S % page
        kq, vq = oracle.quantize_k_int4(K4[:, :, :nq], page), oracle.quantize_v_int4(V4[:, :, :nq])
        Kf = torch.cat([oracle.dequantize_k_int4(*kq, page).half(), K4[:, :, nq:]], 2).float()
        Vf = torch.cat([oracle.dequantize_v_int4(*vq).half(), V4[:, :, nq:]], 2).float()
        n_rep = cfg.q_heads // cfg.kv_heads
        sc = q.transpose(0, 1).float() @ Kf[0].repeat_interleave(n_rep, 0).transpose(-1, -2) / math.sqrt(cfg.head_dim)
        i, j = torch.arange(S)[:, None], torch.arange(S)[None, :]
        att = torch.softmax(sc.masked_fill(j > i, float("-inf")), -1) @ Vf[0].repeat_interleave(n_rep, 0)      # (Hq, S, D)
        x = x + _awq(att.transpose(0, 1).reshape(S, -1).half(), lw.o_proj)
        n = _rms(x, lw.post_norm.cpu(), cfg.rms_eps)
        act = torch.nn.functional.silu(_awq(n, lw.gate_proj).float()).half() * _awq(n, lw.up_proj)
        delta = _awq(act, lw.down_proj)
    x = x + delta
    n = _rms(x[-1:], w.final_norm.cpu(), cfg.rms_eps)
    return (n.float() @ w.lm_head.cpu().float().T).half(), Ks, Vs


def test_prefill_then_decode():
    """Prefill of a 45-token prompt (tensor-core AWQ GEMM, per-token RoPE, bulk quantise-on-append, dense causal
    attention over dequantised pages + tail) against the CPU restatement, then decode steps that continue from
    the cache the prefill left (teacher-forced cache, tight bound)."""
    from flashquest_b200.eager.llama_decode import LlamaConfig, LlamaInt4Decoder, random_llama_weights
    cfg = LlamaConfig(hidden=256, layers=2, q_heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=512)
    w = random_llama_weights(cfg, "cuda", seed=5)
    page, S = 16, 45
    dec = LlamaInt4Decoder(cfg, w, batch_size=1, max_seq_len=96, page_size=page, retention=1.0, num_sinks=1, window_pages=1)
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, cfg.vocab, (S,), generator=g, dtype=torch.int32)
    nxt = dec.prefill(ids.cuda())
    got = dec.logits.float().cpu()
    want, Ks, Vs = _ref_prefill(cfg, w, ids, page)
    want = want.float()
    tol = 3e-2 * want.abs().max().item() + 1e-2          # free-running: the 4-bit codes of k / v may differ by a step
    assert (got - want).abs().max().item() <= tol, ((got - want).abs().max().item(), tol)
    assert dec.cache.get_seq_length(0) == S
    # what layer 0 appended depends on the embedding, the norm, the tensor-core GEMM and the per-token RoPE only: tight
    vw = dec.cache.get_views(0)
    for name, ref_t in (("K_partial", Ks[0]), ("V_partial", Vs[0])):
        err = (vw[name].float().cpu() - ref_t[:, :, 32:].float()).abs().max().item()
        assert err <= 2e-3 * ref_t.float().abs().max().item() + 4e-3, (name, err)       # + sin/cos of fp32 angles (see the RoPE op test)
    # decode continues from the prefilled cache
    ref = _Ref(cfg, w, page, 1.0, 1, 1, dec.attn.k_max_static)
    ref.K, ref.V = [k.clone() for k in Ks], [v.clone() for v in Vs]
    ids_t = want.argmax(-1).to(torch.int32)
    for t in range(6):
        dec.decode_step(ids_t.cuda())
        got = dec.logits.float().cpu()
        want = ref.step(ids_t, views_fn=dec.cache.get_views).float()
        tol = 2e-3 * want.abs().max() + 2 ** -11 * want.abs()
        assert ((got - want).abs() <= tol).all(), (t, float((got - want).abs().max()))
        ids_t = want.argmax(-1).to(torch.int32)


def test_graph_replayed_decode_equals_stream_decode():
    """One captured graph replayed per token (positions on the device, ids fed back on the device)
    produces the same logits and tokens as decode_step(), bit for bit, across a page boundary."""
    from flashquest_b200.eager.llama_decode import LlamaConfig, LlamaInt4Decoder, random_llama_weights
    cfg = LlamaConfig(hidden=256, layers=2, q_heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=512)
    w = random_llama_weights(cfg, "cuda", seed=2)
    mk = lambda: LlamaInt4Decoder(cfg, w, batch_size=2, max_seq_len=64, page_size=16, retention=0.5, num_sinks=1, window_pages=1)
    a, b = mk(), mk()
    ids0 = torch.tensor([7, 123], dtype=torch.int32, device="cuda")
    for d in (a, b):                                   # a few ordinary steps first: the capture starts mid-page
        ids = ids0
        for _ in range(5):
            ids = d.decode_step(ids).clone()
    replay = a.capture_decode_graph(ids)
    ids_b = ids
    for t in range(20):
        ids_a = replay().clone()
        la = a.logits.clone()
        ids_b = b.decode_step(ids_b).clone()
        assert torch.equal(la, b.logits), t
        assert torch.equal(ids_a, ids_b), t
    assert a.cache.get_seq_length(0) == b.cache.get_seq_length(0) == 25
