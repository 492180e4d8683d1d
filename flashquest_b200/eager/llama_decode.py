"""A Llama-shaped decode step on top of the sparse-decode path.

The reference reaches its kernels through a monkey-patched Hugging Face attention forward
(flashquest/eager/llama_persistent_patch.py:164-305) inside HF's decoder-layer loop; the norms,
residuals, rotary embedding and the SwiGLU MLP around it are HF's.  This module is that loop
for one new token per sequence, written against the C ABI: per layer

    add+RMSNorm -> fused AWQ q/k/v GEMV -> RoPE -> append + score + select + sparse attention
    -> AWQ o GEMV -> add+RMSNorm -> fused AWQ gate/up GEMV -> SwiGLU -> AWQ down GEMV

and after the last layer add+RMSNorm -> fp16 lm_head GEMV -> argmax.  Weights are passed in;
`random_llama_weights` builds a seeded random-init set of a given architecture (AWQ tensors
with uniform codes, scales ~ U(0.001, 0.02)), which is what the benchmark uses.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import ctypes

import torch

from .._lib import (AwqLinearDesc, LlamaLayerDesc, LlamaModelDesc, LlamaScratchDesc, check, lib, ptr, stream_ptr)
from ..cache.persistent_int4 import PersistentInt4KVCache
from ..kernel.fused_proj import awq_gemv_fused
from ..quant import AWQLinear
from .decode_step import QuestDecodeInt4


@dataclass
class LlamaConfig:
    hidden: int = 3072
    layers: int = 28
    q_heads: int = 24
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 8192
    vocab: int = 128256
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    group_size: int = 128


@dataclass
class LlamaLayerWeights:
    input_norm: torch.Tensor
    q_proj: AWQLinear
    k_proj: AWQLinear
    v_proj: AWQLinear
    o_proj: AWQLinear
    post_norm: torch.Tensor
    gate_proj: AWQLinear
    up_proj: AWQLinear
    down_proj: AWQLinear


@dataclass
class LlamaWeights:
    embed: torch.Tensor                 # (vocab, hidden) fp16
    layers: List[LlamaLayerWeights] = field(default_factory=list)
    final_norm: Optional[torch.Tensor] = None
    lm_head: Optional[torch.Tensor] = None   # (vocab, hidden) fp16


def _awq(K, N, group, gen, dev):
    qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), dtype=torch.int32, device=dev, generator=gen)
    qz = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // group, N // 8), dtype=torch.int32, device=dev, generator=gen)
    sc = (torch.rand(K // group, N, device=dev, generator=gen) * 0.019 + 0.001).half()
    return AWQLinear(qw, sc, qz, group_size=group)


def random_llama_weights(cfg: LlamaConfig, device, seed: int = 0, scale_down: float = 1.0) -> LlamaWeights:
    """Seeded random-init weights of the given architecture.  `scale_down` multiplies the AWQ
    scales (random 4-bit codes with zero-mean offsets make activations grow layer by layer;
    tests use it to keep values inside fp16)."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    H, D = cfg.hidden, cfg.head_dim
    w = LlamaWeights(embed=(torch.randn(cfg.vocab, H, device=dev, generator=g) * 0.02).half())

    def lin(K, N):
        a = _awq(K, N, cfg.group_size, g, dev)
        if scale_down != 1.0:
            a.scales = (a.scales.float() * scale_down).half()
        return a

    for _ in range(cfg.layers):
        w.layers.append(LlamaLayerWeights(
            input_norm=(1.0 + 0.1 * torch.randn(H, device=dev, generator=g)).half(),
            q_proj=lin(H, cfg.q_heads * D), k_proj=lin(H, cfg.kv_heads * D), v_proj=lin(H, cfg.kv_heads * D),
            o_proj=lin(cfg.q_heads * D, H),
            post_norm=(1.0 + 0.1 * torch.randn(H, device=dev, generator=g)).half(),
            gate_proj=lin(H, cfg.ffn), up_proj=lin(H, cfg.ffn), down_proj=lin(cfg.ffn, H)))
    w.final_norm = (1.0 + 0.1 * torch.randn(H, device=dev, generator=g)).half()
    w.lm_head = (torch.randn(cfg.vocab, H, device=dev, generator=g) * 0.02).half()
    return w


class LlamaInt4Decoder:
    """Greedy decode, one token per call and sequence, over a persistent INT4 cache."""

    def __init__(self, cfg: LlamaConfig, weights: LlamaWeights, *, batch_size: int, max_seq_len: int, page_size: int = 16,
                 retention: float = 0.25, num_sinks: int = 1, window_pages: int = 1, device="cuda"):
        self.cfg, self.w = cfg, weights
        self.dev = torch.device(device)
        self.B = batch_size
        self.cache = PersistentInt4KVCache(batch_size=batch_size, num_layers=cfg.layers, num_kv_heads=cfg.kv_heads,
                                           head_dim=cfg.head_dim, max_seq_len=max_seq_len, page_size=page_size,
                                           device=self.dev, dtype=torch.float16)
        self.attn = QuestDecodeInt4(self.cache, num_q_heads=cfg.q_heads, retention=retention, num_sinks=num_sinks,
                                    window_pages=window_pages, q_dtype=torch.float16)
        H = cfg.hidden
        mk = lambda *s: torch.empty(*s, dtype=torch.float16, device=self.dev)
        self.resid = [mk(batch_size, H), mk(batch_size, H)]      # the residual stream alternates between the two
        self.normed, self.act = mk(batch_size, H), mk(batch_size, cfg.ffn)
        self.logits = mk(batch_size, cfg.vocab)
        self.next_ids = torch.empty(batch_size, dtype=torch.int32, device=self.dev)
        self.launches = 0
        self._build_native()

    def _build_native(self):
        """Descriptors of the one-call step (fq_llama_decode_step): weights and scratch."""
        c, w, B, a = self.cfg, self.w, self.B, self.attn
        L = lib()

        def lin(x):
            return AwqLinearDesc(ptr(x.qweight), ptr(x.scales), ptr(x.qzeros), ptr(x.bias), x.in_features, x.out_features)

        self._layers = (LlamaLayerDesc * c.layers)(*[
            LlamaLayerDesc(ptr(lw.input_norm), lin(lw.q_proj), lin(lw.k_proj), lin(lw.v_proj), lin(lw.o_proj),
                           ptr(lw.post_norm), lin(lw.gate_proj), lin(lw.up_proj), lin(lw.down_proj)) for lw in w.layers])
        inter = int(bool(getattr(w.layers[0].q_proj, "interleaved", True)))
        self._model = LlamaModelDesc(c.hidden, c.layers, c.q_heads, c.kv_heads, c.head_dim, c.ffn, c.vocab, c.group_size, inter,
                                     c.rope_theta, c.rms_eps, self._layers, ptr(w.final_norm), ptr(w.lm_head))
        mk = lambda *s: torch.empty(*s, dtype=torch.float16, device=self.dev)
        nq, nkv = c.q_heads * c.head_dim, c.kv_heads * c.head_dim
        self._nat = dict(q=mk(B, nq), k=mk(B, nkv), v=mk(B, nkv), attn_out=mk(B, c.hidden), down=mk(B, c.hidden),
                         gate=mk(B, c.ffn), up=mk(B, c.ffn))
        n = self._nat
        self._scratch = LlamaScratchDesc(
            ptr(self.resid[0]), ptr(self.resid[1]), ptr(self.normed), ptr(n["q"]), ptr(n["k"]), ptr(n["v"]),
            ptr(n["attn_out"]), ptr(n["down"]), ptr(n["gate"]), ptr(n["up"]), ptr(self.logits), ptr(self.next_ids),
            ptr(a.scores), a.scores.stride(0), ptr(a.compact), a.compact.stride(0), ptr(a.O), a.O.stride(0),
            ptr(a.workspace), a.workspace.stride(0), a.workspace.shape[1])

    def decode_step(self, token_ids: torch.Tensor) -> torch.Tensor:
        """token_ids (B,) -> next token ids (B,) int32 (greedy), the whole step in one foreign call
        (fq_llama_decode_step); logits of the step stay in self.logits."""
        c = self.cache
        n_l = self.cfg.layers
        x = self.w.embed[token_ids.long()]                       # (B, H) gather: plumbing
        seen = (ctypes.c_int * n_l)(*c._seen_tokens[:n_l])
        if c._seen_tokens[0] + 1 > c.max_seq_len:
            raise RuntimeError(f"PersistentInt4KVCache: seen+new={c._seen_tokens[0] + 1} exceeds max_seq_len={c.max_seq_len}")
        check(lib().fq_llama_decode_step(ctypes.byref(self._model), ctypes.byref(self.attn._cdesc), ctypes.byref(self.attn._prm),
                                         seen, ptr(x), self.B, ctypes.byref(self._scratch), stream_ptr(self.dev)))
        for li in range(n_l):
            c._seen_tokens[li] += 1
        self.launches += 8 * n_l + 3
        return self.next_ids

    def prefill(self, token_ids: torch.Tensor) -> torch.Tensor:
        """Prefill of ONE sequence (batch_size must be 1): token_ids (S,) are run through all layers at
        once — the S_q > 1 branch of the reference's patched forward
        (flashquest/eager/llama_persistent_patch.py:196-201) inside HF's layer loop: per layer
        add+RMSNorm over all rows, fused AWQ q/k/v on the tensor-core dequant-GEMM, RoPE per token,
        bulk quantise-on-append of the S tokens, dense causal attention over the dequantised
        completed pages followed by the staged tail, AWQ o / gate / up / down GEMMs, SwiGLU; after
        the last layer the final norm, lm_head and argmax of the LAST token only.  Returns the next
        token id (1,) int32 (greedy); self.logits holds the last token's logits."""
        from ..kernel.fused_proj import awq_gemm_fused, awq_linear_fused
        from ..kernel.kv_quant import dequantize_k_int4, dequantize_v_int4
        from ..kernel.prefill_attn import prefill_causal_attention
        c, w = self.cfg, self.w
        if self.B != 1:
            raise NotImplementedError("prefill runs one sequence; batch the decode steps instead")
        cache = self.cache
        if cache.get_seq_length(0) != 0:
            raise RuntimeError("prefill expects an empty cache")
        S = int(token_ids.numel())
        if S > cache.max_seq_len:
            raise RuntimeError(f"PersistentInt4KVCache: seen+new={S} exceeds max_seq_len={cache.max_seq_len}")
        L = lib()
        st = stream_ptr(self.dev)
        H, D, Hq, Hkv = c.hidden, c.head_dim, c.q_heads, c.kv_heads
        lin = awq_linear_fused                                     # the GEMV below 9 rows, the tensor-core GEMM above
        x = w.embed[token_ids.to(self.dev).long()]                # (S, H) gather: plumbing
        normed = torch.empty_like(x)
        delta = None
        for li, lw in enumerate(w.layers):
            if delta is None:
                check(L.fq_add_rmsnorm(ptr(x), None, ptr(lw.input_norm), c.rms_eps, S, H, None, ptr(normed), st))
            else:
                x2 = torch.empty_like(x)
                check(L.fq_add_rmsnorm(ptr(x), ptr(delta), ptr(lw.input_norm), c.rms_eps, S, H, ptr(x2), ptr(normed), st))
                x = x2
            q, k, v = lin(normed, (lw.q_proj, lw.k_proj, lw.v_proj))                 # (S, Hq*D), (S, Hkv*D) x2
            check(L.fq_rope_tokens(ptr(q), Hq * D, D, Hq, ptr(k), Hkv * D, D, Hkv, S, D, 0, c.rope_theta, st))
            q4 = q.view(1, S, Hq, D).transpose(1, 2)               # (1, Hq, S, D) views, token stride Hq*D
            k4, v4 = k.view(1, S, Hkv, D).transpose(1, 2), v.view(1, S, Hkv, D).transpose(1, 2)
            cache.update_quantized(k4, v4, li)
            vw = cache.get_views(li)
            if vw["completed_len"] > 0:
                # bf16 -> fp16 is exact: the reference's bf16-rounded dequantised values, in the staging dtype
                Kd = dequantize_k_int4(vw["K_packed"], vw["K_scale"], vw["K_mn"], cache.page_size).to(cache.dtype)
                Vd = dequantize_v_int4(vw["V_packed"], vw["V_scale"], vw["V_mn"]).to(cache.dtype)
                K_full, V_full = torch.cat([Kd, vw["K_partial"]], 2), torch.cat([Vd, vw["V_partial"]], 2)
                del Kd, Vd
            else:
                K_full, V_full = vw["K_partial"], vw["V_partial"]
            attn = prefill_causal_attention(q4, K_full, V_full, out_bshd=True).view(S, Hq * D)
            del K_full, V_full, q, k, v
            (attn_out,) = lin(attn, (lw.o_proj,))
            x2 = torch.empty_like(x)
            check(L.fq_add_rmsnorm(ptr(x), ptr(attn_out), ptr(lw.post_norm), c.rms_eps, S, H, ptr(x2), ptr(normed), st))
            x = x2
            gate, up = lin(normed, (lw.gate_proj, lw.up_proj))
            act = torch.empty_like(gate)
            check(L.fq_swiglu(ptr(gate), ptr(up), gate.numel(), ptr(act), st))
            (delta,) = lin(act, (lw.down_proj,))
            del gate, up, act, attn, attn_out
            self.launches += 12
        last = torch.empty(1, H, dtype=torch.float16, device=self.dev)
        check(L.fq_add_rmsnorm(ptr(x[S - 1:]), ptr(delta[S - 1:]), ptr(w.final_norm), c.rms_eps, 1, H, ptr(last), ptr(self.normed), st))
        check(L.fq_gemv_f16(ptr(self.normed), ptr(w.lm_head), 1, H, c.vocab, ptr(self.logits), st))
        check(L.fq_argmax_f16(ptr(self.logits), 1, c.vocab, ptr(self.next_ids), st))
        self.launches += 3
        return self.next_ids

    # -- thin wrappers over the C ABI ------------------------------------------------------
    def _add_rmsnorm(self, a, b, weight, sum_out, y):
        check(lib().fq_add_rmsnorm(ptr(a), ptr(b), ptr(weight), self.cfg.rms_eps, a.shape[0], a.shape[1],
                                   ptr(sum_out), ptr(y), stream_ptr(self.dev)))
        self.launches += 1

    def _rope(self, q, k, pos):
        c = self.cfg
        check(lib().fq_rope(ptr(q), q.stride(0), q.stride(1), c.q_heads, ptr(k), k.stride(0), k.stride(1), c.kv_heads,
                            self.B, c.head_dim, int(pos), c.rope_theta, stream_ptr(self.dev)))
        self.launches += 1

    def capture_decode_graph(self, token_ids: torch.Tensor):
        """CUDA graph of one greedy step that feeds itself: embedding gather of the ids buffer, the
        whole step with the positions read on the device (fq_llama_decode_step_dev), and the copy
        of the chosen ids back into the buffer.  Returns `replay`; each call decodes one more token
        per sequence with no host work besides the launch (`replay.ids` holds the latest ids,
        self.logits the latest logits).  Do not mix with decode_step() without capturing again."""
        c, n_l = self.cache, self.cfg.layers
        ids = token_ids.to(device=self.dev, dtype=torch.int32).clone()
        pos = torch.tensor(c._seen_tokens[:n_l], dtype=torch.int32, device=self.dev)
        # stateless warm-up launches: lazily set kernel attributes stay outside the capture
        cfg = self.cfg
        self.attn.attend(torch.zeros(self.B, cfg.q_heads, 1, cfg.head_dim, dtype=torch.float16, device=self.dev), 0)
        lw = self.w.layers[0]
        awq_gemv_fused(self.normed.view(self.B, 1, -1), (lw.q_proj, lw.k_proj, lw.v_proj))
        awq_gemv_fused(self.act.view(self.B, 1, -1), (lw.down_proj,))       # shared memory size of the widest K range
        torch.cuda.synchronize(self.dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            x = self.w.embed[ids.long()]
            check(lib().fq_llama_decode_step_dev(ctypes.byref(self._model), ctypes.byref(self.attn._cdesc),
                                                 ctypes.byref(self.attn._prm), ptr(pos), ptr(x), self.B,
                                                 ctypes.byref(self._scratch), stream_ptr(self.dev)))
            ids.copy_(self.next_ids)

        def replay():
            if c._seen_tokens[0] + 1 > c.max_seq_len:
                raise RuntimeError(f"PersistentInt4KVCache: seen+new={c._seen_tokens[0] + 1} exceeds max_seq_len={c.max_seq_len}")
            graph.replay()
            for li in range(n_l):
                c._seen_tokens[li] += 1
            self.launches += 8 * n_l + 4
            return ids

        replay.graph, replay.ids, replay.pos = graph, ids, pos
        return replay

    def decode_step_per_op(self, token_ids: torch.Tensor, trace: Optional[list] = None) -> torch.Tensor:
        """The same step issued operator by operator from Python (one foreign call per kernel group).
        `trace`, if given, receives a copy of the residual stream after every addition (2 per layer + 1):
        the hidden states a per-block comparison needs."""
        c, w, B = self.cfg, self.w, self.B
        L = lib()
        st = stream_ptr(self.dev)
        pos = self.cache.get_seq_length(0)
        x = w.embed[token_ids.long()]                            # (B, H) gather: plumbing
        flip = 0

        def add_norm(x, delta, weight):
            """x <- x + delta (into the residual buffer that does not hold x); normed <- RMSNorm(x)."""
            nonlocal flip
            if delta is None:
                self._add_rmsnorm(x, None, weight, None, self.normed)
                return x
            out = self.resid[flip]
            flip ^= 1
            self._add_rmsnorm(x, delta, weight, out, self.normed)
            if trace is not None:
                trace.append(out.clone())
            return out

        delta = None                                             # output of the previous block, not yet added
        for li, lw in enumerate(w.layers):
            x = add_norm(x, delta, lw.input_norm)
            q, k, v = awq_gemv_fused(self.normed.view(B, 1, -1), (lw.q_proj, lw.k_proj, lw.v_proj))
            q = q.view(B, c.q_heads, c.head_dim)
            k = k.view(B, c.kv_heads, c.head_dim)
            v = v.view(B, c.kv_heads, 1, c.head_dim)
            self._rope(q, k, pos)
            O, _ = self.attn.step(k.unsqueeze(2), v, q.unsqueeze(2), li)
            (attn_out,) = awq_gemv_fused(O.reshape(B, 1, c.q_heads * c.head_dim), (lw.o_proj,))
            x = add_norm(x, attn_out.view(B, -1), lw.post_norm)
            gate, up = awq_gemv_fused(self.normed.view(B, 1, -1), (lw.gate_proj, lw.up_proj))
            check(L.fq_swiglu(ptr(gate), ptr(up), gate.numel(), ptr(self.act), st))
            (down,) = awq_gemv_fused(self.act.view(B, 1, -1), (lw.down_proj,))
            delta = down.view(B, -1)
            self.launches += 5
        x = add_norm(x, delta, w.final_norm)
        check(L.fq_gemv_f16(ptr(self.normed), ptr(w.lm_head), B, c.hidden, c.vocab, ptr(self.logits), st))
        check(L.fq_argmax_f16(ptr(self.logits), B, c.vocab, ptr(self.next_ids), st))
        self.launches += 2
        return self.next_ids
