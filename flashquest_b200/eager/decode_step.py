"""Decode-branch dispatcher for the persistent INT4 cache: score -> select -> attend.

Host-side counterpart of the decode branch of make_quest_persistent_forward
(flashquest/eager/llama_persistent_patch.py:202-245): static k_max / BUCKET_MAX computed
once (:77-85), per-head retention from a head pattern (:214-219), page scores from the
metadata, top-k + compact index, sparse attention over the selected pages, and the staged
tail merged in the same softmax.  Three kernel launches per layer, no allocation per step
(all outputs preallocated), so a whole multi-layer step can be captured in a CUDA graph.
"""
from __future__ import annotations

import ctypes
import math

import torch

from .._lib import DecodeParams, Int4CacheDesc, TurboCacheDesc, check, dtype_code, lib, ptr, stream_ptr


class QuestDecodeInt4:
    def __init__(self, cache, *, num_q_heads: int, retention: float = 0.20, num_sinks: int = 4,
                 window_pages: int = 2, head_pattern_layer: torch.Tensor | None = None,
                 q_dtype=torch.bfloat16, n_split: int | None = None):
        if getattr(cache, "kv_bits", None) != 4:
            raise NotImplementedError(f"QuestDecodeInt4 only supports kv_bits=4; got {getattr(cache, 'kv_bits', None)}")
        if not (0.0 <= float(retention) <= 1.0):
            raise ValueError(f"scalar retention must be in [0, 1]; got {retention}")
        self.cache = cache
        self.Hq = num_q_heads
        self.Hkv = cache.num_kv_heads
        if self.Hq % self.Hkv != 0:
            raise ValueError(f"H_q={self.Hq} must be divisible by H_kv={self.Hkv}")
        self.D = cache.head_dim
        self.page = cache.page_size
        self.B = cache.batch_size
        self.retention = float(retention)
        self.num_sinks = int(num_sinks)
        self.window_pages = int(window_pages)
        # eager/llama_persistent_patch.py:77-85
        P_max = cache.max_seq_len // self.page
        self.k_max_static = math.ceil(self.retention * P_max)
        self.bucket = max(1, self.k_max_static + self.num_sinks + self.window_pages)
        dev = cache.K_packed.device
        self.device = dev
        self.q_dtype = q_dtype
        self.sm_scale = 1.0 / math.sqrt(self.D)
        self.retention_per_q = None
        if head_pattern_layer is not None:
            # retrieval heads keep `retention`, streaming heads 0 (:214-219)
            n_rep = self.Hq // self.Hkv
            pat = head_pattern_layer.to(dev).bool().repeat_interleave(n_rep)
            self.retention_per_q = torch.where(pat, torch.full((self.Hq,), self.retention, device=dev),
                                               torch.zeros(self.Hq, device=dev)).float().contiguous()
        L = cache.num_layers
        self.scores = torch.empty(L, self.B, self.Hq, max(P_max, 1), dtype=torch.float32, device=dev)
        self.compact = torch.empty(L, self.B, self.Hq, self.bucket, dtype=torch.int32, device=dev)
        self.O = torch.empty(L, self.B, self.Hq, self.D, dtype=q_dtype, device=dev)
        self.lse = torch.empty(L, self.B, self.Hq, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            self.n_split = n_split or lib().fq_sparse_decode_default_splits(self.B, self.Hq, self.bucket, self.page)
            nbytes = lib().fq_sparse_decode_workspace_bytes(self.B, self.Hq, self.D, self.n_split)
        # one split-K workspace per layer: launches of different layers may overlap in a graph
        self.ws_bytes = (nbytes + 255) // 256 * 256
        self.workspace = torch.zeros(L, max(self.ws_bytes, 256), dtype=torch.uint8, device=dev)
        self.launches = 0
        # descriptors for the one-call-per-layer entry point
        c = cache
        self._cdesc = Int4CacheDesc(
            c.K_packed.data_ptr(), c.V_packed.data_ptr(), *c.K_packed.stride()[:4],
            c.K_scale.data_ptr(), c.K_mn.data_ptr(), *c.K_scale.stride()[:4],
            c.V_scale.data_ptr(), c.V_mn.data_ptr(), *c.V_scale.stride()[:3],
            c.K_partial.data_ptr(), c.V_partial.data_ptr(), *c.K_partial.stride()[:4],
            dtype_code(c.K_partial), c.num_layers, self.B, self.Hkv, self.D, self.page, c.max_seq_len)
        self._prm = DecodeParams(
            self.Hq, self.retention_per_q.data_ptr() if self.retention_per_q is not None else None, self.retention,
            self.k_max_static, self.num_sinks, self.window_pages, self.bucket, self.sm_scale, self.n_split)

    def params_for(self, head_pattern_layer: torch.Tensor):
        """fq_decode_params of one layer whose retrieval / streaming KV heads are given by
        head_pattern_layer (H_kv,) bool: retrieval heads keep `retention`, streaming heads 0
        (eager/llama_persistent_patch.py:214-219).  Returns (struct, tensor kept alive by the caller)."""
        n_rep = self.Hq // self.Hkv
        pat = head_pattern_layer.to(self.device).bool().repeat_interleave(n_rep)
        r = torch.where(pat, torch.full((self.Hq,), self.retention, device=self.device),
                        torch.zeros(self.Hq, device=self.device)).float().contiguous()
        return DecodeParams(self.Hq, r.data_ptr(), self.retention, self.k_max_static, self.num_sinks, self.window_pages,
                            self.bucket, self.sm_scale, self.n_split), r

    def step(self, k_new: torch.Tensor, v_new: torch.Tensor, q: torch.Tensor, layer_idx: int, prm=None):
        """Append k_new, v_new (B,H_kv,n,D) to the layer and attend with q (B,H_q,1,D) in ONE
        foreign call (fq_decode_layer_int4): what cache.update_quantized followed by attend()
        does, without the per-call slicing.  Tensors must have the cache's dtype.  `prm`: a
        per-layer fq_decode_params (params_for) instead of the engine's own."""
        c = self.cache
        if layer_idx < 0 or layer_idx >= c.num_layers:
            raise IndexError(f"layer_idx {layer_idx} out of range [0, {c.num_layers})")
        seen = c._seen_tokens[layer_idx]
        n_new = k_new.shape[2]
        if seen + n_new > c.max_seq_len:
            raise RuntimeError(f"PersistentInt4KVCache: seen+new={seen + n_new} exceeds max_seq_len={c.max_seq_len}")
        if k_new.dtype != c.dtype or v_new.dtype != c.dtype:
            k_new, v_new = k_new.to(c.dtype), v_new.to(c.dtype)
        if k_new.stride(3) != 1 or v_new.stride() != k_new.stride():
            k_new, v_new = k_new.contiguous(), v_new.contiguous()
        q3 = q.reshape(self.B, self.Hq, self.D)
        O, lse = self.O[layer_idx], self.lse[layer_idx]
        check(lib().fq_decode_layer_int4(
            ctypes.byref(self._cdesc), layer_idx, seen,
            ptr(k_new), ptr(v_new), k_new.stride(0), k_new.stride(1), k_new.stride(2), n_new,
            ptr(q3), dtype_code(q3), q3.stride(0), q3.stride(1), ctypes.byref(prm if prm is not None else self._prm),
            ptr(self.scores[layer_idx]), ptr(self.compact[layer_idx]), ptr(O), ptr(lse),
            ptr(self.workspace[layer_idx]), self.workspace.shape[1], stream_ptr(self.device)))
        c._seen_tokens[layer_idx] = seen + n_new
        self.launches += 4
        return O.unsqueeze(2), lse.unsqueeze(2)

    def step_all(self, k_new: torch.Tensor, v_new: torch.Tensor, q: torch.Tensor):
        """step() for every layer in ONE foreign call (fq_decode_step_int4): k_new, v_new
        (L,B,H_kv,n,D) in the cache's dtype, q (L,B,H_q,1,D).  For callers that hold all layers'
        projections at once (stacked independent layers); returns (O (L,B,H_q,1,D), lse (L,B,H_q,1))."""
        c = self.cache
        Ln = c.num_layers
        n_new = k_new.shape[3]
        if k_new.shape[0] != Ln or q.shape[0] != Ln:
            raise ValueError(f"expected {Ln} layers, got {k_new.shape[0]} / {q.shape[0]}")
        for li in range(Ln):
            if c._seen_tokens[li] + n_new > c.max_seq_len:
                raise RuntimeError(f"PersistentInt4KVCache: seen+new={c._seen_tokens[li] + n_new} exceeds max_seq_len={c.max_seq_len}")
        if k_new.dtype != c.dtype or v_new.dtype != c.dtype:
            k_new, v_new = k_new.to(c.dtype), v_new.to(c.dtype)
        if k_new.stride(4) != 1 or v_new.stride() != k_new.stride():
            k_new, v_new = k_new.contiguous(), v_new.contiguous()
        q4 = q.reshape(Ln, self.B, self.Hq, self.D)
        if q4.stride(3) != 1:
            q4 = q4.contiguous()
        seen = (ctypes.c_int * Ln)(*c._seen_tokens[:Ln])
        check(lib().fq_decode_step_int4(
            ctypes.byref(self._cdesc), Ln, seen,
            ptr(k_new), ptr(v_new), k_new.stride(0), k_new.stride(1), k_new.stride(2), k_new.stride(3), n_new,
            ptr(q4), dtype_code(q4), q4.stride(0), q4.stride(1), q4.stride(2), ctypes.byref(self._prm), 0,
            ptr(self.scores), self.scores.stride(0), ptr(self.compact), self.compact.stride(0),
            ptr(self.O), self.O.stride(0), ptr(self.lse), self.lse.stride(0),
            ptr(self.workspace), self.workspace.stride(0), self.workspace.shape[1], stream_ptr(self.device)))
        for li in range(Ln):
            c._seen_tokens[li] += n_new
        self.launches += 4 * Ln
        return self.O.unsqueeze(3), self.lse.unsqueeze(3)

    def capture_step_graph(self, k_new: torch.Tensor, v_new: torch.Tensor, q: torch.Tensor, before=None, after=None):
        """CUDA graph of step_all() for the STATIC input buffers k_new, v_new (L,B,H_kv,n,D) and q
        (L,B,H_q,1,D): refill the buffers, call the returned `replay()`, read self.O / self.lse.
        The launches read the sequence length from a device array (fq_decode_step_int4_dev), so one
        capture serves every later token.  `before` / `after` (callables) are captured in the same graph
        around the step, e.g. the copies from and to pinned host buffers.  replay() keeps the cache's
        host-side counters in step;
        do not mix it with step()/step_all()/update_quantized() without capturing again."""
        c = self.cache
        Ln = c.num_layers
        n_new = k_new.shape[3]
        if not (1 <= n_new < self.page):
            raise ValueError(f"n_new={n_new} must be in [1, page_size)")
        if k_new.dtype != c.dtype or v_new.dtype != c.dtype or k_new.stride(4) != 1 or v_new.stride() != k_new.stride():
            raise ValueError("k_new / v_new must be dense tensors of the cache's dtype with equal strides")
        q4 = q.view(Ln, self.B, self.Hq, self.D)
        pos = torch.tensor(c._seen_tokens[:Ln], dtype=torch.int32, device=self.device)
        self.attend(q[0], 0)                                       # one ordinary launch: lazy kernel attributes are set outside the capture
        torch.cuda.synchronize(self.device)

        def launch():
            check(lib().fq_decode_step_int4_dev(
                ctypes.byref(self._cdesc), Ln, ptr(pos),
                ptr(k_new), ptr(v_new), k_new.stride(0), k_new.stride(1), k_new.stride(2), k_new.stride(3), n_new,
                ptr(q4), dtype_code(q4), q4.stride(0), q4.stride(1), q4.stride(2), ctypes.byref(self._prm), 0,
                ptr(self.scores), self.scores.stride(0), ptr(self.compact), self.compact.stride(0),
                ptr(self.O), self.O.stride(0), ptr(self.lse), self.lse.stride(0),
                ptr(self.workspace), self.workspace.stride(0), self.workspace.shape[1], stream_ptr(self.device)))

        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            if before is not None:
                before()
            launch()
            if after is not None:
                after()

        def replay():
            seen = max(c._seen_tokens[:Ln])
            if seen + n_new > c.max_seq_len:
                raise RuntimeError(f"PersistentInt4KVCache: seen+new={seen + n_new} exceeds max_seq_len={c.max_seq_len}")
            graph.replay()
            c._seen_tokens[:Ln] = [t + n_new for t in c._seen_tokens[:Ln]]
            self.launches += 3 * Ln + 2          # one append for all layers, 3 per layer, the position update
            return self.O.unsqueeze(3), self.lse.unsqueeze(3)

        replay.graph, replay.pos = graph, pos
        return replay

    def attend(self, q: torch.Tensor, layer_idx: int):
        """q (B,H_q,1,D) or (B,H_q,D), the cache's dtype family (fp16/bf16).  Returns views
        (O (B,H_q,1,D), lse (B,H_q,1)) of preallocated per-layer buffers."""
        c = self.cache
        seen = c._seen_tokens[layer_idx]
        page = self.page
        partial_len = seen % page
        completed = seen - partial_len
        P = completed // page
        q3 = q.reshape(self.B, self.Hq, self.D)
        li = layer_idx
        L = lib()
        st = stream_ptr(self.device)
        scores, compact = self.scores[li], self.compact[li]
        Ks, Km = c.K_scale[li], c.K_mn[li]
        if P > 0:
            check(L.fq_page_scores_int4(
                ptr(q3), dtype_code(q3), q3.stride(0), q3.stride(1),
                ptr(Ks), ptr(Km), Ks.stride(0), Ks.stride(1), Ks.stride(2),
                self.B, self.Hq, self.Hkv, P, self.D, ptr(scores), scores.stride(0), scores.stride(1), st))
            check(L.fq_select_pages(
                ptr(scores), scores.stride(0), scores.stride(1), self.B, self.Hq, P,
                ptr(self.retention_per_q), self.retention, min(self.k_max_static, P), self.num_sinks,
                self.window_pages, None, 0, 0, ptr(compact), compact.stride(0), compact.stride(1), self.bucket,
                None, st))
            self.launches += 2
        Kp, Vp, Vs, Vm = c.K_packed[li], c.V_packed[li], c.V_scale[li], c.V_mn[li]
        Kt, Vt = c.K_partial[li], c.V_partial[li]
        O, lse = self.O[li], self.lse[li]
        check(L.fq_sparse_decode_int4(
            ptr(q3), dtype_code(q3), q3.stride(0), q3.stride(1),
            ptr(Kp), Kp.stride(0), Kp.stride(1),
            ptr(Ks), ptr(Km), Ks.stride(0), Ks.stride(1), Ks.stride(2),
            ptr(Vp), Vp.stride(0), Vp.stride(1),
            ptr(Vs), ptr(Vm), Vs.stride(0), Vs.stride(1),
            ptr(compact), compact.stride(0), compact.stride(1), self.bucket if P > 0 else 0,
            ptr(Kt) if partial_len else None, ptr(Vt) if partial_len else None, dtype_code(Kt),
            Kt.stride(0), Kt.stride(1), Kt.stride(2), partial_len,
            self.B, self.Hq, self.Hkv, completed, P, self.D, page, self.sm_scale,
            ptr(O), O.stride(0), O.stride(1), ptr(lse),
            ptr(self.workspace[li]), self.workspace.shape[1], self.n_split, st))
        self.launches += 1
        return O.unsqueeze(2), lse.unsqueeze(2)


class QuestDecodeTurbo:
    """Decode-branch dispatcher for the persistent TurboQuant (K3-V3) cache: the kv_bits == 3 route of
    make_quest_persistent_forward (flashquest/eager/llama_persistent_patch.py:93-115,202-245) as ONE
    foreign call per layer (fq_decode_layer_turbo): append, page scores from the raw page metadata,
    top-k + compact index, rotation of Q, sparse attention in the rotated basis, rotation of O, tail
    attention and LSE merge.  All buffers are preallocated."""

    def __init__(self, cache, *, num_q_heads: int, retention: float = 0.20, num_sinks: int = 4, window_pages: int = 2,
                 q_dtype=torch.bfloat16, n_split: int | None = None):
        if getattr(cache, "kv_bits", None) != 3:
            raise NotImplementedError(f"QuestDecodeTurbo only supports kv_bits=3; got {getattr(cache, 'kv_bits', None)}")
        if not (0.0 <= float(retention) <= 1.0):
            raise ValueError(f"scalar retention must be in [0, 1]; got {retention}")
        self.cache = cache
        self.Hq, self.Hkv = num_q_heads, cache.num_kv_heads
        if self.Hq % self.Hkv != 0:
            raise ValueError(f"H_q={self.Hq} must be divisible by H_kv={self.Hkv}")
        self.D, self.page, self.B = cache.head_dim, cache.page_size, cache.batch_size
        if self.page % 16 != 0:
            raise NotImplementedError(f"the TurboQuant attention kernel needs page_size a multiple of 16; got {self.page}")
        self.retention, self.num_sinks, self.window_pages = float(retention), int(num_sinks), int(window_pages)
        P_max = cache.max_seq_len // self.page
        self.k_max_static = math.ceil(self.retention * P_max)
        self.bucket = max(1, self.k_max_static + self.num_sinks + self.window_pages)
        dev = cache.K_msb.device
        self.device, self.q_dtype = dev, q_dtype
        self.sm_scale = 1.0 / math.sqrt(self.D)
        self.scores = torch.empty(self.B, self.Hq, max(P_max, 1), dtype=torch.float32, device=dev)
        self.compact = torch.empty(self.B, self.Hq, self.bucket, dtype=torch.int32, device=dev)
        self.O = torch.empty(cache.num_layers, self.B, self.Hq, self.D, dtype=q_dtype, device=dev)
        self.lse = torch.empty(cache.num_layers, self.B, self.Hq, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            self.n_split = n_split or max(1, min(lib().fq_sparse_decode_default_splits(self.B, self.Hq, self.bucket, self.page), 64))
            self.scratch = torch.empty(lib().fq_decode_layer_turbo_scratch_bytes(self.B, self.Hq, self.D), dtype=torch.uint8, device=dev)
            self.workspace = torch.zeros(max(lib().fq_sparse_decode_workspace_bytes(self.B, self.Hq, self.D, self.n_split), 256),
                                         dtype=torch.uint8, device=dev)
        c = cache
        self._cdesc = TurboCacheDesc(
            c.K_msb.data_ptr(), c.K_lsb.data_ptr(), c.V_msb.data_ptr(), c.V_lsb.data_ptr(),
            *c.K_msb.stride()[:4], *c.K_lsb.stride()[:4],
            c.K_scale_turbo.data_ptr(), c.V_scale_turbo.data_ptr(), *c.K_scale_turbo.stride()[:3],
            c.K_scale_raw.data_ptr(), c.K_mn_raw.data_ptr(), *c.K_scale_raw.stride()[:4],
            c.K_partial.data_ptr(), c.V_partial.data_ptr(), *c.K_partial.stride()[:4],
            dtype_code(c.K_partial), c.num_layers, self.B, self.Hkv, self.D, self.page, c.max_seq_len)
        self._prm = DecodeParams(self.Hq, None, self.retention, self.k_max_static, self.num_sinks, self.window_pages,
                                 self.bucket, self.sm_scale, self.n_split)
        self.launches = 0

    params_for = QuestDecodeInt4.params_for

    def step(self, k_new: torch.Tensor, v_new: torch.Tensor, q: torch.Tensor, layer_idx: int, prm=None):
        """Append k_new, v_new (B,H_kv,n,D) and attend with q (B,H_q,1,D) (raw basis): (O (B,H_q,1,D), lse (B,H_q,1))."""
        c = self.cache
        if layer_idx < 0 or layer_idx >= c.num_layers:
            raise IndexError(f"layer_idx {layer_idx} out of range [0, {c.num_layers})")
        seen = c._seen_tokens[layer_idx]
        n_new = k_new.shape[2]
        if seen + n_new > c.max_seq_len:
            raise RuntimeError(f"PersistentTurboKVCache: seen+new={seen + n_new} exceeds max_seq_len={c.max_seq_len}")
        if k_new.dtype != c.dtype or v_new.dtype != c.dtype:
            k_new, v_new = k_new.to(c.dtype), v_new.to(c.dtype)
        if k_new.stride(3) != 1 or v_new.stride() != k_new.stride():
            k_new, v_new = k_new.contiguous(), v_new.contiguous()
        q3 = q.reshape(self.B, self.Hq, self.D).contiguous()
        O, lse = self.O[layer_idx], self.lse[layer_idx]
        check(lib().fq_decode_layer_turbo(
            ctypes.byref(self._cdesc), layer_idx, seen,
            ptr(k_new), ptr(v_new), k_new.stride(0), k_new.stride(1), k_new.stride(2), n_new,
            ptr(q3), dtype_code(q3), q3.stride(0), q3.stride(1), ctypes.byref(prm if prm is not None else self._prm),
            ptr(self.scores), ptr(self.compact), ptr(self.scratch), self.scratch.numel(), ptr(O), ptr(lse),
            ptr(self.workspace), self.workspace.numel(), stream_ptr(self.device)))
        c._seen_tokens[layer_idx] = seen + n_new
        self.launches += 10
        return O.unsqueeze(2), lse.unsqueeze(2)
