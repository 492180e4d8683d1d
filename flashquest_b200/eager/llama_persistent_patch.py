"""Monkey-patch of Hugging Face's LlamaAttention.forward onto the persistent quantised caches —
CUDA counterpart of flashquest/eager/llama_persistent_patch.py:64-305, same two entry points,
keywords, defaults and error messages, so that switching is one import.

Per call the patched forward projects q/k/v with the module's own linears, applies HF's rotary
embedding, appends k/v to the persistent cache and attends:

  * prefill (S_q > 1, reference :196-201): dense causal attention over the dequantised
    completed pages followed by the staged tail (fq_prefill_attention);
  * decode (S_q == 1, reference :202-245): page scores from the quantised metadata, static-k_max
    top-k with per-head retention from the head pattern, sparse attention over the selected
    pages, tail attention over the staged tokens and the LSE merge.
      kv_bits == 4 or 8, use_compact_kernel=False: the reference's own sequence of steps — bool
        mask, sparse kernel, separate tail attention, two-way merge of bf16 partial results;
      kv_bits == 4, use_compact_kernel=True: ONE foreign call per layer (fq_decode_layer_int4:
        append + scores + top-k with compact index + attention with the tail in the same softmax);
      kv_bits == 3: ONE foreign call per layer (fq_decode_layer_turbo).
    An empty cache (no completed page) and a cache without tail take the reference's branches
    (:206-209, :236-237).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from transformers.models.llama.modeling_llama import LlamaAttention, apply_rotary_pos_emb

from ..kernel.kv_quant import (dequantize_k, dequantize_k_int4, dequantize_k_turbo, dequantize_v, dequantize_v_int4,
                               dequantize_v_turbo)
from ..kernel.prefill_attn import prefill_causal_attention
from ..kernel.sparse_fwd import flash_attn_sparse_fwd
from ..kernel.sparse_int4_fwd import flash_attn_sparse_int4_fwd
from .criticality import page_scores_int4_fast, page_scores_int8_fast
from .decode_step import QuestDecodeInt4, QuestDecodeTurbo
from .selection import select_pages_vectorized
from .tail_merge import _bf16_dense_attn_with_lse, _merge_two_attentions

# Test hook: a callable (layer_idx, q, k, v, attn_output) invoked after every attention of a patched
# module, with q/k/v as they go into the cache (after the rotary embedding and the dtype cast) and
# attn_output (B,H_q,S_q,D) as it leaves the attention.  None in normal use.
TRACE = None


def _engine(cache, kind, num_q_heads, retention, num_sinks, window_pages):
    """One preallocated native step object per cache and configuration, shared by all layers."""
    key = (kind, num_q_heads, float(retention), int(num_sinks), int(window_pages))
    store = cache.__dict__.setdefault("_fq_engines", {})
    if key not in store:
        cls = QuestDecodeInt4 if kind == 4 else QuestDecodeTurbo
        store[key] = cls(cache, num_q_heads=num_q_heads, retention=retention, num_sinks=num_sinks,
                         window_pages=window_pages, q_dtype=cache.dtype)
    return store[key]


def make_quest_persistent_forward(
    *,
    cache,
    head_pattern_layer: torch.Tensor,
    retention: float,
    num_sinks: int,
    window_pages: int,
    page_size: int,
    use_compact_kernel: bool = False,
):
    kv_bits = getattr(cache, "kv_bits", 8)
    head_dim = cache.head_dim

    # static k_max + BUCKET_MAX, no per-step .item() (reference :77-85)
    max_seq_len = getattr(cache, "max_seq_len", 32768)
    P_max = max_seq_len // page_size
    if isinstance(retention, float):
        retention_max = float(retention)
    else:
        retention_max = float(retention.max().item())
    k_max_static = math.ceil(retention_max * P_max)

    if use_compact_kernel and kv_bits != 4:
        raise NotImplementedError(
            f"Phase 8a: use_compact_kernel only supports kv_bits=4; got {kv_bits}. "
            f"INT8/Turbo compact kernels deferred to Phase 8b."
        )
    if kv_bits == 3:
        def _dequant_k_from_views(views):
            return dequantize_k_turbo(views["K_msb"], views["K_lsb"], views["K_scale_turbo"], head_dim=head_dim)

        def _dequant_v_from_views(views):
            return dequantize_v_turbo(views["V_msb"], views["V_lsb"], views["V_scale_turbo"], head_dim=head_dim)
    elif kv_bits == 4:
        def _dequant_k_from_views(views):
            return dequantize_k_int4(views["K_packed"], views["K_scale"], views["K_mn"], page_size=page_size)

        def _dequant_v_from_views(views):
            return dequantize_v_int4(views["V_packed"], views["V_scale"], views["V_mn"])
    elif kv_bits == 8:
        def _dequant_k_from_views(views):
            return dequantize_k(views["K_uint8"], views["K_scale"], views["K_mn"], page_size=page_size)

        def _dequant_v_from_views(views):
            return dequantize_v(views["V_uint8"], views["V_scale"], views["V_mn"])
    else:
        raise ValueError(f"unsupported cache.kv_bits={kv_bits!r}")
    if page_size != cache.page_size:
        raise ValueError(f"page_size={page_size} differs from the cache's page_size={cache.page_size}")
    state = {}       # per-layer fq_decode_params (+ the retention tensor it points to), built on first use

    def _layer_params(engine, device):
        if "prm" not in state:
            state["prm"] = engine.params_for(head_pattern_layer.to(device))
        return state["prm"][0]

    def forward(
        self,
        hidden_states: torch.Tensor,
        position_embeddings: tuple[torch.Tensor, torch.Tensor],
        attention_mask: Optional[torch.Tensor] = None,
        past_key_values: Optional[object] = None,
        cache_position: Optional[torch.LongTensor] = None,
        **kwargs,
    ) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
        input_shape = hidden_states.shape[:-1]
        hidden_shape = (*input_shape, -1, self.head_dim)

        q = self.q_proj(hidden_states).view(hidden_shape).transpose(1, 2)
        k = self.k_proj(hidden_states).view(hidden_shape).transpose(1, 2)
        v = self.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)

        cos, sin = position_embeddings
        q, k = apply_rotary_pos_emb(q, k, cos, sin)

        # the kernels and the cache work in the cache's staging dtype (bf16 in the reference);
        # AWQ models are fp16: cast in, cast back before o_proj (reference :182-190)
        model_dtype = q.dtype
        if model_dtype != cache.dtype:
            q, k, v = q.to(cache.dtype), k.to(cache.dtype), v.to(cache.dtype)

        S_q = q.shape[2]
        H_q = q.shape[1]
        li = self.layer_idx

        if S_q > 1:
            cache.update_quantized(k, v, layer_idx=li)
            views = cache.get_views(li)
            if views["completed_len"] > 0:
                K_full = torch.cat([_dequant_k_from_views(views).to(cache.dtype), views["K_partial"]], dim=2)
                V_full = torch.cat([_dequant_v_from_views(views).to(cache.dtype), views["V_partial"]], dim=2)
            else:
                K_full, V_full = views["K_partial"], views["V_partial"]
            attn_bhsd = None
            attn_output = prefill_causal_attention(q, K_full, V_full, out_bshd=True)            # (B,S_q,H_q,D)
            if TRACE is not None:
                attn_bhsd = attn_output.transpose(1, 2)
        elif kv_bits == 3 or use_compact_kernel:
            engine = _engine(cache, kv_bits, H_q, retention, num_sinks, window_pages)
            O, _ = engine.step(k, v, q, li, prm=_layer_params(engine, q.device))
            attn_bhsd = O
            attn_output = O.transpose(1, 2)
        else:
            cache.update_quantized(k, v, layer_idx=li)
            views = cache.get_views(li)
            partial_len = views["partial_len"]
            completed_len = views["completed_len"]
            if completed_len == 0:
                attn_bhsd, _ = _bf16_dense_attn_with_lse(q, views["K_partial"], views["V_partial"])
            else:
                H_kv = cache.num_kv_heads
                n_rep = H_q // H_kv
                pattern_per_q = head_pattern_layer.to(q.device).repeat_interleave(n_rep)
                retention_per_q = torch.where(
                    pattern_per_q,
                    torch.full((H_q,), retention, device=q.device),
                    torch.zeros(H_q, device=q.device),
                )
                score_fn = page_scores_int4_fast if kv_bits == 4 else page_scores_int8_fast
                scores = score_fn(q, views["K_scale"], views["K_mn"])
                sel = select_pages_vectorized(scores, retention=retention_per_q, num_sinks=num_sinks,
                                              window_pages=window_pages, k_max_static=k_max_static)
                if kv_bits == 4:
                    O_sparse, lse_sparse = flash_attn_sparse_int4_fwd(
                        q, views["K_packed"], views["K_scale"], views["K_mn"],
                        views["V_packed"], views["V_scale"], views["V_mn"],
                        selection_mask=sel, page_size=page_size, return_lse=True)
                else:
                    O_sparse, lse_sparse = flash_attn_sparse_fwd(
                        q, views["K_uint8"], views["K_scale"], views["K_mn"],
                        views["V_uint8"], views["V_scale"], views["V_mn"],
                        selection_mask=sel, page_size=page_size, return_lse=True)
                if partial_len == 0:
                    attn_bhsd = O_sparse
                else:
                    O_partial, lse_partial = _bf16_dense_attn_with_lse(q, views["K_partial"], views["V_partial"])
                    attn_bhsd = _merge_two_attentions(O_sparse, lse_sparse, O_partial, lse_partial)
            attn_output = attn_bhsd.transpose(1, 2)

        if TRACE is not None:
            TRACE(li, q, k, v, attn_bhsd)
        attn_output = attn_output.reshape(*input_shape, -1)
        if attn_output.dtype != model_dtype:
            attn_output = attn_output.to(model_dtype)
        attn_output = self.o_proj(attn_output)
        return attn_output, None

    return forward


def patch_llama_for_quest_persistent(
    model: torch.nn.Module,
    *,
    cache,
    head_pattern: torch.Tensor,
    retention: float = 0.20,
    num_sinks: int = 4,
    window_pages: int = 2,
    page_size: int = 64,
    use_compact_kernel: bool = False,
) -> None:
    """Replace every LlamaAttention.forward with the persistent-cache version
    (reference :255-305).  head_pattern (num_layers, num_kv_heads) bool: True = retrieval head
    (keeps `retention` of the pages), False = streaming head (sinks + window only)."""
    if head_pattern.ndim != 2:
        raise ValueError(
            f"head_pattern must be 2D (num_layers, num_kv_heads); got {tuple(head_pattern.shape)}"
        )
    num_layers = head_pattern.shape[0]
    n_patched = 0
    for module in model.modules():
        if isinstance(module, LlamaAttention):
            li = module.layer_idx
            if li >= num_layers:
                raise ValueError(
                    f"head_pattern has {num_layers} layers but model layer_idx={li}"
                )
            fwd = make_quest_persistent_forward(
                cache=cache,
                head_pattern_layer=head_pattern[li].to("cuda"),
                retention=retention,
                num_sinks=num_sinks,
                window_pages=window_pages,
                page_size=page_size,
                use_compact_kernel=use_compact_kernel,
            )
            module.forward = fwd.__get__(module, type(module))
            n_patched += 1
    if n_patched == 0:
        raise RuntimeError("patch_llama_for_quest_persistent: no LlamaAttention modules")
    if n_patched != num_layers:
        raise ValueError(
            f"head_pattern has {num_layers} layers but model has {n_patched}"
        )
