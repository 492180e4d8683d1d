"""Persistent packed-INT4 KV cache — CUDA counterpart of
flashquest/cache/persistent_int4.py:14-166.

Same constructor keywords, attributes, view keys and error behaviour.  Differences that do
not change results: the append is ONE kernel launch (stage + quantise completed pages,
written straight into the preallocated storage, no temporaries), and the staging dtype is a
constructor argument (default bf16 as in the reference).
"""
from __future__ import annotations

import torch
from transformers.cache_utils import Cache

from ..kernel.kv_quant import quantize_kv_int4_into


class PersistentInt4KVCache(Cache):
    kv_bits = 4

    def __init__(self, *, batch_size: int, num_layers: int, num_kv_heads: int, head_dim: int,
                 max_seq_len: int, page_size: int = 64, device="cuda", dtype=torch.bfloat16):
        if head_dim % 2 != 0:
            raise ValueError(f"PersistentInt4KVCache requires even head_dim (2 INT4 per byte); got {head_dim}")
        self.layers: list = []
        self.layer_class_to_replicate = None
        self.offloading = False
        self.batch_size = batch_size
        self.num_layers = num_layers
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.max_seq_len = max_seq_len
        self.page_size = page_size
        self.dtype = dtype
        max_pages = (max_seq_len + page_size - 1) // page_size
        self.max_pages = max_pages
        dev = torch.device(device)
        L, B, H, D = num_layers, batch_size, num_kv_heads, head_dim
        # token axis padded to a multiple of 8 so every (b,h) row of the bf16 V metadata starts
        # on a 16-byte boundary (needed by the attention kernel's bulk copies)
        s_alloc = (max_seq_len + 7) // 8 * 8
        self.K_packed = torch.zeros((L, B, H, s_alloc, D // 2), dtype=torch.uint8, device=dev)[:, :, :, :max_seq_len]
        self.V_packed = torch.zeros((L, B, H, s_alloc, D // 2), dtype=torch.uint8, device=dev)[:, :, :, :max_seq_len]
        self.K_scale = torch.zeros((L, B, H, max_pages, D), dtype=torch.bfloat16, device=dev)
        self.K_mn = torch.zeros((L, B, H, max_pages, D), dtype=torch.bfloat16, device=dev)
        self.V_scale = torch.zeros((L, B, H, s_alloc, 1), dtype=torch.bfloat16, device=dev)[:, :, :, :max_seq_len]
        self.V_mn = torch.zeros((L, B, H, s_alloc, 1), dtype=torch.bfloat16, device=dev)[:, :, :, :max_seq_len]
        self.K_partial = torch.zeros((L, B, H, page_size, D), dtype=dtype, device=dev)
        self.V_partial = torch.zeros((L, B, H, page_size, D), dtype=dtype, device=dev)
        self._seen_tokens = [0] * num_layers

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seen_tokens[layer_idx]

    def get_max_length(self) -> int:
        return self.max_seq_len

    def _check_layer(self, layer_idx: int) -> None:
        if layer_idx < 0 or layer_idx >= self.num_layers:
            raise IndexError(f"layer_idx {layer_idx} out of range [0, {self.num_layers})")

    def update_quantized(self, K_new: torch.Tensor, V_new: torch.Tensor, layer_idx: int) -> None:
        """Append K_new, V_new (B,H_kv,S_new,D) to layer_idx's cache
        (cache/persistent_int4.py:69-132): completed pages are quantised, the rest staged."""
        self._check_layer(layer_idx)
        seen = self._seen_tokens[layer_idx]
        S_new = K_new.shape[2]
        if seen + S_new > self.max_seq_len:
            raise RuntimeError(
                f"PersistentInt4KVCache: seen+new={seen + S_new} exceeds max_seq_len={self.max_seq_len}")
        if S_new == 0:
            return
        if K_new.dtype != self.dtype:
            K_new = K_new.to(self.dtype)
        if V_new.dtype != self.dtype:
            V_new = V_new.to(self.dtype)
        page = self.page_size
        partial_len = seen % page
        total = partial_len + S_new
        n_quant = (total // page) * page
        tok_start = seen - partial_len
        pg_start = tok_start // page
        li = layer_idx
        quantize_kv_int4_into(
            K_new, V_new, page, n_quant,
            K_packed=self.K_packed[li, :, :, tok_start:], K_scale=self.K_scale[li, :, :, pg_start:],
            K_mn=self.K_mn[li, :, :, pg_start:],
            V_packed=self.V_packed[li, :, :, tok_start:], V_scale=self.V_scale[li, :, :, tok_start:],
            V_mn=self.V_mn[li, :, :, tok_start:],
            K_head=self.K_partial[li], V_head=self.V_partial[li], n_head=partial_len,
            stage_K=self.K_partial[li], stage_V=self.V_partial[li])
        self._seen_tokens[layer_idx] = seen + S_new

    def get_views(self, layer_idx: int) -> dict:
        """Slices of the storage, same keys as the reference (cache/persistent_int4.py:134-159)."""
        self._check_layer(layer_idx)
        seen = self._seen_tokens[layer_idx]
        page = self.page_size
        partial_len = seen % page
        completed_len = seen - partial_len
        n_pages = completed_len // page
        li = layer_idx
        return {
            "seq_len": seen,
            "completed_len": completed_len,
            "partial_len": partial_len,
            "K_packed": self.K_packed[li, :, :, :completed_len, :],
            "V_packed": self.V_packed[li, :, :, :completed_len, :],
            "K_scale": self.K_scale[li, :, :, :n_pages, :],
            "K_mn": self.K_mn[li, :, :, :n_pages, :],
            "V_scale": self.V_scale[li, :, :, :completed_len, :],
            "V_mn": self.V_mn[li, :, :, :completed_len, :],
            "K_partial": self.K_partial[li, :, :, :partial_len, :],
            "V_partial": self.V_partial[li, :, :, :partial_len, :],
        }

    def update(self, *args, **kwargs):
        raise NotImplementedError(
            "PersistentInt4KVCache.update is not used; the patched forward calls update_quantized directly.")
