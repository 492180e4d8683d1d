"""Persistent TurboQuant K3-V3 KV cache — CUDA counterpart of
flashquest/cache/persistent_turbo.py:19-180 (same constructor keywords, attributes, view keys
and error behaviour; the append is three launches and allocates nothing)."""
from __future__ import annotations

import torch
from transformers.cache_utils import Cache

from ..kernel.kv_quant import quantize_kv_int4_into, quantize_turbo_into


class PersistentTurboKVCache(Cache):
    kv_bits = 3

    def __init__(self, *, batch_size: int, num_layers: int, num_kv_heads: int, head_dim: int,
                 max_seq_len: int, page_size: int = 64, device="cuda", dtype=torch.bfloat16):
        if head_dim % 8 != 0:
            raise ValueError(f"PersistentTurboKVCache requires head_dim multiple of 8; got {head_dim}")
        if head_dim & (head_dim - 1) != 0:
            raise ValueError(f"PersistentTurboKVCache requires head_dim power of 2 (WHT); got {head_dim}")
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
        L, B, H, D, S = num_layers, batch_size, num_kv_heads, head_dim, max_seq_len
        u8, bf = torch.uint8, torch.bfloat16
        self.K_msb = torch.zeros((L, B, H, S, D // 8), dtype=u8, device=dev)
        self.K_lsb = torch.zeros((L, B, H, S, D // 4), dtype=u8, device=dev)
        self.K_scale_turbo = torch.zeros((L, B, H, S, 1), dtype=bf, device=dev)
        self.K_scale_raw = torch.zeros((L, B, H, max_pages, D), dtype=bf, device=dev)
        self.K_mn_raw = torch.zeros((L, B, H, max_pages, D), dtype=bf, device=dev)
        self.V_msb = torch.zeros((L, B, H, S, D // 8), dtype=u8, device=dev)
        self.V_lsb = torch.zeros((L, B, H, S, D // 4), dtype=u8, device=dev)
        self.V_scale_turbo = torch.zeros((L, B, H, S, 1), dtype=bf, device=dev)
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
        (cache/persistent_turbo.py:83-147)."""
        self._check_layer(layer_idx)
        seen = self._seen_tokens[layer_idx]
        S_new = K_new.shape[2]
        if seen + S_new > self.max_seq_len:
            raise RuntimeError(
                f"PersistentTurboKVCache: seen+new={seen + S_new} exceeds max_seq_len={self.max_seq_len}")
        if S_new == 0:
            return
        if K_new.dtype != self.dtype:
            K_new = K_new.to(self.dtype)
        if V_new.dtype != self.dtype:
            V_new = V_new.to(self.dtype)
        page = self.page_size
        partial_len = seen % page
        n_quant = ((partial_len + S_new) // page) * page
        tok_start = seen - partial_len
        pg_start = tok_start // page
        li = layer_idx
        if n_quant > 0:
            quantize_turbo_into(K_new, n_quant, msb=self.K_msb[li, :, :, tok_start:], lsb=self.K_lsb[li, :, :, tok_start:],
                                scale=self.K_scale_turbo[li, :, :, tok_start:], head=self.K_partial[li], n_head=partial_len)
            quantize_turbo_into(V_new, n_quant, msb=self.V_msb[li, :, :, tok_start:], lsb=self.V_lsb[li, :, :, tok_start:],
                                scale=self.V_scale_turbo[li, :, :, tok_start:], head=self.V_partial[li], n_head=partial_len)
        # raw per-page K metadata (for scoring) + staging of the left-over tokens, after the
        # launches above have read the staged head
        quantize_kv_int4_into(
            K_new, V_new, page, n_quant,
            K_scale=self.K_scale_raw[li, :, :, pg_start:], K_mn=self.K_mn_raw[li, :, :, pg_start:],
            K_head=self.K_partial[li], V_head=self.V_partial[li], n_head=partial_len,
            stage_K=self.K_partial[li], stage_V=self.V_partial[li])
        self._seen_tokens[layer_idx] = seen + S_new

    def get_views(self, layer_idx: int) -> dict:
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
            "K_msb": self.K_msb[li, :, :, :completed_len, :],
            "K_lsb": self.K_lsb[li, :, :, :completed_len, :],
            "K_scale_turbo": self.K_scale_turbo[li, :, :, :completed_len, :],
            "K_scale_raw": self.K_scale_raw[li, :, :, :n_pages, :],
            "K_mn_raw": self.K_mn_raw[li, :, :, :n_pages, :],
            "V_msb": self.V_msb[li, :, :, :completed_len, :],
            "V_lsb": self.V_lsb[li, :, :, :completed_len, :],
            "V_scale_turbo": self.V_scale_turbo[li, :, :, :completed_len, :],
            "K_partial": self.K_partial[li, :, :, :partial_len, :],
            "V_partial": self.V_partial[li, :, :, :partial_len, :],
        }

    def update(self, *args, **kwargs):
        raise NotImplementedError(
            "PersistentTurboKVCache.update is not used; the patched forward calls update_quantized directly.")
