"""Persistent uint8 (INT8) KV cache — CUDA counterpart of flashquest/cache/persistent_int8.py:20-190:
same constructor keywords, attributes, view keys and error behaviour."""
from __future__ import annotations

import torch
from transformers.cache_utils import Cache

from ..kernel.kv_quant import quantize_kv_int8_into


class PersistentInt8KVCache(Cache):
    kv_bits = 8

    def __init__(self, *, batch_size: int, num_layers: int, num_kv_heads: int, head_dim: int,
                 max_seq_len: int, page_size: int = 64, device="cuda", dtype=torch.bfloat16):
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
        self.K_uint8 = torch.zeros((L, B, H, S, D), dtype=torch.uint8, device=dev)
        self.V_uint8 = torch.zeros((L, B, H, S, D), dtype=torch.uint8, device=dev)
        self.K_scale = torch.zeros((L, B, H, max_pages, D), dtype=torch.bfloat16, device=dev)
        self.K_mn = torch.zeros((L, B, H, max_pages, D), dtype=torch.bfloat16, device=dev)
        self.V_scale = torch.zeros((L, B, H, S, 1), dtype=torch.bfloat16, device=dev)
        self.V_mn = torch.zeros((L, B, H, S, 1), dtype=torch.bfloat16, device=dev)
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
        """Append K_new, V_new (B,H_kv,S_new,D) to layer_idx's cache (cache/persistent_int8.py:72-141): the
        staged partial page is completed first, whole pages are quantised straight into the storage, the rest
        is staged (and the unused part of the staging buffer zeroed, as the reference does)."""
        self._check_layer(layer_idx)
        seen = self._seen_tokens[layer_idx]
        S_new = K_new.shape[2]
        if seen + S_new > self.max_seq_len:
            raise RuntimeError(f"PersistentInt8KVCache: seen+new={seen + S_new} exceeds max_seq_len={self.max_seq_len}")
        page = self.page_size
        li = layer_idx
        partial_len = seen % page
        K_stream = torch.cat([self.K_partial[li, :, :, :partial_len], K_new.to(self.dtype)], dim=2)
        V_stream = torch.cat([self.V_partial[li, :, :, :partial_len], V_new.to(self.dtype)], dim=2)
        tok0 = seen - partial_len
        total = K_stream.shape[2]
        n_pages = total // page
        complete = n_pages * page
        rest = total - complete
        if n_pages > 0:
            pg0 = tok0 // page
            quantize_kv_int8_into(
                K_stream[:, :, :complete], V_stream[:, :, :complete], page,
                K_uint8=self.K_uint8[li, :, :, tok0:tok0 + complete], K_scale=self.K_scale[li, :, :, pg0:pg0 + n_pages],
                K_mn=self.K_mn[li, :, :, pg0:pg0 + n_pages],
                V_uint8=self.V_uint8[li, :, :, tok0:tok0 + complete], V_scale=self.V_scale[li, :, :, tok0:tok0 + complete, 0],
                V_mn=self.V_mn[li, :, :, tok0:tok0 + complete, 0])
        if rest > 0:
            self.K_partial[li, :, :, :rest] = K_stream[:, :, complete:]
            self.V_partial[li, :, :, :rest] = V_stream[:, :, complete:]
        if rest < page:
            self.K_partial[li, :, :, rest:].zero_()
            self.V_partial[li, :, :, rest:].zero_()
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
            "seq_len": seen, "completed_len": completed_len, "partial_len": partial_len,
            "K_uint8": self.K_uint8[li, :, :, :completed_len, :], "V_uint8": self.V_uint8[li, :, :, :completed_len, :],
            "K_scale": self.K_scale[li, :, :, :n_pages, :], "K_mn": self.K_mn[li, :, :, :n_pages, :],
            "V_scale": self.V_scale[li, :, :, :completed_len, :], "V_mn": self.V_mn[li, :, :, :completed_len, :],
            "K_partial": self.K_partial[li, :, :, :partial_len, :], "V_partial": self.V_partial[li, :, :, :partial_len, :],
        }

    def update(self, *args, **kwargs):
        raise NotImplementedError(
            "PersistentInt8KVCache.update is not used; the patched forward calls update_quantized directly.")
