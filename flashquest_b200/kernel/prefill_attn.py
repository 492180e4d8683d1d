"""Dense causal attention of the prefill branch — CUDA counterpart of the
scaled_dot_product_attention(q, K_full, V_full, is_causal=True, enable_gqa=True) call in
flashquest/eager/llama_persistent_patch.py:196-201."""
from __future__ import annotations

import math

import torch

from .._lib import check, dtype_code, lib, ptr, require_cuda, stream_ptr


def _rows16(t: torch.Tensor) -> torch.Tensor:
    ok = t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


def prefill_causal_attention(q: torch.Tensor, K_full: torch.Tensor, V_full: torch.Tensor, sm_scale=None,
                             out_bshd: bool = False) -> torch.Tensor:
    """q (B,H_q,S_q,D), K_full / V_full (B,H_kv,S_kv,D), all fp16 or all bf16 -> (B,H_q,S_q,D)
    in q's dtype; query i attends keys 0..i (torch's top-left causal alignment), grouped-query
    heads.  With out_bshd the result is laid out (B,S_q,H_q,D) (what the patched forward
    reshapes to before o_proj) and returned as that tensor."""
    require_cuda(q, K_full, V_full)
    if q.dtype not in (torch.float16, torch.bfloat16) or K_full.dtype != q.dtype or V_full.dtype != q.dtype:
        raise TypeError("prefill_causal_attention: q, K, V must share one dtype, fp16 or bf16")
    B, Hq, Sq, D = q.shape
    Hkv, Skv = K_full.shape[1], K_full.shape[2]
    if D not in (64, 128):
        raise NotImplementedError(f"head_dim={D} not in (64, 128)")
    if Hq % Hkv != 0:
        raise ValueError(f"H_q={Hq} must be divisible by H_kv={Hkv}")
    q, K_full, V_full = _rows16(q), _rows16(K_full), _rows16(V_full)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    if out_bshd:
        out = torch.empty(B, Sq, Hq, D, dtype=q.dtype, device=q.device)
        o_strides = (out.stride(0), out.stride(2), out.stride(1))
    else:
        out = torch.empty(B, Hq, Sq, D, dtype=q.dtype, device=q.device)
        o_strides = out.stride()[:3]
    with torch.cuda.device(q.device):
        check(lib().fq_prefill_attention(
            ptr(q), *q.stride()[:3], ptr(K_full), *K_full.stride()[:3], ptr(V_full), *V_full.stride()[:3],
            dtype_code(q), B, Hq, Hkv, Sq, Skv, D, float(sm_scale), ptr(out), *o_strides, stream_ptr(q.device)))
    return out
