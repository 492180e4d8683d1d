"""Quest page criticality from the quantised K metadata — CUDA counterparts of
flashquest/eager/criticality.py:128-163 (INT4, 15 levels) and :77-125 (INT8, 255 levels)."""
from __future__ import annotations

import torch

from .._lib import check, dtype_code, inner_contiguous, lib, ptr, require_cuda, stream_ptr


def page_scores_int4_fast(Q: torch.Tensor, K_scale: torch.Tensor, K_mn: torch.Tensor) -> torch.Tensor:
    """score = Q.K_mn + 15 * relu(Q).K_scale per page (eager/criticality.py:128).

    Q (B,H_q,S_q,D) bf16/fp16/fp32; K_scale, K_mn (B,H_kv,P,D) bf16 (views are fine).
    Returns (B,H_q,S_q,P) fp32.  One kernel, one pass over the metadata.
    """
    return _page_scores(Q, K_scale, K_mn, "page_scores_int4_fast", lib().fq_page_scores_int4)


def page_scores_int8_fast(Q: torch.Tensor, K_scale: torch.Tensor, K_mn: torch.Tensor) -> torch.Tensor:
    """score = Q.K_mn + 255 * relu(Q).K_scale per page (eager/criticality.py:77): the INT8 cache's metadata."""
    return _page_scores(Q, K_scale, K_mn, "page_scores_int8_fast", lib().fq_page_scores_int8)


def _page_scores(Q, K_scale, K_mn, name, entry):
    B, H_q, S_q, D = Q.shape
    H_kv, P = K_scale.shape[1], K_scale.shape[2]
    if H_q % H_kv != 0:
        raise ValueError(f"H_q={H_q} must be divisible by H_kv={H_kv}")
    if S_q != 1:
        raise NotImplementedError(f"{name}: decode-only (S_q={S_q})")
    require_cuda(Q, K_scale, K_mn)
    if K_scale.dtype != torch.bfloat16 or K_mn.dtype != torch.bfloat16:
        raise TypeError("K_scale / K_mn must be bfloat16")
    Q = inner_contiguous(Q)
    K_scale, K_mn = inner_contiguous(K_scale), inner_contiguous(K_mn)
    if K_scale.stride() != K_mn.stride():
        K_scale, K_mn = K_scale.contiguous(), K_mn.contiguous()
    scores = torch.empty(B, H_q, 1, P, dtype=torch.float32, device=Q.device)
    with torch.cuda.device(Q.device):
        check(entry(
            ptr(Q), dtype_code(Q), Q.stride(0), Q.stride(1),
            ptr(K_scale), ptr(K_mn), K_scale.stride(0), K_scale.stride(1), K_scale.stride(2),
            B, H_q, H_kv, P, D, ptr(scores), scores.stride(0), scores.stride(1), stream_ptr(Q.device)))
    return scores
