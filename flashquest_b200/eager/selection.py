"""Top-k page selection and compact index — CUDA counterparts of
flashquest/eager/selection.py:65-164."""
from __future__ import annotations

import torch

from .._lib import check, dtype_code, lib, ptr, require_cuda, stream_ptr


def _select(scores, retention, num_sinks, window_pages, k_max_static, want_mask, bucket, want_count=False):
    B, H, S_q, P = scores.shape
    if S_q != 1:
        raise NotImplementedError(f"select_pages_vectorized: decode-only (S_q={S_q})")
    require_cuda(scores)
    if scores.dtype != torch.float32:
        scores = scores.float()
    if scores.stride(-1) != 1:
        scores = scores.contiguous()
    r_ptr, r_scalar = None, 0.0
    if isinstance(retention, torch.Tensor):
        if retention.shape != (H,):
            raise ValueError(f"per-head retention must be shape ({H},); got {tuple(retention.shape)}")
        r_ptr = retention.to(device=scores.device, dtype=torch.float32).contiguous()
    else:
        if not (0.0 <= retention <= 1.0):
            raise ValueError(f"scalar retention must be in [0, 1]; got {retention}")
        r_scalar = float(retention)
    k_max = P if k_max_static is None else min(int(k_max_static), P)
    dev = scores.device
    mask = torch.empty(B, H, 1, P, dtype=torch.bool, device=dev) if want_mask else None
    compact = torch.empty(B, H, 1, bucket, dtype=torch.int32, device=dev) if bucket else None
    count = torch.empty(B, H, dtype=torch.int32, device=dev) if want_count else None
    with torch.cuda.device(dev):
        check(lib().fq_select_pages(
            ptr(scores), scores.stride(0), scores.stride(1), B, H, P,
            ptr(r_ptr), r_scalar, k_max, int(num_sinks), int(window_pages),
            ptr(mask), mask.stride(0) if want_mask else 0, mask.stride(1) if want_mask else 0,
            ptr(compact), compact.stride(0) if bucket else 0, compact.stride(1) if bucket else 0, int(bucket or 0),
            ptr(count), stream_ptr(dev)))
    return mask, compact, count


def select_pages_vectorized(scores, retention, num_sinks, window_pages, *, k_max_static=None):
    """Bool mask (B,H,S_q,P): top-k pages per head, plus sinks and window
    (eager/selection.py:65).  Ties between equal scores go to the lower page index."""
    mask, _, _ = _select(scores, retention, num_sinks, window_pages, k_max_static, True, 0)
    return mask


def select_pages_compact(scores, retention, num_sinks, window_pages, *, k_max_static, BUCKET_MAX,
                         return_mask=False, return_count=False):
    """select_pages_vectorized + build_compact_selection in one kernel: returns the compact
    int32 list (B,H,S_q,BUCKET_MAX) (and optionally the mask / per-row counts)."""
    if BUCKET_MAX < 1:
        raise ValueError(f"BUCKET_MAX must be >= 1, got {BUCKET_MAX}")
    mask, compact, count = _select(scores, retention, num_sinks, window_pages, k_max_static,
                                   return_mask, BUCKET_MAX, return_count)
    out = (compact,)
    if return_mask:
        out += (mask,)
    if return_count:
        out += (count,)
    return out[0] if len(out) == 1 else out


def build_compact_selection(mask: torch.Tensor, BUCKET_MAX: int, *, return_count: bool = False):
    """(B,H,S_q,P) bool -> (B,H,S_q,BUCKET_MAX) int32: selected ids descending, -1 padded
    (eager/selection.py:129).  return_count=True also returns (B,H,S_q) int32: how many entries at the
    front of each list are real (what the counted attention call wants)."""
    if BUCKET_MAX < 1:
        raise ValueError(f"BUCKET_MAX must be >= 1, got {BUCKET_MAX}")
    if mask.dtype != torch.bool:
        raise ValueError(f"mask must be bool, got {mask.dtype}")
    require_cuda(mask)
    B, H, S_q, P = mask.shape
    m = mask.contiguous().view(torch.uint8)
    out = torch.empty(B, H, S_q, BUCKET_MAX, dtype=torch.int32, device=mask.device)
    count = torch.empty(B, H, S_q, dtype=torch.int32, device=mask.device) if return_count else None
    with torch.cuda.device(mask.device):
        check(lib().fq_build_compact_counted(ptr(m), P, B * H * S_q, P, ptr(out), BUCKET_MAX, BUCKET_MAX, ptr(count),
                                             stream_ptr(mask.device)))
    return (out, count) if return_count else out


def score_select_compact(Q: torch.Tensor, K_scale: torch.Tensor, K_mn: torch.Tensor, retention, num_sinks: int,
                         window_pages: int, *, k_max_static: int, BUCKET_MAX: int, levels: int = 15,
                         first_fresh_page: int = 0):
    """page_scores_int4_fast (levels=15) / page_scores_int8_fast (levels=255) -> select_pages_vectorized ->
    build_compact_selection in ONE launch (fq_score_select), the sequence the decode branch runs
    (eager/llama_persistent_patch.py:214-228).  Q (B,H_q,1,D); K_scale, K_mn (B,H_kv,P,D) bf16;
    retention a float or a (H_q,) tensor.  Returns (scores (B,H_q,1,P) fp32, compact (B,H_q,1,BUCKET_MAX)
    int32), bit-identical to the separate calls.  first_fresh_page: see fq_score_select."""
    B, H_q, S_q, D = Q.shape
    if S_q != 1:
        raise NotImplementedError(f"score_select_compact: decode-only (S_q={S_q})")
    require_cuda(Q, K_scale, K_mn)
    H_kv, P = K_scale.shape[1], K_scale.shape[2]
    if not lib().fq_score_select_supported(H_q, H_kv, P, D):
        raise NotImplementedError("score_select_compact: shape outside the fused launch (use the separate calls)")
    Q3 = Q.reshape(B, H_q, D)
    if Q3.stride(2) != 1:
        Q3 = Q3.contiguous()
    if K_scale.stride(3) != 1 or K_scale.stride() != K_mn.stride():
        K_scale, K_mn = K_scale.contiguous(), K_mn.contiguous()
    scores = torch.empty(B, H_q, max(P, 1), dtype=torch.float32, device=Q.device)
    compact = torch.empty(B, H_q, BUCKET_MAX, dtype=torch.int32, device=Q.device)
    r_t = None
    r_f = 0.0
    if isinstance(retention, torch.Tensor):
        r_t = retention.to(device=Q.device, dtype=torch.float32).contiguous()
    else:
        r_f = float(retention)
    with torch.cuda.device(Q.device):
        check(lib().fq_score_select(
            ptr(Q3), dtype_code(Q3), Q3.stride(0), Q3.stride(1), ptr(K_scale), ptr(K_mn), *K_scale.stride()[:3],
            B, H_q, H_kv, P, D, int(levels), ptr(scores), scores.stride(0), scores.stride(1),
            ptr(r_t), r_f, min(int(k_max_static), P), int(num_sinks), int(window_pages),
            ptr(compact), compact.stride(0), compact.stride(1), int(BUCKET_MAX), None, int(first_fresh_page),
            stream_ptr(Q.device)))
    return scores[:, :, :P].unsqueeze(2), compact.unsqueeze(2)
