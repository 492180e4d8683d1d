"""Top-k page selection and compact index — CUDA counterparts of
flashquest/eager/selection.py:65-164."""
from __future__ import annotations

import torch

from .._lib import check, lib, ptr, require_cuda, stream_ptr


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


def build_compact_selection(mask: torch.Tensor, BUCKET_MAX: int) -> torch.Tensor:
    """(B,H,S_q,P) bool -> (B,H,S_q,BUCKET_MAX) int32: selected ids descending, -1 padded
    (eager/selection.py:129)."""
    if BUCKET_MAX < 1:
        raise ValueError(f"BUCKET_MAX must be >= 1, got {BUCKET_MAX}")
    if mask.dtype != torch.bool:
        raise ValueError(f"mask must be bool, got {mask.dtype}")
    require_cuda(mask)
    B, H, S_q, P = mask.shape
    m = mask.contiguous().view(torch.uint8)
    out = torch.empty(B, H, S_q, BUCKET_MAX, dtype=torch.int32, device=mask.device)
    with torch.cuda.device(mask.device):
        check(lib().fq_build_compact(ptr(m), P, B * H * S_q, P, ptr(out), BUCKET_MAX, BUCKET_MAX,
                                     stream_ptr(mask.device)))
    return out
