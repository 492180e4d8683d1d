"""Sparse decode attention over packed INT4 pages driven by a bool page mask — CUDA
counterpart of flashquest/kernel/sparse_int4_fwd.py:160-248."""
from __future__ import annotations

import torch

from ..eager.selection import build_compact_selection
from .sparse_int4_fwd_compact import check_decode_args, sparse_decode_int4


def flash_attn_sparse_int4_fwd(Q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn, *, selection_mask,
                               page_size: int = 64, sm_scale=None, return_lse: bool = True,
                               K_partial=None, V_partial=None, n_split=None):
    """Decode-only sparse forward with INT4 KV (kernel/sparse_int4_fwd.py:160).

    selection_mask (B,H_q,1,num_pages) bool, True = attend.  The mask is turned into a
    compact page list (and the number of real entries per row) by one small kernel, then the
    compact-list attention kernel walks only those entries.
    Returns (O (B,H_q,1,D) Q.dtype, lse (B,H_q,1) fp32 or None).
    """
    check_decode_args("flash_attn_sparse_int4_fwd", Q, K_packed, V_packed)
    B, H_q, _, D = Q.shape
    num_pages = K_scale.shape[2]
    assert selection_mask.shape == (B, H_q, 1, num_pages)
    assert selection_mask.dtype == torch.bool
    compact, count = build_compact_selection(selection_mask, max(num_pages, 1), return_count=True)
    return sparse_decode_int4(Q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn, compact.squeeze(2),
                              page_size=page_size, sm_scale=sm_scale, return_lse=return_lse,
                              K_partial=K_partial, V_partial=V_partial, n_split=n_split, list_count=count)
