"""Sparse decode attention over uint8 (INT8) KV pages driven by a bool page mask — CUDA counterpart
of flashquest/kernel/sparse_fwd.py:140-228."""
from __future__ import annotations

import math

import torch

from .._lib import check, dtype_code, inner_contiguous, lib, ptr, require_cuda, stream_ptr
from ..eager.selection import build_compact_selection

_SUPPORTED_HEAD_DIMS = (64, 128)


def flash_attn_sparse_fwd(Q, K_uint8, K_scale, K_mn, V_uint8, V_scale, V_mn, *, selection_mask, page_size: int = 64,
                          sm_scale=None, return_lse: bool = True, K_partial=None, V_partial=None, n_split=None):
    """Decode-only sparse forward with INT8 KV (kernel/sparse_fwd.py:140).

    Q (B,H_q,1,D) bf16 (fp16 accepted); K_uint8, V_uint8 (B,H_kv,S_kv,D) uint8; K_scale, K_mn
    (B,H_kv,num_pages,D) bf16; V_scale, V_mn (B,H_kv,S_kv,1) bf16; selection_mask (B,H_q,1,num_pages)
    bool, True = attend.  Extension: K_partial / V_partial (B,H_kv,t,D) are attended in the same softmax.
    Returns (O (B,H_q,1,D) Q.dtype, lse (B,H_q,1) fp32 or None)."""
    assert Q.is_cuda and Q.dtype in (torch.bfloat16, torch.float16)
    assert K_uint8.dtype == torch.uint8 and V_uint8.dtype == torch.uint8
    B, H_q, S_q, D = Q.shape
    if S_q != 1:
        raise NotImplementedError(f"flash_attn_sparse_fwd: Phase 3 v1 is decode-only (S_q={S_q}); use flash_attn_fwd for prefill.")
    if D not in _SUPPORTED_HEAD_DIMS:
        raise NotImplementedError(f"head_dim={D} not in {_SUPPORTED_HEAD_DIMS}")
    Bk, H_kv, S_kv, Dk = K_uint8.shape
    assert (B, D) == (Bk, Dk)
    assert H_q % H_kv == 0
    num_pages = K_scale.shape[2]
    assert selection_mask.shape == (B, H_q, 1, num_pages)
    assert selection_mask.dtype == torch.bool
    require_cuda(K_uint8, V_uint8, K_scale, K_mn, V_scale, V_mn, selection_mask)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    dev = Q.device
    compact, count = build_compact_selection(selection_mask, max(num_pages, 1), return_count=True)
    compact = compact.squeeze(2)
    bucket = compact.shape[-1]
    Q3 = Q.reshape(B, H_q, D).contiguous()
    K_uint8, V_uint8 = inner_contiguous(K_uint8), inner_contiguous(V_uint8)
    if K_uint8.stride() != V_uint8.stride():
        K_uint8, V_uint8 = K_uint8.contiguous(), V_uint8.contiguous()
    K_scale, K_mn = inner_contiguous(K_scale), inner_contiguous(K_mn)
    if K_scale.stride() != K_mn.stride():
        K_scale, K_mn = K_scale.contiguous(), K_mn.contiguous()
    Vs = V_scale.squeeze(-1) if V_scale.dim() == 4 else V_scale
    Vm = V_mn.squeeze(-1) if V_mn.dim() == 4 else V_mn
    if (S_kv > 1 and (Vs.stride(2) != 1 or Vm.stride(2) != 1)) or Vs.stride() != Vm.stride():
        Vs, Vm = Vs.contiguous(), Vm.contiguous()
    tail_len, tl, tcode = 0, (0, 0, 0), 2
    if K_partial is not None and K_partial.shape[2] > 0:
        if K_partial.stride(3) != 1 or K_partial.stride() != V_partial.stride():
            K_partial, V_partial = K_partial.contiguous(), V_partial.contiguous()
        tail_len, tl, tcode = K_partial.shape[2], K_partial.stride()[:3], dtype_code(K_partial)
    else:
        K_partial = V_partial = None
    O = torch.empty(B, H_q, D, dtype=Q.dtype, device=dev)
    L = torch.empty(B, H_q, dtype=torch.float32, device=dev) if return_lse else None
    if n_split is None:
        # a warp should walk at least six to eight pages (the list made from a mask is as wide as the page count and
        # about a quarter of it is real: one split per 96 entries at most), and about sixteen 128-thread CTAs per SM
        # are enough to fill the GPU (measured at 2048 pages: 16-24 splits best at batch 1, 4-8 at batch 16)
        n_split = max(1, min(64, bucket // 96, max(1, (16 * 148) // max(B * H_q, 1))))
    with torch.cuda.device(dev):
        ws = torch.empty(lib().fq_sparse_decode_int8_workspace_bytes(B, H_q, D, n_split), dtype=torch.uint8, device=dev)
        check(lib().fq_sparse_decode_int8_counted(
            ptr(Q3), dtype_code(Q3), Q3.stride(0), Q3.stride(1),
            ptr(K_uint8), ptr(V_uint8), *K_uint8.stride()[:3],
            ptr(K_scale), ptr(K_mn), *K_scale.stride()[:3], ptr(Vs), ptr(Vm), Vs.stride(0), Vs.stride(1),
            ptr(compact), compact.stride(0), compact.stride(1), bucket, ptr(count),
            ptr(K_partial), ptr(V_partial), tcode, *tl, tail_len,
            B, H_q, H_kv, S_kv, num_pages, D, int(page_size), float(sm_scale),
            ptr(O), ptr(L), ptr(ws), ws.numel(), int(n_split), stream_ptr(dev)))
    return O.unsqueeze(2), (L.unsqueeze(2) if L is not None else None)
