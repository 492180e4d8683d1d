"""Sparse decode attention over TurboQuant K3-V3 KV — CUDA counterpart of
flashquest/kernel/sparse_turbo_fwd.py:254-346."""
from __future__ import annotations

import math

import torch

from .._lib import check, dtype_code, inner_contiguous, lib, ptr, require_cuda, stream_ptr
from ..eager.selection import build_compact_selection
from .sparse_int4_fwd_compact import _workspace
from .wht import wht_along_head_dim

_SUPPORTED_HEAD_DIMS = (64, 128)


def _scale3(t, B, H, S):
    if t.dim() == 4:
        t = t.squeeze(-1)
    if t.dtype != torch.bfloat16:
        raise TypeError("K_scale_turbo / V_scale_turbo must be bfloat16")
    return t if S <= 1 or t.stride(2) == 1 else t.contiguous()


def sparse_decode_turbo_rotated(Q_rot, K_msb, K_lsb, K_scale_turbo, V_msb, V_lsb, V_scale_turbo, *,
                                selection_mask, page_size: int = 64, sm_scale=None, return_lse: bool = True,
                                n_split=None):
    """The kernel of flash_attn_sparse_turbo_fwd alone, in the ROTATED basis: Q_rot (B,H_q,1,D) is
    taken as it is (no WHT before), O_rot comes back un-rotated-back (no WHT after).  This is the part
    of kernel/sparse_turbo_fwd.py:92-251 that runs on the GPU in the reference; parity of the
    arithmetic is checked here, the two bf16 rotations are checked by the WHT tests."""
    assert Q_rot.is_cuda and Q_rot.dtype in (torch.bfloat16, torch.float16)
    assert K_msb.dtype == torch.uint8 and K_lsb.dtype == torch.uint8
    assert V_msb.dtype == torch.uint8 and V_lsb.dtype == torch.uint8
    B, H_q, S_q, D = Q_rot.shape
    if S_q != 1:
        raise NotImplementedError(f"flash_attn_sparse_turbo_fwd: decode-only (S_q={S_q})")
    if D not in _SUPPORTED_HEAD_DIMS:
        raise NotImplementedError(f"head_dim={D} not in {_SUPPORTED_HEAD_DIMS}")
    Bk, H_kv, S_kv, _ = K_msb.shape
    assert B == Bk
    assert H_q % H_kv == 0
    num_pages = selection_mask.shape[-1]
    assert selection_mask.shape == (B, H_q, 1, num_pages)
    assert selection_mask.dtype == torch.bool
    require_cuda(K_msb, K_lsb, V_msb, V_lsb, K_scale_turbo, V_scale_turbo, selection_mask)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    dev = Q_rot.device
    Q_rot = Q_rot.reshape(B, H_q, D)
    if Q_rot.stride(-1) != 1 or Q_rot.stride(0) % 8 or Q_rot.stride(1) % 8 or Q_rot.data_ptr() % 16:
        Q_rot = Q_rot.contiguous()
    O_rot = torch.empty(B, H_q, D, dtype=Q_rot.dtype, device=dev)
    L = torch.empty(B, H_q, dtype=torch.float32, device=dev) if return_lse else None
    compact = build_compact_selection(selection_mask, max(num_pages, 1)).squeeze(2)
    bucket = compact.shape[-1]
    K_msb, K_lsb, V_msb, V_lsb = (inner_contiguous(t) for t in (K_msb, K_lsb, V_msb, V_lsb))
    ks, vs = _scale3(K_scale_turbo, B, H_kv, S_kv), _scale3(V_scale_turbo, B, H_kv, S_kv)
    with torch.cuda.device(dev):
        if n_split is None:
            n_split = max(1, min(lib().fq_sparse_decode_default_splits(B, H_q, bucket, int(page_size)), 64))
        ws, ws_bytes = None, 0
        if n_split > 1:
            ws_bytes = lib().fq_sparse_decode_workspace_bytes(B, H_q, D, n_split)
            ws = _workspace(dev, ws_bytes, B * H_q)
        check(lib().fq_sparse_decode_turbo(
            ptr(Q_rot), dtype_code(Q_rot), Q_rot.stride(0), Q_rot.stride(1),
            ptr(K_msb), *K_msb.stride()[:3], ptr(K_lsb), *K_lsb.stride()[:3], ptr(ks), ks.stride(0), ks.stride(1),
            ptr(V_msb), *V_msb.stride()[:3], ptr(V_lsb), *V_lsb.stride()[:3], ptr(vs), vs.stride(0), vs.stride(1),
            ptr(compact), compact.stride(0), compact.stride(1), bucket,
            B, H_q, H_kv, S_kv, num_pages, D, int(page_size), float(sm_scale),
            ptr(O_rot), O_rot.stride(0), O_rot.stride(1), ptr(L),
            ptr(ws), ws.numel() if ws is not None else 0, int(n_split), stream_ptr(dev)))
    return O_rot.unsqueeze(2), (L.unsqueeze(2) if L is not None else None)


def flash_attn_sparse_turbo_fwd(Q, K_msb, K_lsb, K_scale_turbo, V_msb, V_lsb, V_scale_turbo, *,
                                selection_mask, page_size: int = 64, sm_scale=None, return_lse: bool = True,
                                n_split=None):
    """Decode-only fused TurboQuant sparse forward (K3-V3), kernel/sparse_turbo_fwd.py:254.

    Q (B,H_q,1,D) bf16 (fp16 accepted) in the RAW basis: it is rotated with the WHT before the
    kernel and the output is rotated back after it, as the reference wrapper does
    (kernel/sparse_turbo_fwd.py:305,343-344).
    Returns (O (B,H_q,1,D) Q.dtype, lse (B,H_q,1) fp32 or None), both in the raw basis."""
    assert Q.is_cuda and Q.dtype in (torch.bfloat16, torch.float16)
    if Q.dim() == 4 and Q.shape[2] != 1:
        raise NotImplementedError(f"flash_attn_sparse_turbo_fwd: decode-only (S_q={Q.shape[2]})")
    if Q.shape[-1] not in _SUPPORTED_HEAD_DIMS:
        raise NotImplementedError(f"head_dim={Q.shape[-1]} not in {_SUPPORTED_HEAD_DIMS}")
    O_rot, L = sparse_decode_turbo_rotated(wht_along_head_dim(Q), K_msb, K_lsb, K_scale_turbo, V_msb, V_lsb, V_scale_turbo,
                                           selection_mask=selection_mask, page_size=page_size, sm_scale=sm_scale,
                                           return_lse=return_lse, n_split=n_split)
    return wht_along_head_dim(O_rot), L
