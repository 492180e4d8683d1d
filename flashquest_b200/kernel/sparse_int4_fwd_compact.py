"""Sparse decode attention over packed INT4 pages, compact-list variant — CUDA counterpart
of flashquest/kernel/sparse_int4_fwd_compact.py:153-244."""
from __future__ import annotations

import math

import torch

from .._lib import check, dtype_code, lib, ptr, require_cuda, stream_ptr

_SUPPORTED_HEAD_DIMS = (64, 128)
_workspaces: dict = {}


def _workspace(device, nbytes: int, rows: int):
    """Split-K scratch, one per (device, stream).  The kernel expects the ticket words at its
    start (one per (batch, head) row) to be zero before a call and leaves them zero after it;
    that only holds while the row count stays the same, because the partial results of a
    call with fewer rows land where a call with more rows keeps its tickets.  So the ticket
    region is cleared whenever the row count changes."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    ws, last_rows = _workspaces.get(key, (None, -1))
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        last_rows = rows
    if last_rows != rows:
        ws[: (rows * 4 + 255) // 256 * 256].zero_()
    _workspaces[key] = (ws, rows)
    return ws


def reset_workspaces():
    """Zeroes every cached scratch buffer.  To be called after fq_device_status() has reported a
    timed-out wait: a kernel that gave up leaves its ticket words non-zero."""
    for ws, _ in _workspaces.values():
        ws.zero_()


def _vmeta(t: torch.Tensor, B, H, S):
    """V_scale / V_mn as (B,H,S) with unit token stride and 16-byte aligned (b,h) rows; the
    reference passes (B,H,S,1) from the caches and (B,H,S) from some tests."""
    if t.dim() == 4:
        t = t.squeeze(-1)
    if t.dtype != torch.bfloat16:
        raise TypeError("V_scale / V_mn must be bfloat16")
    ok = (S <= 1 or t.stride(2) == 1) and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0
    if ok:
        return t
    S8 = (S + 7) // 8 * 8
    buf = torch.zeros(B, H, S8, dtype=torch.bfloat16, device=t.device)
    buf[:, :, :S] = t
    return buf


def _kmeta(t: torch.Tensor):
    if t.dtype != torch.bfloat16:
        raise TypeError("K_scale / K_mn must be bfloat16")
    ok = t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


def _packed(t: torch.Tensor, Dp):
    ok = (t.stride(3) == 1 and t.stride(2) == Dp and t.stride(0) % 16 == 0 and t.stride(1) % 16 == 0
          and t.data_ptr() % 16 == 0)
    return t if ok else t.contiguous()


def sparse_decode_int4(Q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn, sel_3d, *, page_size, sm_scale,
                       return_lse, K_partial=None, V_partial=None, n_split=None, list_count=None):
    """Shared launcher: sel_3d is (B,H_q,bucket) int32 with -1 sentinels; list_count (B*H_q int32, contiguous)
    bounds the entries walked per row when the real ones sit at the front."""
    B, H_q, S_q, D = Q.shape
    Bk, H_kv, S_kv, Dp = K_packed.shape
    P = K_scale.shape[2]
    dev = Q.device
    require_cuda(Q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn, sel_3d)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    Q_2d = Q.squeeze(2)
    if Q_2d.stride(-1) != 1 or Q_2d.stride(0) % 8 or Q_2d.stride(1) % 8 or Q_2d.data_ptr() % 16:
        Q_2d = Q_2d.contiguous()
    O_2d = torch.empty(B, H_q, D, dtype=Q.dtype, device=dev)
    L = torch.empty(B, H_q, dtype=torch.float32, device=dev) if return_lse else None
    K_packed, V_packed = _packed(K_packed, Dp), _packed(V_packed, Dp)
    K_scale, K_mn = _kmeta(K_scale), _kmeta(K_mn)
    if K_scale.stride() != K_mn.stride():
        K_scale, K_mn = K_scale.contiguous(), K_mn.contiguous()
    V_scale, V_mn = _vmeta(V_scale, B, H_kv, S_kv), _vmeta(V_mn, B, H_kv, S_kv)
    if V_scale.stride() != V_mn.stride():
        S8 = (S_kv + 7) // 8 * 8
        both = torch.zeros(2, B, H_kv, S8, dtype=torch.bfloat16, device=dev)
        both[0, :, :, :S_kv], both[1, :, :, :S_kv] = V_scale, V_mn
        V_scale, V_mn = both[0], both[1]
    sel = sel_3d if sel_3d.stride(-1) == 1 else sel_3d.contiguous()
    bucket = sel.shape[-1]
    tail_len = 0
    tail_code = 2
    tl = (0, 0, 0)
    if K_partial is not None and K_partial.shape[2] > 0:
        require_cuda(K_partial, V_partial)
        if K_partial.dtype != V_partial.dtype or K_partial.dtype not in (torch.float16, torch.bfloat16):
            raise TypeError("K_partial / V_partial must both be fp16 or bf16")
        if K_partial.stride(3) != 1 or K_partial.stride() != V_partial.stride():
            K_partial, V_partial = K_partial.contiguous(), V_partial.contiguous()
        tail_len = K_partial.shape[2]
        tail_code = dtype_code(K_partial)
        tl = (K_partial.stride(0), K_partial.stride(1), K_partial.stride(2))
    else:
        K_partial = V_partial = None
    with torch.cuda.device(dev):
        if n_split is None:
            n_split = lib().fq_sparse_decode_default_splits(B, H_q, bucket, int(page_size))
        ws = None
        ws_bytes = 0
        if n_split > 1:
            ws_bytes = lib().fq_sparse_decode_workspace_bytes(B, H_q, D, n_split)
            ws = _workspace(dev, ws_bytes, B * H_q)
        if list_count is not None:
            require_cuda(list_count)
            assert list_count.dtype == torch.int32 and list_count.numel() == B * H_q and list_count.is_contiguous()
        check(lib().fq_sparse_decode_int4_counted(
            ptr(Q_2d), dtype_code(Q_2d), Q_2d.stride(0), Q_2d.stride(1),
            ptr(K_packed), K_packed.stride(0), K_packed.stride(1),
            ptr(K_scale), ptr(K_mn), K_scale.stride(0), K_scale.stride(1), K_scale.stride(2),
            ptr(V_packed), V_packed.stride(0), V_packed.stride(1),
            ptr(V_scale), ptr(V_mn), V_scale.stride(0), V_scale.stride(1),
            ptr(sel), sel.stride(0), sel.stride(1), bucket, ptr(list_count),
            ptr(K_partial), ptr(V_partial), tail_code, *tl, tail_len,
            B, H_q, H_kv, S_kv, P, D, int(page_size), float(sm_scale),
            ptr(O_2d), O_2d.stride(0), O_2d.stride(1), ptr(L),
            ptr(ws), ws.numel() if ws is not None else 0, int(n_split), stream_ptr(dev)))
    O = O_2d.unsqueeze(2)
    return O, (L.unsqueeze(2) if L is not None else None)


def check_decode_args(name, Q, K_packed, V_packed):
    if not Q.is_cuda or Q.dtype not in (torch.bfloat16, torch.float16):
        raise AssertionError(f"{name}: Q must be a CUDA bf16 (or fp16) tensor")
    if K_packed.dtype != torch.uint8 or V_packed.dtype != torch.uint8:
        raise AssertionError(f"{name}: K_packed / V_packed must be uint8")
    B, H_q, S_q, D = Q.shape
    if S_q != 1:
        raise NotImplementedError(f"{name}: decode-only (S_q={S_q})")
    if D not in _SUPPORTED_HEAD_DIMS:
        raise NotImplementedError(f"head_dim={D} not in {_SUPPORTED_HEAD_DIMS}")
    Bk, H_kv, S_kv, Dp = K_packed.shape
    assert B == Bk
    assert Dp == D // 2, f"K_packed last axis {Dp} != D/2={D // 2}"
    assert H_q % H_kv == 0


def flash_attn_sparse_int4_fwd_compact(Q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn, *,
                                       selected_page_ids, page_size: int = 64, sm_scale=None,
                                       return_lse: bool = True, K_partial=None, V_partial=None, n_split=None):
    """Decode-only sparse forward with INT4 KV over a compact page list
    (kernel/sparse_int4_fwd_compact.py:153).

    Q (B,H_q,1,D) bf16 (fp16 also accepted); K_packed/V_packed (B,H_kv,S_kv,D/2) uint8;
    K_scale/K_mn (B,H_kv,P,D) bf16; V_scale/V_mn (B,H_kv,S_kv[,1]) bf16;
    selected_page_ids (B,H_q,[1,]BUCKET_MAX) int32 with -1 sentinels.
    Extension over the reference: K_partial/V_partial (B,H_kv,t,D) adds the staged tail
    tokens to the same softmax (what _bf16_dense_attn_with_lse + _merge_two_attentions do,
    eager/llama_persistent_patch.py:30-61).
    Returns (O (B,H_q,1,D) Q.dtype, lse (B,H_q,1) fp32 nats or None).
    """
    check_decode_args("compact INT4", Q, K_packed, V_packed)
    assert selected_page_ids.dtype == torch.int32
    if selected_page_ids.dim() == 4:
        sel_3d = selected_page_ids.squeeze(2)
    elif selected_page_ids.dim() == 3:
        sel_3d = selected_page_ids
    else:
        raise ValueError(f"selected_page_ids must be 3D or 4D; got {selected_page_ids.dim()}D")
    assert sel_3d.shape[0] == Q.shape[0] and sel_3d.shape[1] == Q.shape[1]
    return sparse_decode_int4(Q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn, sel_3d,
                              page_size=page_size, sm_scale=sm_scale, return_lse=return_lse,
                              K_partial=K_partial, V_partial=V_partial, n_split=n_split)
