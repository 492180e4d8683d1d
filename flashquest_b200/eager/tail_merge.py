"""Partial-page tail attention and LSE merge — CUDA counterparts of
_bf16_dense_attn_with_lse and _merge_two_attentions
(flashquest/eager/llama_persistent_patch.py:30-61)."""
from __future__ import annotations

import torch

from .._lib import check, dtype_code, lib, ptr, require_cuda, stream_ptr
from ..kernel.sparse_int4_fwd_compact import sparse_decode_int4


def _bf16_dense_attn_with_lse(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor):
    """Dense attention of Q (B,H_q,1,D) over the staged tokens K, V (B,H_kv,t,D), fp32 softmax.
    Returns (O in Q's dtype, lse (B,H_q,1) in nats).  Runs as the tail-only case of the sparse
    decode kernel (no packed pages), so K/V are read once and nothing is repeated per GQA head."""
    B, H_q, S_q, D = Q.shape
    H_kv = K.shape[1]
    dev = Q.device
    empty_u8 = torch.empty(B, H_kv, 0, D // 2, dtype=torch.uint8, device=dev)
    empty_meta = torch.empty(B, H_kv, 0, D, dtype=torch.bfloat16, device=dev)
    empty_v = torch.empty(B, H_kv, 0, dtype=torch.bfloat16, device=dev)
    sel = torch.full((B, H_q, 1), -1, dtype=torch.int32, device=dev)
    return sparse_decode_int4(Q, empty_u8, empty_meta, empty_meta, empty_u8, empty_v, empty_v, sel,
                              page_size=16, sm_scale=None, return_lse=True, K_partial=K, V_partial=V, n_split=1)


def merge_attentions(O_parts: torch.Tensor, lse_parts: torch.Tensor):
    """n-way online-softmax merge: O_parts (n,B,H_q,1,D), lse_parts (n,B,H_q,1) ->
    (O (B,H_q,1,D) in O_parts' dtype, lse (B,H_q,1))."""
    require_cuda(O_parts, lse_parts)
    n, D = O_parts.shape[0], O_parts.shape[-1]
    Op = O_parts.contiguous()
    lp = lse_parts.float().contiguous()
    rows = Op[0].numel() // D
    O = torch.empty_like(Op[0])
    lse = torch.empty_like(lp[0])
    with torch.cuda.device(Op.device):
        check(lib().fq_lse_merge(ptr(Op), ptr(lp), dtype_code(Op), n, rows, D, ptr(O), ptr(lse), stream_ptr(Op.device)))
    return O, lse


def _merge_two_attentions(O_a, lse_a, O_b, lse_b) -> torch.Tensor:
    """Online-softmax merge of two partial attention results sharing Q
    (eager/llama_persistent_patch.py:50); result in O_a's dtype."""
    O, _ = merge_attentions(torch.stack([O_a, O_b.to(O_a.dtype)]), torch.stack([lse_a, lse_b]))
    return O
