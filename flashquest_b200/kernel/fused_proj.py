"""Fused AWQ projections — counterpart of flashquest/kernel/fused_proj.py:18-53.

The reference calls the q/k/v (or gate/up) AutoAWQ modules one after the other; here the
projections that share one input run in ONE launch, reading each module's qweight / scales /
qzeros in place: the W4A16 GEMV (`fq_awq_gemv`, CUDA cores) for decode shapes of at most 8
rows, the tensor-core dequant-GEMM (`fq_awq_gemm`, tcgen05) for prefill / batched shapes."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from .._lib import (GEMV_ADD_RMSNORM, GEMV_SWIGLU, GemvPrologue, GemvRope, check, lib, ptr, require_cuda,
                    stream_ptr)

def awq_gemv_fused(hidden: torch.Tensor, projs: Sequence, *, add: Optional[torch.Tensor] = None,
                   norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-5, return_sum: bool = False,
                   swiglu_up: Optional[torch.Tensor] = None, rope: Optional[dict] = None,
                   k_split: Optional[int] = None) -> tuple[torch.Tensor, ...]:
    """y_i = op(hidden) @ dequant(projs[i]) (+ bias) for up to 4 AWQ linears in one launch.

    hidden (..., K) fp16 with at most 8 rows in total; each proj has .qweight (K, N/8) int32,
    .scales (K/G, N) fp16, .qzeros (K/G, N/8) int32 and optionally .bias, .group_size,
    .interleaved (default: AutoAWQ's nibble order).

    op, folded into the launch (the Hugging Face modules in front of the linears):
      norm_weight given: RMSNorm(hidden + add) * norm_weight (add optional); with return_sum the sum
        hidden + add (the new residual stream) is appended to the returned tuple;
      swiglu_up given: silu(hidden) * swiglu_up (hidden = gate).
    rope: dict(mask=<bit i: rotate projection i>, theta=, head_dim=, pos=<int> or pos_dev=<int32 tensor>):
      rotary embedding (rotate_half) of those outputs at one position for all rows."""
    require_cuda(hidden)
    if hidden.dtype != torch.float16:
        raise NotImplementedError(f"AWQ GEMV computes in fp16 (AutoAWQ's dtype), got {hidden.dtype}")
    K = hidden.shape[-1]
    x = hidden.reshape(-1, K).contiguous()
    M = x.shape[0]
    n = len(projs)
    group = getattr(projs[0], "group_size", 128)
    inter = bool(getattr(projs[0], "interleaved", True))
    outs, Ns = [], []
    for pj in projs:
        qw, sc, qz = pj.qweight, pj.scales, pj.qzeros
        N = qw.shape[1] * 8
        if qw.dtype != torch.int32 or qz.dtype != torch.int32 or sc.dtype != torch.float16:
            raise ValueError("AWQ linear needs int32 qweight / qzeros and fp16 scales")
        if qw.shape[0] != K or tuple(sc.shape) != (K // group, N) or tuple(qz.shape) != (K // group, N // 8):
            raise ValueError(f"AWQ layout mismatch: qweight {tuple(qw.shape)}, scales {tuple(sc.shape)}, "
                             f"qzeros {tuple(qz.shape)} for K={K}, group={group}")
        if not (qw.is_contiguous() and sc.is_contiguous() and qz.is_contiguous()):
            raise ValueError("AWQ tensors must be contiguous")
        if getattr(pj, "group_size", group) != group or bool(getattr(pj, "interleaved", True)) != inter:
            raise ValueError("fused projections must share group size and nibble order")
        Ns.append(N)
        outs.append(torch.empty(M, N, dtype=torch.float16, device=hidden.device))
    VP = ctypes.c_void_p * n
    biases = [getattr(pj, "bias", None) for pj in projs]
    for b, N in zip(biases, Ns):
        if b is not None and (b.dtype != torch.float16 or b.numel() != N or not b.is_contiguous()):
            raise ValueError("bias must be a contiguous fp16 vector of out_features")
    bias_arr = VP(*[ptr(b) if b is not None else None for b in biases]) if any(b is not None for b in biases) else None
    pro, keep, summed = None, [], None
    if norm_weight is not None and swiglu_up is not None:
        raise ValueError("norm_weight and swiglu_up are different operators; give one")
    if norm_weight is not None:
        if norm_weight.dtype != torch.float16 or norm_weight.numel() != K:
            raise ValueError("norm_weight must be an fp16 vector of in_features")
        if add is not None:
            add = add.reshape(-1, K).to(torch.float16).contiguous()
            if add.shape[0] != M:
                raise ValueError("add must have the shape of hidden")
        if return_sum:
            summed = torch.empty_like(x)
        keep = [add, norm_weight.contiguous(), summed]
        pro = GemvPrologue(GEMV_ADD_RMSNORM, ptr(add), ptr(keep[1]), float(eps), ptr(summed))
    elif swiglu_up is not None:
        up = swiglu_up.reshape(-1, K).contiguous()
        if up.dtype != torch.float16 or up.shape[0] != M:
            raise ValueError("swiglu_up must be fp16 with the shape of hidden")
        keep = [up]
        pro = GemvPrologue(GEMV_SWIGLU, ptr(up), None, 0.0, None)
    elif add is not None or return_sum:
        raise ValueError("add / return_sum belong to the RMSNorm prologue: give norm_weight")
    rp = None
    if rope is not None:
        pos_dev = rope.get("pos_dev")
        if pos_dev is not None and (pos_dev.dtype != torch.int32 or not pos_dev.is_cuda):
            raise ValueError("rope pos_dev must be an int32 CUDA tensor")
        rp = GemvRope(int(rope["mask"]), ptr(pos_dev), int(rope.get("pos", 0)), float(rope["theta"]), int(rope["head_dim"]))
    L = lib()
    n_total = sum(Ns)
    with torch.cuda.device(hidden.device):
        ks = int(k_split) if k_split is not None else L.fq_awq_gemv_default_splits(K, n_total, group)
        check(L.fq_awq_gemv_fused(
            ptr(x), M, K, group, n,
            VP(*[ptr(pj.qweight) for pj in projs]), VP(*[ptr(pj.scales) for pj in projs]),
            VP(*[ptr(pj.qzeros) for pj in projs]), bias_arr, (ctypes.c_int * n)(*Ns), VP(*[ptr(o) for o in outs]),
            int(inter), ctypes.byref(pro) if pro is not None else None, ctypes.byref(rp) if rp is not None else None, ks,
            stream_ptr(hidden.device)))
    lead = hidden.shape[:-1]
    res = tuple(o.reshape(*lead, N) for o, N in zip(outs, Ns))
    return res + (summed.reshape(hidden.shape),) if summed is not None else res


def awq_gemm_fused(hidden: torch.Tensor, projs: Sequence) -> tuple[torch.Tensor, ...]:
    """y_i = hidden @ dequant(projs[i]) (+ bias) for up to 4 AWQ linears in one launch of the
    tensor-core dequant-GEMM, any number of rows.  Same module attributes as awq_gemv_fused;
    every out_features must be a multiple of 128."""
    require_cuda(hidden)
    if hidden.dtype != torch.float16:
        raise NotImplementedError(f"AWQ GEMM computes in fp16 (AutoAWQ's dtype), got {hidden.dtype}")
    K = hidden.shape[-1]
    x = hidden.reshape(-1, K).contiguous()
    M = x.shape[0]
    n = len(projs)
    group = getattr(projs[0], "group_size", 128)
    inter = bool(getattr(projs[0], "interleaved", True))
    outs, Ns = [], []
    for pj in projs:
        qw, sc, qz = pj.qweight, pj.scales, pj.qzeros
        N = qw.shape[1] * 8
        if qw.dtype != torch.int32 or qz.dtype != torch.int32 or sc.dtype != torch.float16:
            raise ValueError("AWQ linear needs int32 qweight / qzeros and fp16 scales")
        if qw.shape[0] != K or tuple(sc.shape) != (K // group, N) or tuple(qz.shape) != (K // group, N // 8):
            raise ValueError(f"AWQ layout mismatch: qweight {tuple(qw.shape)}, scales {tuple(sc.shape)}, "
                             f"qzeros {tuple(qz.shape)} for K={K}, group={group}")
        if not (qw.is_contiguous() and sc.is_contiguous() and qz.is_contiguous()):
            raise ValueError("AWQ tensors must be contiguous")
        if getattr(pj, "group_size", group) != group or bool(getattr(pj, "interleaved", True)) != inter:
            raise ValueError("fused projections must share group size and nibble order")
        Ns.append(N)
        outs.append(torch.empty(M, N, dtype=torch.float16, device=hidden.device))
    VP = ctypes.c_void_p * n
    biases = [getattr(pj, "bias", None) for pj in projs]
    bias_arr = VP(*[ptr(b) if b is not None else None for b in biases]) if any(b is not None for b in biases) else None
    with torch.cuda.device(hidden.device):
        if M > 0:
            check(lib().fq_awq_gemm(
                ptr(x), M, K, group, n,
                VP(*[ptr(pj.qweight) for pj in projs]), VP(*[ptr(pj.scales) for pj in projs]),
                VP(*[ptr(pj.qzeros) for pj in projs]), bias_arr, (ctypes.c_int * n)(*Ns), VP(*[ptr(o) for o in outs]),
                int(inter), stream_ptr(hidden.device)))
    lead = hidden.shape[:-1]
    return tuple(o.reshape(*lead, N) for o, N in zip(outs, Ns))


def awq_linear_fused(hidden: torch.Tensor, projs: Sequence) -> tuple[torch.Tensor, ...]:
    """The GEMV for decode shapes (at most 8 rows), the tensor-core GEMM above that."""
    rows = hidden.numel() // hidden.shape[-1]
    return awq_gemv_fused(hidden, projs) if rows <= 8 else awq_gemm_fused(hidden, projs)


def fused_qkv_proj(hidden: torch.Tensor, q_proj, k_proj, v_proj) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(Q, K, V) = hidden through the three AWQ linears, one launch."""
    q, k, v = awq_linear_fused(hidden, (q_proj, k_proj, v_proj))
    return q, k, v


def fused_gate_up_proj(hidden: torch.Tensor, gate_proj, up_proj) -> tuple[torch.Tensor, torch.Tensor]:
    """(gate, up) = hidden through the two AWQ linears, one launch; the caller applies SwiGLU."""
    gate, up = awq_linear_fused(hidden, (gate_proj, up_proj))
    return gate, up
