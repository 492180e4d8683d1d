"""Fused AWQ projections — counterpart of flashquest/kernel/fused_proj.py:18-53.

The reference calls the q/k/v (or gate/up) AutoAWQ modules one after the other; here the
projections that share one input run in ONE launch, reading each module's qweight / scales /
qzeros in place: the W4A16 GEMV (`fq_awq_gemv`, CUDA cores) for decode shapes of at most 8
rows, the tensor-core dequant-GEMM (`fq_awq_gemm`, tcgen05) for prefill / batched shapes."""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from .._lib import check, lib, ptr, require_cuda, stream_ptr

_WS: dict = {}


def _workspace(device: torch.device, nbytes: int, key) -> torch.Tensor:
    """Zero-initialised split-K scratch per device; the kernel leaves its tickets at zero, so
    the buffer is cleared only when it is created, grown, or used for another shape."""
    ent = _WS.get(device)
    if ent is None or ent[0].numel() < nbytes:
        ent = [torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device), key]
        _WS[device] = ent
    elif ent[1] != key:
        ent[0][:4096].zero_()
        ent[1] = key
    return ent[0]


def awq_gemv_fused(hidden: torch.Tensor, projs: Sequence) -> tuple[torch.Tensor, ...]:
    """y_i = hidden @ dequant(projs[i]) (+ bias) for up to 4 AWQ linears in one launch.

    hidden (..., K) fp16 with at most 8 rows in total; each proj has .qweight (K, N/8) int32,
    .scales (K/G, N) fp16, .qzeros (K/G, N/8) int32 and optionally .bias, .group_size,
    .interleaved (default: AutoAWQ's nibble order)."""
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
    L = lib()
    n_total = sum(Ns)
    with torch.cuda.device(hidden.device):
        ks = L.fq_awq_gemv_default_splits(K, n_total, group)
        need = L.fq_awq_gemv_workspace_bytes(M, n_total, ks)
        ws = _workspace(hidden.device, need, (M, n_total, ks)) if need else None
        check(L.fq_awq_gemv(
            ptr(x), M, K, group, n,
            VP(*[ptr(pj.qweight) for pj in projs]), VP(*[ptr(pj.scales) for pj in projs]),
            VP(*[ptr(pj.qzeros) for pj in projs]), bias_arr, (ctypes.c_int * n)(*Ns), VP(*[ptr(o) for o in outs]),
            int(inter), ptr(ws) if ws is not None else None, ws.numel() if ws is not None else 0, ks,
            stream_ptr(hidden.device)))
    lead = hidden.shape[:-1]
    return tuple(o.reshape(*lead, N) for o, N in zip(outs, Ns))


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
