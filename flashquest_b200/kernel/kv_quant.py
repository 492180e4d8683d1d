"""INT4 KV quantisation primitives — CUDA counterparts of flashquest/kernel/kv_quant.py.

Same names, argument order, return tuples and error messages as the reference functions
(kernel/kv_quant.py:152-215); results are bit-identical to the reference's CPU path.
"""
from __future__ import annotations

import torch

from .. import _lib
from .._lib import check, dtype_code, inner_contiguous, lib, ptr, require_cuda, stream_ptr


def _strides3(t):
    """(b, h, row) element strides of a (B, H, rows, inner) or (B, H, rows) tensor."""
    return t.stride(0), t.stride(1), t.stride(2)


def quantize_kv_int4_into(K_new, V_new, page_size, n_quant, *, K_packed=None, K_scale=None, K_mn=None,
                          V_packed=None, V_scale=None, V_mn=None, K_head=None, V_head=None, n_head=0,
                          stage_K=None, stage_V=None):
    """One launch of fq_quantize_kv_int4: quantise the first n_quant tokens of the stream
    head[:n_head] ++ new, writing into the given (possibly strided) output views, and copy
    the left-over tokens into the staging views.  This is the page-flush step of
    PersistentInt4KVCache.update_quantized (cache/persistent_int4.py:94-130) as one kernel."""
    ref = K_new if K_new is not None else V_new
    require_cuda(ref)
    B, H, n_new, D = ref.shape
    if D % 2 != 0:
        raise ValueError(f"quantize_k_int4 requires even head_dim; got {D}")
    K_new = inner_contiguous(K_new) if K_new is not None else None
    V_new = inner_contiguous(V_new) if V_new is not None else None
    src = K_new if K_new is not None else V_new
    if K_new is not None and V_new is not None and _strides3(K_new) != _strides3(V_new):
        V_new = V_new.contiguous()
        K_new = K_new.contiguous()
        src = K_new
    hd = K_head if K_head is not None else V_head
    pk = K_packed if K_packed is not None else V_packed
    st = stage_K if stage_K is not None else stage_V
    z3 = (0, 0, 0)
    hs = _strides3(hd) if hd is not None else z3
    ns = _strides3(src)
    ps = _strides3(pk) if pk is not None else z3
    ks = _strides3(K_scale) if K_scale is not None else z3
    vs = _strides3(V_scale) if V_scale is not None else z3
    ss = _strides3(st) if st is not None else z3
    with torch.cuda.device(ref.device):
        check(lib().fq_quantize_kv_int4(
            ptr(K_head), ptr(V_head), *hs, int(n_head),
            ptr(K_new), ptr(V_new), *ns, int(n_new),
            dtype_code(ref), B, H, D, int(page_size), int(n_quant),
            ptr(K_packed), ptr(V_packed), *ps,
            ptr(K_scale), ptr(K_mn), *ks,
            ptr(V_scale), ptr(V_mn), *vs,
            ptr(stage_K), ptr(stage_V), *ss,
            stream_ptr(ref.device)))


def quantize_k_int4(K: torch.Tensor, page_size: int):
    """KIVI-style asymmetric INT4 K quant, packed 2-per-byte along head_dim
    (kernel/kv_quant.py:152).

    Returns (K_packed (B,H,S,D//2) uint8, scale (B,H,num_pages,D) bf16, mn (B,H,num_pages,D) bf16).
    """
    B, H, S, D = K.shape
    if D % 2 != 0:
        raise ValueError(f"quantize_k_int4 requires even head_dim; got {D}")
    require_cuda(K)
    P = (S + page_size - 1) // page_size
    K_packed = torch.empty(B, H, S, D // 2, dtype=torch.uint8, device=K.device)
    scale = torch.empty(B, H, P, D, dtype=torch.bfloat16, device=K.device)
    mn = torch.empty(B, H, P, D, dtype=torch.bfloat16, device=K.device)
    if S > 0:
        quantize_kv_int4_into(K, None, page_size, S, K_packed=K_packed, K_scale=scale, K_mn=mn)
    return K_packed, scale, mn


def quantize_v_int4(V: torch.Tensor):
    """Per-token V quant, packed 2-per-byte along head_dim (kernel/kv_quant.py:189).

    Returns (V_packed (B,H,S,D//2) uint8, scale (B,H,S,1) bf16, mn (B,H,S,1) bf16).
    """
    if V.shape[-1] % 2 != 0:
        raise ValueError(f"quantize_v_int4 requires even head_dim; got {V.shape[-1]}")
    require_cuda(V)
    B, H, S, D = V.shape
    V_packed = torch.empty(B, H, S, D // 2, dtype=torch.uint8, device=V.device)
    scale = torch.empty(B, H, S, 1, dtype=torch.bfloat16, device=V.device)
    mn = torch.empty(B, H, S, 1, dtype=torch.bfloat16, device=V.device)
    if S > 0:
        # page size only groups tokens into warps here; V metadata is per token
        quantize_kv_int4_into(None, V, 16, S, V_packed=V_packed, V_scale=scale, V_mn=mn)
    return V_packed, scale, mn


def _dequantize_int4(packed, scale, mn, page_size, per_page):
    require_cuda(packed, scale, mn)
    B, H, S, Dp = packed.shape
    D = Dp * 2
    packed = inner_contiguous(packed)
    scale, mn = inner_contiguous(scale), inner_contiguous(mn)
    if _strides3(scale) != _strides3(mn):
        scale, mn = scale.contiguous(), mn.contiguous()
    out = torch.empty(B, H, S, D, dtype=torch.bfloat16, device=packed.device)
    with torch.cuda.device(packed.device):
        check(lib().fq_dequantize_int4(
            ptr(packed), *_strides3(packed), ptr(scale), ptr(mn), *_strides3(scale),
            1 if per_page else 0, B, H, S, D, int(page_size),
            ptr(out), *_strides3(out), stream_ptr(packed.device)))
    return out


def dequantize_k_int4(K_packed, scale, mn, page_size: int) -> torch.Tensor:
    """Inverse of quantize_k_int4 (kernel/kv_quant.py:174).  Returns bf16."""
    return _dequantize_int4(K_packed, scale, mn, page_size, True)


def dequantize_v_int4(V_packed, scale, mn) -> torch.Tensor:
    """Inverse of quantize_v_int4 (kernel/kv_quant.py:208).  Returns bf16."""
    return _dequantize_int4(V_packed, scale, mn, 1, False)


# === INT8 KV variant (kernel/kv_quant.py:18-103) ===

def quantize_kv_int8_into(K, V, page_size, *, K_uint8=None, K_scale=None, K_mn=None, V_uint8=None, V_scale=None, V_mn=None):
    """One call of fq_quantize_kv_int8 writing into (possibly strided) output views; K or V may be None."""
    ref = K if K is not None else V
    require_cuda(ref)
    B, H, S, D = ref.shape
    K = inner_contiguous(K) if K is not None else None
    V = inner_contiguous(V) if V is not None else None
    if K is not None and V is not None and _strides3(K) != _strides3(V):
        K, V = K.contiguous(), V.contiguous()
    src = K if K is not None else V
    cod = K_uint8 if K_uint8 is not None else V_uint8
    if K_uint8 is not None and V_uint8 is not None and _strides3(K_uint8) != _strides3(V_uint8):
        raise ValueError("K_uint8 and V_uint8 must share their strides")
    z3 = (0, 0, 0)
    with torch.cuda.device(ref.device):
        check(lib().fq_quantize_kv_int8(
            ptr(K), ptr(V), *_strides3(src), dtype_code(ref), B, H, S, D, int(page_size),
            ptr(K_uint8), ptr(V_uint8), *_strides3(cod),
            ptr(K_scale), ptr(K_mn), *(_strides3(K_scale) if K_scale is not None else z3),
            ptr(V_scale), ptr(V_mn), *(V_scale.stride()[:2] if V_scale is not None else (0, 0)),
            stream_ptr(ref.device)))


def quantize_k(K: torch.Tensor, page_size: int):
    """uint8 K with per-page per-channel (scale, mn) (kernel/kv_quant.py:45).
    Returns (K_uint8 (B,H,S,D), scale (B,H,num_pages,D) bf16, mn (B,H,num_pages,D) bf16)."""
    B, H, S, D = K.shape
    require_cuda(K)
    P = (S + page_size - 1) // page_size
    codes = torch.empty(B, H, S, D, dtype=torch.uint8, device=K.device)
    scale = torch.empty(B, H, P, D, dtype=torch.bfloat16, device=K.device)
    mn = torch.empty(B, H, P, D, dtype=torch.bfloat16, device=K.device)
    if S > 0:
        quantize_kv_int8_into(K, None, page_size, K_uint8=codes, K_scale=scale, K_mn=mn)
    return codes, scale, mn


def quantize_v(V: torch.Tensor):
    """uint8 V per token (kernel/kv_quant.py:81).  Returns (V_uint8 (B,H,S,D), scale (B,H,S,1) bf16, mn (B,H,S,1) bf16)."""
    B, H, S, D = V.shape
    require_cuda(V)
    codes = torch.empty(B, H, S, D, dtype=torch.uint8, device=V.device)
    scale = torch.empty(B, H, S, 1, dtype=torch.bfloat16, device=V.device)
    mn = torch.empty(B, H, S, 1, dtype=torch.bfloat16, device=V.device)
    if S > 0:
        quantize_kv_int8_into(None, V, 16, V_uint8=codes, V_scale=scale, V_mn=mn)
    return codes, scale, mn


def _dequantize_int8(codes, scale, mn, page_size, per_page):
    require_cuda(codes, scale, mn)
    B, H, S, D = codes.shape
    codes = inner_contiguous(codes)
    scale, mn = inner_contiguous(scale), inner_contiguous(mn)
    if _strides3(scale) != _strides3(mn):
        scale, mn = scale.contiguous(), mn.contiguous()
    out = torch.empty(B, H, S, D, dtype=torch.bfloat16, device=codes.device)
    if S > 0:
        with torch.cuda.device(codes.device):
            check(lib().fq_dequantize_int8(ptr(codes), *_strides3(codes), ptr(scale), ptr(mn), *_strides3(scale),
                                           1 if per_page else 0, B, H, S, D, int(page_size), ptr(out), *_strides3(out),
                                           stream_ptr(codes.device)))
    return out


def dequantize_k(K_uint8, scale, mn, page_size: int) -> torch.Tensor:
    """Inverse of quantize_k (kernel/kv_quant.py:65).  Returns bf16."""
    return _dequantize_int8(K_uint8, scale, mn, page_size, True)


def dequantize_v(V_uint8, scale, mn) -> torch.Tensor:
    """Inverse of quantize_v (kernel/kv_quant.py:96).  Returns bf16."""
    return _dequantize_int8(V_uint8, scale, mn, 1, False)


# === TurboQuant K3-V3 (kernel/kv_quant.py:225-420) ===

K_TURBO_CODEBOOK_VALUES = (-2.1519, -1.3439, -0.7560, -0.2451, 0.2451, 0.7560, 1.3439, 2.1519)


def quantize_turbo_into(x_new, n_quant, *, msb, lsb, scale, head=None, n_head=0):
    """One launch of fq_quantize_turbo over the stream head[:n_head] ++ x_new, writing planes
    and scales into (possibly strided) views."""
    require_cuda(x_new)
    B, H, n_new, D = x_new.shape
    x_new = inner_contiguous(x_new)
    z3 = (0, 0, 0)
    hs = _strides3(head) if head is not None else z3
    with torch.cuda.device(x_new.device):
        check(lib().fq_quantize_turbo(
            ptr(head), *hs, int(n_head), ptr(x_new), *_strides3(x_new), int(n_new),
            dtype_code(x_new), B, H, D, int(n_quant),
            ptr(msb), *_strides3(msb), ptr(lsb), *_strides3(lsb), ptr(scale), *_strides3(scale),
            stream_ptr(x_new.device)))


def _quantize_turbo(x: torch.Tensor, name: str):
    B, H, S, D = x.shape
    if D % 8 != 0:
        raise ValueError(f"{name} requires head_dim multiple of 8; got {D}")
    require_cuda(x)
    msb = torch.empty(B, H, S, D // 8, dtype=torch.uint8, device=x.device)
    lsb = torch.empty(B, H, S, D // 4, dtype=torch.uint8, device=x.device)
    scale = torch.empty(B, H, S, 1, dtype=torch.bfloat16, device=x.device)
    if S > 0:
        quantize_turbo_into(x, S, msb=msb, lsb=lsb, scale=scale)
    return msb, lsb, scale


def quantize_k_turbo(K: torch.Tensor, page_size: int):
    """TurboQuant K: WHT -> per-token RMS scale -> 3-bit Lloyd-Max -> bit-split planes, plus
    the un-rotated per-page (scale, mn) used for page scoring (kernel/kv_quant.py:327).

    Returns (K_msb (B,H,S,D/8) u8, K_lsb (B,H,S,D/4) u8, K_scale_turbo (B,H,S,1) bf16,
             K_scale_raw (B,H,P,D) bf16, K_mn_raw (B,H,P,D) bf16)."""
    B, H, S, D = K.shape
    msb, lsb, scale = _quantize_turbo(K, "quantize_k_turbo")
    P = (S + page_size - 1) // page_size
    sr = torch.empty(B, H, P, D, dtype=torch.bfloat16, device=K.device)
    mr = torch.empty(B, H, P, D, dtype=torch.bfloat16, device=K.device)
    if S > 0:
        quantize_kv_int4_into(K, None, page_size, S, K_scale=sr, K_mn=mr)     # metadata only
    return msb, lsb, scale, sr, mr


def quantize_v_turbo(V: torch.Tensor):
    """TurboQuant V (K3-V3): same coding as K, no page metadata (kernel/kv_quant.py:381)."""
    return _quantize_turbo(V, "quantize_v_turbo")


def dequantize_k_turbo(K_msb, K_lsb, K_scale_turbo, head_dim: int) -> torch.Tensor:
    """Inverse: planes -> codebook -> * scale -> inverse WHT -> bf16 (kernel/kv_quant.py:366)."""
    require_cuda(K_msb, K_lsb, K_scale_turbo)
    B, H, S, Dm = K_msb.shape
    if Dm * 8 != head_dim:
        raise ValueError(f"_unpack_bit_split: msb last axis {Dm} * 8 != head_dim {head_dim}")
    if K_lsb.shape[-1] * 4 != head_dim:
        raise ValueError(f"_unpack_bit_split: lsb last axis {K_lsb.shape[-1]} * 4 != head_dim {head_dim}")
    K_msb, K_lsb = inner_contiguous(K_msb), inner_contiguous(K_lsb)
    sc = K_scale_turbo
    out = torch.empty(B, H, S, head_dim, dtype=torch.bfloat16, device=K_msb.device)
    with torch.cuda.device(K_msb.device):
        check(lib().fq_dequantize_turbo(
            ptr(K_msb), *_strides3(K_msb), ptr(K_lsb), *_strides3(K_lsb), ptr(sc), *_strides3(sc),
            B, H, S, head_dim, ptr(out), *_strides3(out), stream_ptr(K_msb.device)))
    return out


dequantize_v_turbo = dequantize_k_turbo
