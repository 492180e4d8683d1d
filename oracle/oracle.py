"""ctypes front-end of the C oracle (``fq_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Every function takes and returns torch CPU tensors (used purely as typed memory; all
arithmetic happens in C) and carries the name, argument order and return tuple of the
reference function it restates.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
import threading

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "fq_oracle.c")
_LIB = os.path.join(_HERE, "libfq_oracle.so")
_lock = threading.Lock()
_lib = None

__all__ = [
    "quantize_k_int4", "quantize_v_int4", "dequantize_k_int4", "dequantize_v_int4",
    "k_page_meta_int4", "wht_along_head_dim", "quantize_k_turbo", "quantize_v_turbo",
    "dequantize_k_turbo", "dequantize_v_turbo", "turbo_codebook", "page_scores_int4_fast",
    "k_per_head", "select_pages_vectorized", "build_compact_selection", "sparse_attn_int4",
    "sparse_attn_turbo", "sparse_attn_turbo_rotated", "lse_merge", "quantize_k", "quantize_v", "dequantize_k", "dequantize_v",
    "page_scores_int8_fast", "sparse_attn_int8", "awq_gemv", "awq_pack", "set_num_threads",
]


def lib_path() -> str:
    return _LIB


def build_oracle(force: bool = False) -> str:
    """Compile fq_oracle.c into libfq_oracle.so beside it (gcc, OpenMP, no fast-math,
    no FMA contraction)."""
    with _lock:
        if (not force and os.path.exists(_LIB)
                and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC)):
            return _LIB
        cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-mavx2",
               "-mfma", "-mf16c", "-shared", "-fPIC", _SRC, "-o", _LIB, "-lm"]
        subprocess.run(cmd, check=True)
        return _LIB


def _load():
    global _lib
    if _lib is None:
        build_oracle()
        _lib = ctypes.CDLL(_LIB)
        try:
            _lib_omp = ctypes.CDLL("libgomp.so.1")
            _lib._omp = _lib_omp
        except OSError:  # pragma: no cover
            _lib._omp = None
    return _lib


def set_num_threads(n: int) -> None:
    """OpenMP thread count used by the oracle loops."""
    lib = _load()
    if lib._omp is not None:
        lib._omp.omp_set_num_threads(int(n))


_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _dt(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        raise TypeError(f"oracle supports fp32/fp16/bf16, got {t.dtype}")
    return _DT[t.dtype]


def _c(t: torch.Tensor) -> torch.Tensor:
    if t.device.type != "cpu":
        raise ValueError("oracle takes CPU tensors")
    return t.contiguous()


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _bf16_empty(*shape):
    return torch.empty(*shape, dtype=torch.bfloat16)


# ---------------------------------------------------------------- INT4

def quantize_k_int4(K: torch.Tensor, page_size: int):
    """kernel/kv_quant.py:152 — (K_packed u8, scale bf16 (B,H,P,D), mn bf16)."""
    B, H, S, D = K.shape
    if D % 2 != 0:
        raise ValueError(f"quantize_k_int4 requires even head_dim; got {D}")
    K = _c(K)
    P = (S + page_size - 1) // page_size
    packed = torch.empty(B, H, S, D // 2, dtype=torch.uint8)
    scale, mn = _bf16_empty(B, H, P, D), _bf16_empty(B, H, P, D)
    _load().orc_quantize_k_int4(_p(K), _dt(K), B, H, S, D, page_size, _p(packed), _p(scale), _p(mn))
    return packed, scale, mn


def k_page_meta_int4(K: torch.Tensor, page_size: int):
    """kernel/kv_quant.py:131 rounded to bf16 as quantize_k_turbo returns it (:355-362)."""
    B, H, S, D = K.shape
    K = _c(K)
    P = (S + page_size - 1) // page_size
    scale, mn = _bf16_empty(B, H, P, D), _bf16_empty(B, H, P, D)
    _load().orc_k_page_meta(_p(K), _dt(K), B, H, S, D, page_size, _p(scale), _p(mn))
    return scale, mn


def quantize_v_int4(V: torch.Tensor):
    """kernel/kv_quant.py:189 — (V_packed u8, scale bf16 (B,H,S,1), mn bf16)."""
    B, H, S, D = V.shape
    if D % 2 != 0:
        raise ValueError(f"quantize_v_int4 requires even head_dim; got {D}")
    V = _c(V)
    packed = torch.empty(B, H, S, D // 2, dtype=torch.uint8)
    scale, mn = _bf16_empty(B, H, S, 1), _bf16_empty(B, H, S, 1)
    _load().orc_quantize_v_int4(_p(V), _dt(V), ctypes.c_long(B * H * S), D, _p(packed), _p(scale), _p(mn))
    return packed, scale, mn


def dequantize_k_int4(K_packed, scale, mn, page_size: int):
    """kernel/kv_quant.py:174 — bf16 (B,H,S,D)."""
    B, H, S, Dp = K_packed.shape
    out = _bf16_empty(B, H, S, Dp * 2)
    _load().orc_dequantize_int4(_p(_c(K_packed)), _p(_c(scale)), _p(_c(mn)), ctypes.c_long(B * H),
                                S, Dp * 2, page_size, 1, _p(out))
    return out


def dequantize_v_int4(V_packed, scale, mn):
    """kernel/kv_quant.py:208 — bf16 (B,H,S,D)."""
    B, H, S, Dp = V_packed.shape
    out = _bf16_empty(B, H, S, Dp * 2)
    _load().orc_dequantize_int4(_p(_c(V_packed)), _p(_c(scale)), _p(_c(mn)), ctypes.c_long(B * H),
                                S, Dp * 2, 1, 0, _p(out))
    return out


# ---------------------------------------------------------------- WHT / Turbo

def wht_along_head_dim(x: torch.Tensor) -> torch.Tensor:
    """kernel/wht.py:17."""
    D = x.shape[-1]
    if D & (D - 1) != 0 or D == 0:
        raise ValueError(f"head_dim must be a positive power of 2, got {D}")
    x = _c(x)
    out = torch.empty_like(x)
    _load().orc_wht(_p(x), _dt(x), ctypes.c_long(x.numel() // D), D, _p(out))
    return out


def turbo_codebook() -> torch.Tensor:
    out = torch.empty(8, dtype=torch.float32)
    _load().orc_turbo_codebook(_p(out))
    return out


def _quantize_turbo(x: torch.Tensor):
    B, H, S, D = x.shape
    x = _c(x)
    msb = torch.empty(B, H, S, D // 8, dtype=torch.uint8)
    lsb = torch.empty(B, H, S, D // 4, dtype=torch.uint8)
    scale = _bf16_empty(B, H, S, 1)
    _load().orc_quantize_turbo(_p(x), _dt(x), ctypes.c_long(B * H * S), D, _p(msb), _p(lsb), _p(scale))
    return msb, lsb, scale


def quantize_k_turbo(K: torch.Tensor, page_size: int):
    """kernel/kv_quant.py:327 — (K_msb, K_lsb, K_scale_turbo, K_scale_raw, K_mn_raw)."""
    if K.shape[-1] % 8 != 0:
        raise ValueError(f"quantize_k_turbo requires head_dim multiple of 8; got {K.shape[-1]}")
    msb, lsb, scale = _quantize_turbo(K)
    sr, mr = k_page_meta_int4(K, page_size)
    return msb, lsb, scale, sr, mr


def quantize_v_turbo(V: torch.Tensor):
    """kernel/kv_quant.py:381 — (V_msb, V_lsb, V_scale_turbo)."""
    if V.shape[-1] % 8 != 0:
        raise ValueError(f"quantize_v_turbo requires head_dim multiple of 8; got {V.shape[-1]}")
    return _quantize_turbo(V)


def dequantize_k_turbo(K_msb, K_lsb, K_scale_turbo, head_dim: int):
    """kernel/kv_quant.py:366 — bf16 (B,H,S,D) in the raw basis."""
    B, H, S, _ = K_msb.shape
    out = _bf16_empty(B, H, S, head_dim)
    _load().orc_dequantize_turbo(_p(_c(K_msb)), _p(_c(K_lsb)), _p(_c(K_scale_turbo)),
                                 ctypes.c_long(B * H * S), head_dim, _p(out))
    return out


dequantize_v_turbo = dequantize_k_turbo


# ---------------------------------------------------------------- scores / selection

def page_scores_int4_fast(Q, K_scale, K_mn):
    """eager/criticality.py:128 — (B,H_q,1,P) fp32."""
    B, H_q, S_q, D = Q.shape
    if S_q != 1:
        raise NotImplementedError("oracle scores are decode-only (S_q == 1)")
    H_kv, P = K_scale.shape[1], K_scale.shape[2]
    if H_q % H_kv != 0:
        raise ValueError(f"H_q={H_q} must be divisible by H_kv={H_kv}")
    Q = _c(Q)
    out = torch.empty(B, H_q, 1, P, dtype=torch.float32)
    _load().orc_page_scores_int4(_p(Q), _dt(Q), _p(_c(K_scale)), _p(_c(K_mn)), B, H_q, H_kv, P, D, _p(out))
    return out


def k_per_head(retention, H: int, P: int) -> np.ndarray:
    """eager/selection.py:92-103: k_h = clamp(ceil(fp32(r_h) * P), 0, P), product in fp32."""
    if isinstance(retention, torch.Tensor):
        if tuple(retention.shape) != (H,):
            raise ValueError(f"per-head retention must be shape ({H},); got {tuple(retention.shape)}")
        r = retention.detach().cpu().float().numpy().astype(np.float32)
    else:
        if not (0.0 <= retention <= 1.0):
            raise ValueError(f"scalar retention must be in [0, 1]; got {retention}")
        r = np.full((H,), np.float32(retention), dtype=np.float32)
    k = np.ceil(r * np.float32(P)).astype(np.int64)
    return np.clip(k, 0, P).astype(np.int32)


def select_pages_vectorized(scores, retention, num_sinks, window_pages, *, k_max_static=None):
    """eager/selection.py:65 — bool (B,H,S_q,P).  Ties: lower page index wins."""
    B, H, S_q, P = scores.shape
    if S_q != 1:
        raise NotImplementedError("oracle selection is decode-only (S_q == 1)")
    kh = k_per_head(retention, H, P)
    k_max = int(kh.max()) if k_max_static is None else min(int(k_max_static), P)
    scores = _c(scores.float())
    mask = torch.empty(B, H, 1, P, dtype=torch.uint8)
    kh_t = torch.from_numpy(np.ascontiguousarray(kh))
    _load().orc_select_pages(_p(scores), B, H, P, _p(kh_t), k_max, int(num_sinks), int(window_pages), _p(mask))
    return mask.bool()


def build_compact_selection(mask, BUCKET_MAX: int):
    """eager/selection.py:129 — int32 (B,H,S_q,BUCKET_MAX), descending ids, -1 padded."""
    if BUCKET_MAX < 1:
        raise ValueError(f"BUCKET_MAX must be >= 1, got {BUCKET_MAX}")
    if mask.dtype != torch.bool:
        raise ValueError(f"mask must be bool, got {mask.dtype}")
    B, H, S_q, P = mask.shape
    m8 = _c(mask.to(torch.uint8))
    out = torch.empty(B, H, S_q, BUCKET_MAX, dtype=torch.int32)
    _load().orc_build_compact(_p(m8), ctypes.c_long(B * H * S_q), P, BUCKET_MAX, _p(out))
    return out


# ---------------------------------------------------------------- attention

def sparse_attn_int4(Q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn, *, selection_mask=None,
                     selected_page_ids=None, page_size=64, sm_scale=None, K_partial=None,
                     V_partial=None):
    """kernel/sparse_int4_fwd.py:160 and sparse_int4_fwd_compact.py:153 semantics in fp64
    accumulation; optional bf16/fp16 tail attended in the same softmax
    (eager/llama_persistent_patch.py:30-61).  Returns (O fp32 (B,H_q,1,D), lse (B,H_q,1))."""
    B, H_q, S_q, D = Q.shape
    if S_q != 1:
        raise NotImplementedError(f"decode-only (S_q={S_q})")
    H_kv, S_kv = K_packed.shape[1], K_packed.shape[2]
    P = K_scale.shape[2]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    Q = _c(Q)
    m8 = None
    comp = None
    bucket = 0
    if selection_mask is not None:
        m8 = _c(selection_mask.reshape(B, H_q, P).to(torch.uint8))
    elif selected_page_ids is not None:
        comp = _c(selected_page_ids.reshape(B, H_q, -1).to(torch.int32))
        bucket = comp.shape[-1]
    tail_len = 0
    kt = vt = None
    tail_dt = 2
    if K_partial is not None and K_partial.shape[2] > 0:
        kt, vt = _c(K_partial), _c(V_partial)
        tail_len = kt.shape[2]
        tail_dt = _dt(kt)
    O = torch.empty(B, H_q, 1, D, dtype=torch.float32)
    lse = torch.empty(B, H_q, 1, dtype=torch.float32)
    _load().orc_sparse_attn_int4(
        _p(Q), _dt(Q), _p(_c(K_packed)), _p(_c(K_scale)), _p(_c(K_mn)),
        _p(_c(V_packed)), _p(_c(V_scale)), _p(_c(V_mn)),
        _p(m8), _p(comp), bucket, _p(kt), _p(vt), tail_dt, tail_len,
        B, H_q, H_kv, S_kv, P, D, int(page_size), ctypes.c_float(sm_scale), _p(O), _p(lse))
    return O, lse


def sparse_attn_turbo_rotated(Q_rot, K_msb, K_lsb, K_scale_turbo, V_msb, V_lsb, V_scale_turbo, *,
                              selection_mask, page_size=64, sm_scale=None):
    """The kernel part of kernel/sparse_turbo_fwd.py:92-251 in fp64 accumulation: Q_rot (fp32, fp16 or
    bf16) is already in the rotated basis and O comes back in the rotated basis (fp32), so that a
    GPU kernel can be compared on exactly the same operands, without the two rotations.
    Returns (O_rot fp32 (B,H_q,1,D), lse (B,H_q,1))."""
    B, H_q, S_q, D = Q_rot.shape
    if S_q != 1:
        raise NotImplementedError(f"decode-only (S_q={S_q})")
    H_kv, S_kv = K_msb.shape[1], K_msb.shape[2]
    P = selection_mask.shape[-1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    Q_rot = _c(Q_rot)
    m8 = _c(selection_mask.reshape(B, H_q, P).to(torch.uint8))
    O_rot = torch.empty(B, H_q, 1, D, dtype=torch.float32)
    lse = torch.empty(B, H_q, 1, dtype=torch.float32)
    _load().orc_sparse_attn_turbo(
        _p(Q_rot), _dt(Q_rot), _p(_c(K_msb)), _p(_c(K_lsb)), _p(_c(K_scale_turbo)),
        _p(_c(V_msb)), _p(_c(V_lsb)), _p(_c(V_scale_turbo)), _p(m8),
        B, H_q, H_kv, S_kv, P, D, int(page_size), ctypes.c_float(sm_scale), _p(O_rot), _p(lse))
    return O_rot, lse


def sparse_attn_turbo(Q, K_msb, K_lsb, K_scale_turbo, V_msb, V_lsb, V_scale_turbo, *,
                      selection_mask, page_size=64, sm_scale=None):
    """kernel/sparse_turbo_fwd.py:254 semantics with fp32 rotations and fp64 accumulation:
    Q is rotated (WHT in fp32), attention runs in the rotated basis, O is rotated back in
    fp32.  Returns (O fp32 (B,H_q,1,D) raw basis, lse (B,H_q,1))."""
    O_rot, lse = sparse_attn_turbo_rotated(wht_along_head_dim(Q.float()), K_msb, K_lsb, K_scale_turbo, V_msb, V_lsb,
                                           V_scale_turbo, selection_mask=selection_mask, page_size=page_size, sm_scale=sm_scale)
    return wht_along_head_dim(O_rot), lse


def lse_merge(O_parts: torch.Tensor, lse_parts: torch.Tensor):
    """eager/llama_persistent_patch.py:50 for n parts: O_parts (n, rows..., D) fp32,
    lse_parts (n, rows...) -> (O (rows..., D), lse (rows...))."""
    n = O_parts.shape[0]
    D = O_parts.shape[-1]
    rows = O_parts[0].numel() // D
    Op, lp = _c(O_parts.float()), _c(lse_parts.float())
    O = torch.empty(O_parts.shape[1:], dtype=torch.float32)
    lse = torch.empty(lse_parts.shape[1:], dtype=torch.float32)
    _load().orc_lse_merge(_p(Op), _p(lp), n, ctypes.c_long(rows), D, _p(O), _p(lse))
    return O, lse


# ---------------------------------------------------------------- INT8 KV variant

def quantize_k(K: torch.Tensor, page_size: int):
    """kernel/kv_quant.py:45 — (K_uint8 (B,H,S,D), scale, mn (B,H,P,D) bf16)."""
    B, H, S, D = K.shape
    P = (S + page_size - 1) // page_size
    K = _c(K)
    codes = torch.empty(B, H, S, D, dtype=torch.uint8)
    scale = torch.empty(B, H, P, D, dtype=torch.bfloat16)
    mn = torch.empty(B, H, P, D, dtype=torch.bfloat16)
    _load().orc_quantize_k_int8(_p(K), _dt(K), B, H, S, D, page_size, _p(codes), _p(scale), _p(mn))
    return codes, scale, mn


def quantize_v(V: torch.Tensor):
    """kernel/kv_quant.py:81 — (V_uint8 (B,H,S,D), scale, mn (B,H,S,1) bf16)."""
    B, H, S, D = V.shape
    V = _c(V)
    codes = torch.empty(B, H, S, D, dtype=torch.uint8)
    scale = torch.empty(B, H, S, 1, dtype=torch.bfloat16)
    mn = torch.empty(B, H, S, 1, dtype=torch.bfloat16)
    _load().orc_quantize_v_int8(_p(V), _dt(V), ctypes.c_long(B * H * S), D, _p(codes), _p(scale), _p(mn))
    return codes, scale, mn


def _dequantize_int8(codes, scale, mn, page_size, per_page):
    B, H, S, D = codes.shape
    out = torch.empty(B, H, S, D, dtype=torch.bfloat16)
    _load().orc_dequantize_int8(_p(_c(codes)), _p(_c(scale)), _p(_c(mn)), ctypes.c_long(B * H), S, D, int(page_size),
                                1 if per_page else 0, _p(out))
    return out


def dequantize_k(K_uint8, scale, mn, page_size: int):
    """kernel/kv_quant.py:65."""
    return _dequantize_int8(K_uint8, scale, mn, page_size, True)


def dequantize_v(V_uint8, scale, mn):
    """kernel/kv_quant.py:96."""
    return _dequantize_int8(V_uint8, scale, mn, 1, False)


def page_scores_int8_fast(Q, K_scale, K_mn):
    """eager/criticality.py:77 — (B,H_q,1,P) fp32, same fixed summation order as page_scores_int4_fast."""
    B, H_q, S_q, D = Q.shape
    if S_q != 1:
        raise NotImplementedError("oracle page scores are decode-only (S_q == 1)")
    H_kv, P = K_scale.shape[1], K_scale.shape[2]
    if H_q % H_kv != 0:
        raise ValueError(f"H_q={H_q} must be divisible by H_kv={H_kv}")
    Q = _c(Q)
    out = torch.empty(B, H_q, 1, P, dtype=torch.float32)
    _load().orc_page_scores_int8(_p(Q), _dt(Q), _p(_c(K_scale)), _p(_c(K_mn)), B, H_q, H_kv, P, D, _p(out))
    return out


def sparse_attn_int8(Q, K_uint8, K_scale, K_mn, V_uint8, V_scale, V_mn, *, selection_mask=None, selected_page_ids=None,
                     page_size=64, sm_scale=None, K_partial=None, V_partial=None):
    """kernel/sparse_fwd.py:140 semantics in fp64 accumulation (+ optional staged tail).  Returns (O fp32, lse)."""
    B, H_q, S_q, D = Q.shape
    if S_q != 1:
        raise NotImplementedError(f"decode-only (S_q={S_q})")
    H_kv, S_kv = K_uint8.shape[1], K_uint8.shape[2]
    P = K_scale.shape[2]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    Q = _c(Q)
    m8 = comp = None
    bucket = 0
    if selection_mask is not None:
        m8 = _c(selection_mask.reshape(B, H_q, P).to(torch.uint8))
    elif selected_page_ids is not None:
        comp = _c(selected_page_ids.reshape(B, H_q, -1).to(torch.int32))
        bucket = comp.shape[-1]
    tail_len, kt, vt, tail_dt = 0, None, None, 2
    if K_partial is not None and K_partial.shape[2] > 0:
        kt, vt = _c(K_partial), _c(V_partial)
        tail_len, tail_dt = kt.shape[2], _dt(kt)
    O = torch.empty(B, H_q, 1, D, dtype=torch.float32)
    lse = torch.empty(B, H_q, 1, dtype=torch.float32)
    _load().orc_sparse_attn_int8(
        _p(Q), _dt(Q), _p(_c(K_uint8)), _p(_c(K_scale)), _p(_c(K_mn)), _p(_c(V_uint8)), _p(_c(V_scale)), _p(_c(V_mn)),
        _p(m8), _p(comp), bucket, _p(kt), _p(vt), tail_dt, tail_len,
        B, H_q, H_kv, S_kv, P, D, int(page_size), ctypes.c_float(sm_scale), _p(O), _p(lse))
    return O, lse


# ---------------------------------------------------------------- AWQ

_AWQ_ORDER = [0, 2, 4, 6, 1, 3, 5, 7]


def awq_pack(codes: torch.Tensor, interleaved: bool = True) -> torch.Tensor:
    """Pack 4-bit codes (rows, N) into int32 (rows, N/8) along N (quant/awq_layout.py:26-31).
    interleaved: nibble i of an int32 holds column 8c + [0,2,4,6,1,3,5,7][i] (AutoAWQ's
    GEMM order); otherwise nibble i holds column 8c + i."""
    rows, N = codes.shape
    c = codes.to(torch.int64).reshape(rows, N // 8, 8)
    out = torch.zeros(rows, N // 8, dtype=torch.int64)
    for i in range(8):
        col = _AWQ_ORDER[i] if interleaved else i
        out |= (c[:, :, col] & 15) << (4 * i)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def awq_gemv(x, qweight, scales, qzeros, *, group_size=128, interleaved=True):
    """y = x @ dequant(W): w = (code - zero) * scale (AutoAWQ 0.2.9 GEMM format).
    x (M,K) fp16 -> y (M,N) fp32."""
    M, K = x.shape
    N = scales.shape[1]
    y = torch.empty(M, N, dtype=torch.float32)
    _load().orc_awq_gemv(_p(_c(x.half())), _p(_c(qweight)), _p(_c(scales.half())), _p(_c(qzeros)),
                         M, K, N, int(group_size), 1 if interleaved else 0, _p(y))
    return y
