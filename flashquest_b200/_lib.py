"""ctypes binding of libflashquest_b200.so (the C ABI declared in include/flashquest_b200.h).

The library is the only compute path of this package: if it is missing or cannot be loaded
every operator raises; there is no eager / CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_size_t, c_void_p

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libflashquest_b200.so")

FQ_F32, FQ_F16, FQ_BF16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: FQ_F32, torch.float16: FQ_F16, torch.bfloat16: FQ_BF16}

_lib = None

I, L, P, F, Z = c_int, c_int64, c_void_p, c_float, c_size_t

_PROTOTYPES = {
    "fq_last_error_string": (ctypes.c_char_p, []),
    "fq_version": (ctypes.c_char_p, []),
    "fq_device_status": (I, []),
    "fq_quantize_kv_int4": (I, [P, P, L, L, L, I, P, P, L, L, L, I, I, I, I, I, I, I,
                                P, P, L, L, L, P, P, L, L, L, P, P, L, L, L, P, P, L, L, L, P]),
    "fq_dequantize_int4": (I, [P, L, L, L, P, P, L, L, L, I, I, I, I, I, I, P, L, L, L, P]),
    "fq_page_scores_int4": (I, [P, I, L, L, P, P, L, L, L, I, I, I, I, I, P, L, L, P]),
    "fq_select_pages": (I, [P, L, L, I, I, I, P, F, I, I, I, P, L, L, P, L, L, I, P, P]),
    "fq_build_compact": (I, [P, L, L, I, P, L, I, P]),
    "fq_score_select_supported": (I, [I, I, I, I]),
    "fq_score_select": (I, [P, I, L, L, P, P, L, L, L, I, I, I, I, I, I, P, L, L, P, F, I, I, I, P, L, L, I, P, I, P]),
    "fq_sparse_decode_workspace_bytes": (Z, [I, I, I, I]),
    "fq_sparse_decode_default_splits": (I, [I, I, I, I]),
    "fq_sparse_decode_int4": (I, [P, I, L, L, P, L, L, P, P, L, L, L, P, L, L, P, P, L, L,
                                  P, L, L, I, P, P, I, L, L, L, I,
                                  I, I, I, I, I, I, I, F, P, L, L, P, P, Z, I, P]),
    "fq_sparse_decode_int4_counted": (I, [P, I, L, L, P, L, L, P, P, L, L, L, P, L, L, P, P, L, L,
                                          P, L, L, I, P, P, P, I, L, L, L, I,
                                          I, I, I, I, I, I, I, F, P, L, L, P, P, Z, I, P]),
    "fq_build_compact_counted": (I, [P, L, L, I, P, L, I, P, P]),
}



class Int4CacheDesc(ctypes.Structure):
    """struct fq_int4_cache (include/flashquest_b200.h)."""
    _fields_ = [("K_packed", P), ("V_packed", P), ("pk_sl", L), ("pk_sb", L), ("pk_sh", L), ("pk_ss", L),
                ("K_scale", P), ("K_mn", P), ("km_sl", L), ("km_sb", L), ("km_sh", L), ("km_sp", L),
                ("V_scale", P), ("V_mn", P), ("vm_sl", L), ("vm_sb", L), ("vm_sh", L),
                ("K_partial", P), ("V_partial", P), ("pt_sl", L), ("pt_sb", L), ("pt_sh", L), ("pt_ss", L),
                ("kv_dtype", I), ("L", I), ("B", I), ("Hkv", I), ("D", I), ("page", I), ("max_seq_len", I)]


class DecodeParams(ctypes.Structure):
    """struct fq_decode_params (include/flashquest_b200.h)."""
    _fields_ = [("Hq", I), ("retention_per_head", P), ("retention", F), ("k_max_static", I), ("sinks", I),
                ("window", I), ("bucket", I), ("sm_scale", F), ("n_split", I)]


class TurboCacheDesc(ctypes.Structure):
    """struct fq_turbo_cache (include/flashquest_b200.h)."""
    _fields_ = [("K_msb", P), ("K_lsb", P), ("V_msb", P), ("V_lsb", P),
                ("ms_sl", L), ("ms_sb", L), ("ms_sh", L), ("ms_ss", L), ("ls_sl", L), ("ls_sb", L), ("ls_sh", L), ("ls_ss", L),
                ("K_scale_turbo", P), ("V_scale_turbo", P), ("st_sl", L), ("st_sb", L), ("st_sh", L),
                ("K_scale_raw", P), ("K_mn_raw", P), ("km_sl", L), ("km_sb", L), ("km_sh", L), ("km_sp", L),
                ("K_partial", P), ("V_partial", P), ("pt_sl", L), ("pt_sb", L), ("pt_sh", L), ("pt_ss", L),
                ("kv_dtype", I), ("L", I), ("B", I), ("Hkv", I), ("D", I), ("page", I), ("max_seq_len", I)]


class AwqLinearDesc(ctypes.Structure):
    """struct fq_awq_linear."""
    _fields_ = [("qweight", P), ("scales", P), ("qzeros", P), ("bias", P), ("K", I), ("N", I)]


class LlamaLayerDesc(ctypes.Structure):
    """struct fq_llama_layer."""
    _fields_ = [("input_norm", P), ("q", AwqLinearDesc), ("k", AwqLinearDesc), ("v", AwqLinearDesc), ("o", AwqLinearDesc),
                ("post_norm", P), ("gate", AwqLinearDesc), ("up", AwqLinearDesc), ("down", AwqLinearDesc)]


class LlamaModelDesc(ctypes.Structure):
    """struct fq_llama_model."""
    _fields_ = [("hidden", I), ("n_layers", I), ("q_heads", I), ("kv_heads", I), ("head_dim", I), ("ffn", I), ("vocab", I),
                ("group", I), ("interleaved", I), ("rope_theta", F), ("rms_eps", F),
                ("layers", ctypes.POINTER(LlamaLayerDesc)), ("final_norm", P), ("lm_head", P)]


class LlamaScratchDesc(ctypes.Structure):
    """struct fq_llama_scratch."""
    _fields_ = [("resid0", P), ("resid1", P), ("normed", P), ("q", P), ("k", P), ("v", P), ("attn_out", P), ("down", P),
                ("gate", P), ("up", P), ("logits", P), ("next_ids", P),
                ("scores", P), ("sc_sl", L), ("compact", P), ("cp_sl", L), ("O", P), ("o_sl", L),
                ("attn_ws", P), ("attn_ws_sl", Z), ("attn_ws_bytes", Z)]


_PROTOTYPES["fq_llama_decode_step"] = (I, [ctypes.POINTER(LlamaModelDesc), ctypes.POINTER(Int4CacheDesc),
                                          ctypes.POINTER(DecodeParams), P, P, I, ctypes.POINTER(LlamaScratchDesc), P])
_PROTOTYPES["fq_llama_decode_step_dev"] = _PROTOTYPES["fq_llama_decode_step"]


class GemvPrologue(ctypes.Structure):
    """struct fq_gemv_prologue."""
    _fields_ = [("kind", I), ("b", P), ("weight", P), ("eps", F), ("out", P)]


class GemvRope(ctypes.Structure):
    """struct fq_gemv_rope."""
    _fields_ = [("proj_mask", ctypes.c_uint), ("pos_dev", P), ("pos", I), ("theta", F), ("head_dim", I)]


GEMV_PLAIN, GEMV_ADD_RMSNORM, GEMV_SWIGLU = 0, 1, 2
_PROTOTYPES["fq_awq_gemv_default_splits"] = (I, [I, I, I])
_PROTOTYPES["fq_awq_gemv"] = (I, [P, I, I, I, I, P, P, P, P, P, P, I, I, P])
_PROTOTYPES["fq_awq_gemv_fused"] = (I, [P, I, I, I, I, P, P, P, P, P, P, I, ctypes.POINTER(GemvPrologue), ctypes.POINTER(GemvRope), I, P])
_PROTOTYPES["fq_awq_gemm"] = (I, [P, I, I, I, I, P, P, P, P, P, P, I, P])
_PROTOTYPES["fq_wht"] = (I, [P, P, I, L, I, P])
_PROTOTYPES["fq_quantize_turbo"] = (I, [P, L, L, L, I, P, L, L, L, I, I, I, I, I, I, P, L, L, L, P, L, L, L, P, L, L, L, P])
_PROTOTYPES["fq_dequantize_turbo"] = (I, [P, L, L, L, P, L, L, L, P, L, L, L, I, I, I, I, P, L, L, L, P])
_PROTOTYPES["fq_sparse_decode_turbo"] = (I, [P, I, L, L, P, L, L, L, P, L, L, L, P, L, L, P, L, L, L, P, L, L, L, P, L, L,
                                            P, L, L, I, I, I, I, I, I, I, I, F, P, L, L, P, P, Z, I, P])
_PROTOTYPES["fq_lse_merge"] = (I, [P, P, I, I, L, I, P, P, P])
_PROTOTYPES["fq_sparse_decode_int4_static"] = (I, [P, I, L, L, P, L, L, P, P, L, L, L, P, L, L, P, P, L, L,
                                                  P, L, L, I, P, P, I, L, L, L, I,
                                                  I, I, I, I, I, I, I, F, P, L, L, P, I, P])
_PROTOTYPES["fq_decode_layer_int4"] = (I, [ctypes.POINTER(Int4CacheDesc), I, I, P, P, L, L, L, I, P, I, L, L,
                                          ctypes.POINTER(DecodeParams), P, P, P, P, P, Z, P])

_PROTOTYPES["fq_decode_step_int4"] = (I, [ctypes.POINTER(Int4CacheDesc), I, P, P, P, L, L, L, L, I, P, I, L, L, L,
                                         ctypes.POINTER(DecodeParams), Z, P, L, P, L, P, L, P, L, P, Z, Z, P])

_PROTOTYPES["fq_add_rmsnorm"] = (I, [P, P, P, F, L, I, P, P, P])
_PROTOTYPES["fq_rope"] = (I, [P, L, L, I, P, L, L, I, I, I, I, F, P])
_PROTOTYPES["fq_rope_tokens"] = (I, [P, L, L, I, P, L, L, I, I, I, I, F, P])
_PROTOTYPES["fq_swiglu"] = (I, [P, P, L, P, P])
_PROTOTYPES["fq_gemv_f16"] = (I, [P, P, I, I, I, P, P])
_PROTOTYPES["fq_argmax_f16"] = (I, [P, L, I, P, P])

_PROTOTYPES["fq_decode_step_int4_dev"] = _PROTOTYPES["fq_decode_step_int4"]
_PROTOTYPES["fq_decode_layer_turbo_scratch_bytes"] = (Z, [I, I, I])
_PROTOTYPES["fq_decode_layer_turbo"] = (I, [ctypes.POINTER(TurboCacheDesc), I, I, P, P, L, L, L, I, P, I, L, L,
                                           ctypes.POINTER(DecodeParams), P, P, P, Z, P, P, P, Z, P])
_PROTOTYPES["fq_lse_merge_strided"] = (I, [P, L, P, L, I, I, L, I, P, P, P])
_PROTOTYPES["fq_ctx_scratch_bytes"] = (Z, [I, I, I, I, I, I])
_PROTOTYPES["fq_ctx_local_candidates"] = (I, [P, I, L, L, P, P, L, L, L, I, I, I, I, I, I, I, I, I, P, Z, P, P])
_PROTOTYPES["fq_ctx_select_attend"] = (I, [P, I, I, I, I, I, I, I, I, P, I, L, L, P, L, L, P, P, L, L, L, P, L, L, P, P, L, L,
                                          P, P, I, L, L, L, I, I, I, I, I, I, F, I, P, Z, P, P, P, Z, I, P])
_PROTOTYPES["fq_quantize_kv_int8"] = (I, [P, P, L, L, L, I, I, I, I, I, I, P, P, L, L, L, P, P, L, L, L, P, P, L, L, P])
_PROTOTYPES["fq_dequantize_int8"] = (I, [P, L, L, L, P, P, L, L, L, I, I, I, I, I, I, P, L, L, L, P])
_PROTOTYPES["fq_page_scores_int8"] = (I, [P, I, L, L, P, P, L, L, L, I, I, I, I, I, P, L, L, P])
_PROTOTYPES["fq_sparse_decode_int8_workspace_bytes"] = (Z, [I, I, I, I])
_PROTOTYPES["fq_sparse_decode_int8"] = (I, [P, I, L, L, P, P, L, L, L, P, P, L, L, L, P, P, L, L, P, L, L, I,
                                           P, P, I, L, L, L, I, I, I, I, I, I, I, I, F, P, P, P, Z, I, P])
_PROTOTYPES["fq_sparse_decode_int8_counted"] = (I, [P, I, L, L, P, P, L, L, L, P, P, L, L, L, P, P, L, L, P, L, L, I, P,
                                                   P, P, I, L, L, L, I, I, I, I, I, I, I, I, F, P, P, P, Z, I, P])
_PROTOTYPES["fq_prefill_attention"] = (I, [P, L, L, L, P, L, L, L, P, L, L, L, I, I, I, I, I, I, I, F, P, L, L, L, P])

# entry points added by later sources register themselves here (name -> (restype, argtypes))
EXTRA_PROTOTYPES: dict = {}


class FlashQuestError(RuntimeError):
    pass


def lib():
    """The loaded shared library; raises if it has not been built (python -m flashquest_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FlashQuestError(
                f"{LIB_PATH} is missing: build it with `python -m flashquest_b200.build` "
                "(nvcc, sm_100a).  flashquest_b200 has no fallback path.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in {**_PROTOTYPES, **EXTRA_PROTOTYPES}.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def exported_symbols():
    return sorted({**_PROTOTYPES, **EXTRA_PROTOTYPES})


def check(rc: int, exc=FlashQuestError):
    if rc != 0:
        msg = lib().fq_last_error_string().decode()
        if rc in (-1, -4) and exc is FlashQuestError:
            exc = ValueError if rc == -1 else NotImplementedError
        raise exc(msg)


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float32, float16 or bfloat16") from None


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise FlashQuestError("flashquest_b200 operators take CUDA tensors (no CPU path)")


def ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def stream_ptr(device=None):
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def inner_contiguous(t: torch.Tensor) -> torch.Tensor:
    """Strided views are taken as they are as long as the last dimension is dense."""
    if t.dim() > 0 and t.shape[-1] > 1 and t.stride(-1) != 1:
        return t.contiguous()
    return t
