"""Normalised Walsh-Hadamard transform along the last dimension — CUDA counterpart of
flashquest/kernel/wht.py:17-41 (bit-identical, dtype preserved, self-inverse)."""
from __future__ import annotations

import torch

from .._lib import check, dtype_code, lib, ptr, require_cuda, stream_ptr


def wht_along_head_dim(x: torch.Tensor) -> torch.Tensor:
    D = x.shape[-1]
    if D & (D - 1) != 0 or D == 0:
        raise ValueError(f"head_dim must be a positive power of 2, got {D}")
    require_cuda(x)
    xc = x.contiguous()
    out = torch.empty_like(xc)
    with torch.cuda.device(x.device):
        check(lib().fq_wht(ptr(xc), ptr(out), dtype_code(xc), xc.numel() // D, D, stream_ptr(x.device)))
    return out
