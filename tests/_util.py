"""Shared helpers for the parity tests: golden-fixture access and seeded inputs."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def from_bits(a: np.ndarray, dtype=None) -> torch.Tensor:
    """Inverse of the fixture encoding: uint16 arrays hold bf16 bit patterns."""
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    t = torch.from_numpy(a.copy())
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    return t


class Golden:
    """Outputs of the reference implementation, produced by tests/golden/make_golden.py."""

    def __init__(self):
        with open(os.path.join(GOLDEN_DIR, "golden.json")) as f:
            self.meta = json.load(f)
        self._files = {}

    def npz(self, name):
        if name not in self._files:
            self._files[name] = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
        return self._files[name]

    def get(self, file, key, *, as_bool=False, dtype=None):
        a = self.npz(file)[key]
        t = from_bits(a, dtype)
        return t.bool() if as_bool else t


def bit_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Exact equality of the underlying bits (NaN-safe, -0 != +0)."""
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    a, b = a.contiguous().cpu(), b.contiguous().cpu()
    if a.dtype in (torch.bfloat16, torch.float16):
        return torch.equal(a.view(torch.int16), b.view(torch.int16))
    if a.dtype == torch.float32:
        return torch.equal(a.view(torch.int32), b.view(torch.int32))
    return torch.equal(a, b)


def make_kv(seed, shape, dtype, outliers=(3, 17, 64, 100), scale=8.0):
    """K/V ~ N(0,1) from numpy's seeded PCG64 stream; fixed outlier channels scaled."""
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal(shape, dtype=np.float32))
    for c in outliers:
        if c < shape[-1]:
            x[..., c] *= scale
    return x.to(dtype)


def make_q(seed, shape, dtype):
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.standard_normal(shape, dtype=np.float32)).to(dtype)
