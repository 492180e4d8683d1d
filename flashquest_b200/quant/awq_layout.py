"""AWQ tensor layout (AutoAWQ GEMM format) — same constants, shapes and checks as
flashquest/quant/awq_layout.py:13-88, plus a holder for one quantised linear so the
projections can be used without AutoAWQ's module classes."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

AWQ_GROUP_SIZE = 128       # rows of the in-axis that share one scale / zero
AWQ_PACK_FACTOR = 8        # 4-bit codes per int32, packed along the out-axis
AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)   # column held by nibble i of an int32 (AutoAWQ GEMM order)


@dataclass(frozen=True)
class AWQLayout:
    """Shapes of the quantised state of a linear with K inputs and N outputs:
    qweight (K, N/8) int32, scales (K/G, N), qzeros (K/G, N/8) int32."""
    in_features: int
    out_features: int

    @property
    def qweight_shape(self) -> tuple[int, int]:
        return (self.in_features, self.out_features // AWQ_PACK_FACTOR)

    @property
    def scales_shape(self) -> tuple[int, int]:
        return (self.in_features // AWQ_GROUP_SIZE, self.out_features)

    @property
    def qzeros_shape(self) -> tuple[int, int]:
        return (self.in_features // AWQ_GROUP_SIZE, self.out_features // AWQ_PACK_FACTOR)


def assert_awq_layout(layer, in_features: int, out_features: int, *, name: str = "<unnamed>") -> AWQLayout:
    """Raise ValueError unless `layer` carries qweight / scales / qzeros of the AWQ layout
    for (in_features, out_features); returns the layout."""
    expected = AWQLayout(in_features, out_features)
    qw = getattr(layer, "qweight", None)
    sc = getattr(layer, "scales", None)
    qz = getattr(layer, "qzeros", None)
    if qw is None or sc is None or qz is None:
        raise ValueError(f"{name}: layer is not an AutoAWQ-quantized Linear (missing qweight/scales/qzeros)")
    for what, t, want in (("qweight", qw, expected.qweight_shape), ("scales", sc, expected.scales_shape),
                          ("qzeros", qz, expected.qzeros_shape)):
        if tuple(t.shape) != want:
            raise ValueError(f"{name}: {what} shape {tuple(t.shape)} != expected {want}")
    if qw.dtype != torch.int32:
        raise ValueError(f"{name}: qweight dtype {qw.dtype} != int32")
    if qz.dtype != torch.int32:
        raise ValueError(f"{name}: qzeros dtype {qz.dtype} != int32")
    return expected


class AWQLinear:
    """Quantised state of one linear: the attributes an AutoAWQ `WQLinear_GEMM` exposes
    (qweight, scales, qzeros, bias, in_features, out_features, group_size).  Calling it runs
    the W4A16 GEMV for up to 8 rows."""

    def __init__(self, qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor,
                 bias: Optional[torch.Tensor] = None, group_size: int = AWQ_GROUP_SIZE, interleaved: bool = True):
        self.qweight, self.scales, self.qzeros, self.bias = qweight, scales, qzeros, bias
        self.in_features = qweight.shape[0]
        self.out_features = qweight.shape[1] * AWQ_PACK_FACTOR
        self.group_size = group_size
        self.interleaved = interleaved

    def __call__(self, hidden: torch.Tensor) -> torch.Tensor:
        from ..kernel.fused_proj import awq_gemv_fused
        return awq_gemv_fused(hidden, (self,))[0]
