"""flashquest_b200 — B200 (sm_100a) kernels for flashquest's sparse-decode hot path.

The sub-packages mirror the reference's module layout so that imports translate one to one:

    flashquest.kernel.kv_quant          -> flashquest_b200.kernel.kv_quant
    flashquest.eager.criticality        -> flashquest_b200.eager.criticality
    flashquest.eager.selection          -> flashquest_b200.eager.selection
    flashquest.kernel.sparse_int4_fwd*  -> flashquest_b200.kernel.sparse_int4_fwd*
    flashquest.cache.persistent_int4    -> flashquest_b200.cache.persistent_int4

Every function launches hand-written CUDA through the C ABI in include/flashquest_b200.h;
nothing here computes on the CPU.
"""
from ._lib import FlashQuestError, LIB_PATH, lib  # noqa: F401

__version__ = "0.1.0"
