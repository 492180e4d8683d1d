"""CPU oracle for the sparse-decode path.  TEST INFRASTRUCTURE ONLY.

A plain-C restatement (``fq_oracle.c``) of the reference's eager arithmetic, wrapped for
torch CPU tensors with the reference's own function names so the parity tests read like
the reference's tests.  Only ``tests/``, the smoke check and the benchmark's CPU-baseline
leg may import this package; the product package never does.
"""
from .oracle import *  # noqa: F401,F403
from .oracle import build_oracle, lib_path  # noqa: F401
