"""The shared library loads without a GPU and exports every function the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "flashquest_b200.h")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = _declared()
    for want in ("fq_quantize_kv_int4", "fq_page_scores_int4", "fq_select_pages", "fq_build_compact",
                 "fq_sparse_decode_int4", "fq_sparse_decode_turbo", "fq_lse_merge", "fq_awq_gemv"):
        assert want in names


def test_library_exports_every_declared_symbol():
    from flashquest_b200 import build
    path = build.LIB
    if not os.path.exists(path):
        pytest.skip("library not built (python -m flashquest_b200.build)")
    so = ctypes.CDLL(path)
    missing = [n for n in _declared() if not hasattr(so, n)]
    assert not missing, missing


def test_bindings_cover_the_header():
    from flashquest_b200 import _lib
    assert sorted(_lib._PROTOTYPES) == _declared()


def test_host_only_entry_points_answer_without_a_gpu():
    from flashquest_b200 import build
    path = build.LIB
    if not os.path.exists(path):
        pytest.skip("library not built")
    so = ctypes.CDLL(path)
    so.fq_version.restype = ctypes.c_char_p
    assert so.fq_version()
    assert so.fq_awq_gemv_default_splits(3072, 5120, 128) in (1, 2, 4, 8)
    assert so.fq_awq_gemv_default_splits(64, 256, 64) == 1          # one group: nothing to split
    # split count of the sparse decode attention (444 CTA slots on a B200): one full wave at batch 1; three times the
    # CTAs when a single wave would leave more than 7 % of the slots empty and a CTA keeps 8 iterations; one per row
    # beyond that; never more splits than list entries
    splits = so.fq_sparse_decode_default_splits
    assert splits(1, 24, 514, 16) == 18
    assert splits(16, 24, 514, 16) == 3 and splits(16, 24, 1026, 16) == 3
    assert splits(8, 24, 514, 16) == 2 and splits(4, 24, 514, 16) == 4
    assert splits(64, 24, 514, 16) == 1
    assert splits(1, 24, 3, 16) == 1 and splits(1, 1, 5, 64) <= 5
    assert splits(0, 24, 514, 16) == 1
    so.fq_sparse_decode_workspace_bytes.restype = ctypes.c_size_t
    assert so.fq_sparse_decode_workspace_bytes(1, 24, 128, 18) >= 24 * 18 * 130 * 4
