"""DuoAttention head patterns — counterpart of flashquest/duo/pattern.py:16-49.

A pattern file is tab-separated text: one line per layer, one field per KV head, each field the
probability in [0, 1] that the head needs full retrieval attention.  Thresholded, it becomes the
`head_pattern` argument of patch_llama_for_quest_persistent: True marks a retrieval head (keeps
`retention` of the pages), False a streaming head (attention sinks and the recent window only, which
the selection kernel gets as a per-head retention of 0).
"""
from __future__ import annotations

import os

import torch


def _parse_fields(text: str, where: str) -> list:
    """Non-blank lines of `text` as lists of floats; every line must have as many fields as the first."""
    table = []
    for number, raw in enumerate(text.splitlines(), start=1):
        fields = [f for f in raw.strip().split("\t") if f]
        if not fields:
            continue
        if table and len(fields) != len(table[0]):
            raise ValueError(
                f"DuoAttention pattern at {where}:{number} has {len(fields)} cols, expected {len(table[0])}")
        table.append([float(f) for f in fields])
    return table


def load_duo_pattern(path, threshold: float = 0.5) -> torch.Tensor:
    """(num_layers, num_kv_heads) bool tensor on the CPU; probabilities >= threshold are retrieval heads.

    FileNotFoundError when `path` is no file; ValueError for an empty file or a ragged line."""
    where = os.fspath(path)
    if not os.path.isfile(where):
        raise FileNotFoundError(f"DuoAttention pattern not found: {where}")
    with open(where, "r") as handle:
        table = _parse_fields(handle.read(), where)
    if len(table) == 0:
        raise ValueError(f"DuoAttention pattern at {where} is empty")
    probabilities = torch.tensor(table, dtype=torch.float32)
    return probabilities.ge(threshold)
