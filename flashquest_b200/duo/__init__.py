"""DuoAttention head patterns (flashquest/duo/__init__.py); the per-head retrieval / streaming split
itself is the `head_pattern` argument of patch_llama_for_quest_persistent."""
from .pattern import load_duo_pattern

__all__ = ["load_duo_pattern"]
