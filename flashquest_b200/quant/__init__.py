"""AWQ W4A16 weights: layout constants, a plain holder for a quantised linear."""
from .awq_layout import AWQ_GROUP_SIZE, AWQ_PACK_FACTOR, AWQLayout, AWQLinear, assert_awq_layout

__all__ = ["AWQ_GROUP_SIZE", "AWQ_PACK_FACTOR", "AWQLayout", "AWQLinear", "assert_awq_layout"]
