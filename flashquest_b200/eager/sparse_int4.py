"""Public alias of the INT4 sparse decode kernel (flashquest/eager/sparse_int4.py:12-24)."""
from ..kernel.sparse_int4_fwd import flash_attn_sparse_int4_fwd


def quest_sparse_int4_fwd(Q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn, *, selection_mask,
                          page_size: int = 64, sm_scale=None, return_lse: bool = True):
    return flash_attn_sparse_int4_fwd(Q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn,
                                      selection_mask=selection_mask, page_size=page_size,
                                      sm_scale=sm_scale, return_lse=return_lse)
