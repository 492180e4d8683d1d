"""Context split of ONE long sequence over the ranks of a process group (one process per GPU).

Not in the reference (it is single-GPU): the pages of a sequence are split by contiguous range,
rank r owns pages [r*P/G, (r+1)*P/G) with their packed codes and metadata, Q is replicated.
One decode step of one layer is then

  1. page scores of the local pages (local kernel);
  2. exact global top-k: every rank takes its local top-min(k, P_local) pages (same order as
     the single-GPU selection: score descending, lower page index first), all ranks all-gather
     the candidates' (score, global page id), and every rank runs the same top-k over the
     gathered candidates, laid out in ascending global page id so that ties resolve as on one
     GPU; a rank keeps the winners that fall in its range, plus its share of the forced sink
     and window pages.  The union over the ranks is identical to the single-GPU page set;
  3. sparse attention over the local selection -> (O_r, lse_r); all-gather of those
     (H_q*(D+1) values per rank) and an n-way LSE merge on every rank.

Both exchanges arrive in the rank's own memory through the collective before any kernel reads
them.  The three local primitives are injectable (`ops`), which is how the protocol is tested
on CPU ranks with the `gloo` backend.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Callable, Optional

import numpy as np
import torch
import torch.distributed as dist


def page_range(rank: int, world: int, P: int) -> tuple[int, int]:
    """Pages [lo, hi) owned by `rank` when P pages are split over `world` ranks."""
    return rank * P // world, (rank + 1) * P // world


def global_k(retention: float, P: int, k_max_static: Optional[int] = None) -> int:
    """k of the single-GPU selection (flashquest/eager/selection.py:92-103):
    clamp(ceil(fp32(retention) * P), 0, P), capped by the static k_max."""
    if not (0.0 <= retention <= 1.0):
        raise ValueError(f"scalar retention must be in [0, 1]; got {retention}")
    k = int(np.ceil(np.float32(retention) * np.float32(P)))
    k = max(0, min(k, P))
    return k if k_max_static is None else min(k, int(k_max_static))


@dataclass
class ContextSplitOps:
    """Local primitives.  top_k_mask(scores (B,H,1,P) fp32, k) -> bool (B,H,1,P), ties to the lower
    index; merge(O_parts (n,B,H,1,D), lse_parts (n,B,H,1)) -> (O, lse)."""
    top_k_mask: Callable
    merge: Callable
    compact: Optional[Callable] = None     # compact(mask (B,H,1,P) bool, bucket) -> (B,H,1,bucket) int32 descending ids, -1 padded


def cuda_ops() -> ContextSplitOps:
    from .selection import build_compact_selection, select_pages_vectorized
    from .tail_merge import merge_attentions

    def top_k_mask(scores, k):
        return select_pages_vectorized(scores, 1.0, 0, 0, k_max_static=k)

    return ContextSplitOps(top_k_mask=top_k_mask, merge=merge_attentions, compact=build_compact_selection)


def _all_gather(t: torch.Tensor, group) -> torch.Tensor:
    """(world, *t.shape): one collective into one preallocated tensor where the backend has it."""
    world = dist.get_world_size(group)
    t = t.contiguous()
    out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    try:
        dist.all_gather_into_tensor(out, t, group=group)
    except (RuntimeError, NotImplementedError):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t, group=group)
        out = torch.stack(parts)
    return out


def select_pages_context_split(scores_local: torch.Tensor, *, P_global: int, retention: float, num_sinks: int,
                               window_pages: int, k_max_static: Optional[int] = None, group=None,
                               ops: Optional[ContextSplitOps] = None) -> torch.Tensor:
    """scores_local (B,H,1,P_local) fp32: scores of this rank's page range.  Returns the bool
    mask (B,H,1,P_local) that equals the slice of the single-GPU mask for this range."""
    ops = ops or cuda_ops()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    lo, hi = page_range(rank, world, P_global)
    B, H, S_q, P_local = scores_local.shape
    if S_q != 1:
        raise NotImplementedError(f"select_pages_context_split: decode-only (S_q={S_q})")
    if P_local != hi - lo:
        raise ValueError(f"rank {rank} owns pages [{lo},{hi}) but got {P_local} local scores")
    dev = scores_local.device
    k = global_k(float(retention), P_global, k_max_static)
    # every rank contributes the same number of candidate slots so that the gather is regular
    k_c = min(k, max(page_range(r, world, P_global)[1] - page_range(r, world, P_global)[0] for r in range(world)))
    mask = torch.zeros(B, H, 1, P_local, dtype=torch.bool, device=dev)
    if k > 0 and k_c > 0:
        scores_local = scores_local.float()
        cand = torch.full((B, H, 2, k_c), float("-inf"), dtype=torch.float32, device=dev)
        ids = torch.full((B, H, k_c), -1, dtype=torch.int32, device=dev)
        if P_local > 0:
            n_c = min(k_c, P_local)
            local_mask4 = ops.top_k_mask(scores_local, n_c)                                   # (B,H,1,P_local), exactly n_c set
            if ops.compact is not None:
                # the compact list is descending: reversed it is the ascending ids of the candidates
                order = ops.compact(local_mask4, n_c)[:, :, 0].flip(-1).long()
            else:
                # stable sort of "not selected" keeps page order
                order = torch.sort((~local_mask4[:, :, 0]).to(torch.uint8), dim=-1, stable=True).indices[..., :n_c]
            cand[:, :, 0, :n_c] = torch.gather(scores_local[:, :, 0], -1, order)
            ids[:, :, :n_c] = (order + lo).to(torch.int32)
        cand[:, :, 1] = ids.view(torch.float32)                    # page ids travel bit-cast in the same message
        gathered = _all_gather(cand, group)                        # (G,B,H,2,k_c), rank-major = ascending page id
        g_scores = gathered[:, :, :, 0].permute(1, 2, 0, 3).reshape(B, H, world * k_c)
        g_ids = gathered[:, :, :, 1].contiguous().view(torch.int32).permute(1, 2, 0, 3).reshape(B, H, world * k_c)
        # padding slots (id -1, score -inf) go behind every real candidate, keeping the ascending page order of
        # the rest: a page whose real score is -inf must win a tie against a slot that holds no page
        order = torch.sort((g_ids < 0).to(torch.uint8), dim=-1, stable=True).indices
        g_scores = torch.gather(g_scores, -1, order).unsqueeze(2).contiguous()
        g_ids = torch.gather(g_ids, -1, order)
        win = ops.top_k_mask(g_scores, min(k, world * k_c))[:, :, 0]                           # (B,H,G*k_c)
        mine = win & (g_ids >= lo) & (g_ids < hi)
        # winners of other ranks go to a spare column past the end
        buf = torch.zeros(B, H, P_local + 1, dtype=torch.bool, device=dev)
        idx = torch.where(mine, g_ids.long() - lo, torch.full_like(g_ids, P_local, dtype=torch.long))
        buf.scatter_(-1, idx, mine)
        mask = buf[..., :P_local].unsqueeze(2).contiguous()
    return _force_pages(mask, lo, hi, P_global, num_sinks, window_pages)


def _force_pages(mask, lo, hi, P_global, num_sinks, window_pages):
    ns = min(int(num_sinks), P_global)
    if ns > lo:
        mask[..., : min(ns, hi) - lo] = True
    w0 = P_global - min(int(window_pages), P_global)
    if hi > w0:
        mask[..., max(w0, lo) - lo:] = True
    return mask


def merge_context_split(O_local: torch.Tensor, lse_local: torch.Tensor, *, group=None,
                        ops: Optional[ContextSplitOps] = None):
    """All-gather of every rank's (O (B,H,1,D), lse (B,H,1)) and n-way LSE merge; a rank with
    nothing selected contributes lse = -inf.  One message per rank: lse rides as an extra column."""
    ops = ops or cuda_ops()
    msg = torch.cat([O_local.float(), lse_local.float().unsqueeze(-1)], dim=-1)
    parts = _all_gather(msg, group)                               # (G,B,H,1,D+1)
    O, lse = ops.merge(parts[..., :-1].to(O_local.dtype).contiguous(), parts[..., -1].contiguous())
    return O, lse


def decode_context_split_int4(Q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn, *, P_global: int, page_size: int,
                              retention: float, num_sinks: int, window_pages: int, k_max_static: Optional[int] = None,
                              sm_scale: Optional[float] = None, K_partial=None, V_partial=None, group=None,
                              timings: Optional[dict] = None):
    """One decode step of one layer for a sequence whose pages are split over the group.

    The K/V tensors are this rank's page range only (layout as in the single-GPU call,
    S_local = P_local * page_size); Q (B,H_q,1,D) is the same on every rank; the staged tail
    (K_partial / V_partial) is passed on the last rank only.  Returns (O (B,H_q,1,D), lse (B,H_q,1)),
    identical on every rank.  With `timings` (a dict) CUDA events around the two exchanges are
    recorded so that the collective time can be reported apart from the kernels."""
    from ..kernel.sparse_int4_fwd_compact import flash_attn_sparse_int4_fwd_compact
    from .criticality import page_scores_int4_fast
    from .selection import build_compact_selection

    def mark(name):
        if timings is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            timings.setdefault(name, []).append(ev)

    P_local = K_scale.shape[2]
    B, H_q = Q.shape[0], Q.shape[1]
    mark("start")
    if P_local > 0:
        scores = page_scores_int4_fast(Q, K_scale, K_mn)
    else:
        scores = torch.empty(B, H_q, 1, 0, dtype=torch.float32, device=Q.device)
    mark("scored")
    mask = select_pages_context_split(scores, P_global=P_global, retention=retention, num_sinks=num_sinks,
                                      window_pages=window_pages, k_max_static=k_max_static, group=group)
    mark("selected")
    bucket = max(1, min(P_local, global_k(float(retention), P_global, k_max_static) + int(num_sinks) + int(window_pages)))
    if P_local > 0:
        compact = build_compact_selection(mask, bucket)
    else:
        compact = torch.full((B, H_q, 1, 1), -1, dtype=torch.int32, device=Q.device)
    O_r, lse_r = flash_attn_sparse_int4_fwd_compact(
        Q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn, selected_page_ids=compact, page_size=page_size,
        sm_scale=sm_scale, return_lse=True, K_partial=K_partial, V_partial=V_partial)
    mark("attended")
    out = merge_context_split(O_r, lse_r, group=group)
    mark("merged")
    return out


class ContextSplitInt4:
    """The same decode step with everything preallocated and the device work in three foreign calls
    (fq_ctx_local_candidates, fq_ctx_select_attend, fq_lse_merge_strided) around the two all-gathers,
    so that a whole layer-step — collectives included — can be captured in ONE CUDA graph and
    replayed without host work.  Scalar retention only.  One instance serves one (shape, group)."""

    def __init__(self, *, batch_size: int, num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, P_global: int,
                 retention: float, num_sinks: int, window_pages: int, k_max_static: Optional[int] = None,
                 q_dtype=torch.float16, group=None, device=None, n_split: Optional[int] = None):
        from .._lib import lib
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.B, self.Hq, self.Hkv, self.D, self.page = batch_size, num_q_heads, num_kv_heads, head_dim, page_size
        self.P_global, self.sinks, self.window = int(P_global), int(num_sinks), int(window_pages)
        self.lo, self.hi = page_range(self.rank, self.world, self.P_global)
        self.P_local = self.hi - self.lo
        self.k = global_k(float(retention), self.P_global, k_max_static)
        p_max = max(page_range(r, self.world, self.P_global)[1] - page_range(r, self.world, self.P_global)[0] for r in range(self.world))
        self.k_c = max(1, min(self.k, p_max))
        self.bucket_local = max(1, min(self.P_local, self.k + self.sinks + self.window))
        dev = torch.device(device if device is not None else torch.cuda.current_device())
        self.device, self.q_dtype = dev, q_dtype
        self.sm_scale = 1.0 / math.sqrt(head_dim)
        rows = batch_size * num_q_heads
        L = lib()
        with torch.cuda.device(dev):
            self.n_split = n_split or L.fq_sparse_decode_default_splits(batch_size, num_q_heads, self.bucket_local, page_size)
            self.scratch = torch.empty(L.fq_ctx_scratch_bytes(batch_size, num_q_heads, self.world, self.k_c, self.P_local, self.bucket_local),
                                       dtype=torch.uint8, device=dev)
            self.workspace = torch.zeros(max(L.fq_sparse_decode_workspace_bytes(batch_size, num_q_heads, head_dim, self.n_split), 256),
                                         dtype=torch.uint8, device=dev)
        self.msg = torch.empty(batch_size, num_q_heads, 2, self.k_c, dtype=torch.float32, device=dev)
        self.gathered = torch.empty(self.world, batch_size, num_q_heads, 2, self.k_c, dtype=torch.float32, device=dev)
        self.o_bytes = rows * head_dim * 2
        self.msg2 = torch.empty(self.o_bytes + rows * 4, dtype=torch.uint8, device=dev)
        self.gathered2 = torch.empty(self.world, self.msg2.numel(), dtype=torch.uint8, device=dev)
        self.O = torch.empty(batch_size, num_q_heads, head_dim, dtype=q_dtype, device=dev)
        self.lse = torch.empty(batch_size, num_q_heads, dtype=torch.float32, device=dev)

    def step(self, q, K_packed, K_scale, K_mn, V_packed, V_scale, V_mn, K_partial=None, V_partial=None, marks=None):
        """q (B,H_q,1,D) (same on every rank); K/V tensors: this rank's page range, laid out as for
        flash_attn_sparse_int4_fwd_compact (contiguous; V_scale / V_mn (B,H_kv,S_local[,1])); the staged tail on
        the last rank only.  Returns (O (B,H_q,1,D), lse (B,H_q,1)), identical on every rank.  `marks`: an
        optional callable(name) invoked between the phases (e.g. to record CUDA events)."""
        from .._lib import check, dtype_code, lib, ptr, stream_ptr
        L = lib()
        st = stream_ptr(self.device)
        B, Hq, Hkv, D = self.B, self.Hq, self.Hkv, self.D
        q3 = q.reshape(B, Hq, D)
        if q3.dtype != self.q_dtype or not q3.is_contiguous():
            q3 = q3.to(self.q_dtype).contiguous()
        Vs = V_scale.squeeze(-1) if V_scale.dim() == 4 else V_scale
        Vm = V_mn.squeeze(-1) if V_mn.dim() == 4 else V_mn
        mark = marks or (lambda name: None)
        mark("start")
        check(L.fq_ctx_local_candidates(
            ptr(q3), dtype_code(q3), q3.stride(0), q3.stride(1), ptr(K_scale), ptr(K_mn), *K_scale.stride()[:3],
            B, Hq, Hkv, self.P_local, D, self.lo, self.k_c, self.world, self.bucket_local,
            ptr(self.scratch), self.scratch.numel(), ptr(self.msg), st))
        mark("candidates")
        dist.all_gather_into_tensor(self.gathered, self.msg, group=self.group)
        mark("gathered")
        tail_len, tl, tcode, Kt, Vt = 0, (0, 0, 0), 2, None, None
        if K_partial is not None and K_partial.shape[2] > 0:
            Kt, Vt = K_partial, V_partial
            if Kt.stride(3) != 1 or Kt.stride() != Vt.stride():
                Kt, Vt = Kt.contiguous(), Vt.contiguous()
            tail_len, tl, tcode = Kt.shape[2], Kt.stride()[:3], dtype_code(Kt)
        lse_ptr = ctypes.c_void_p(self.msg2.data_ptr() + self.o_bytes)
        check(L.fq_ctx_select_attend(
            ptr(self.gathered), self.world, self.k_c, self.k, self.sinks, self.window, self.lo, self.hi, self.P_global,
            ptr(q3), dtype_code(q3), q3.stride(0), q3.stride(1),
            ptr(K_packed), K_packed.stride(0), K_packed.stride(1), ptr(K_scale), ptr(K_mn), *K_scale.stride()[:3],
            ptr(V_packed), V_packed.stride(0), V_packed.stride(1), ptr(Vs), ptr(Vm), Vs.stride(0), Vs.stride(1),
            ptr(Kt), ptr(Vt), tcode, *tl, tail_len,
            B, Hq, Hkv, D, self.page, self.sm_scale, self.bucket_local,
            ptr(self.scratch), self.scratch.numel(), ptr(self.msg2), lse_ptr,
            ptr(self.workspace), self.workspace.numel(), self.n_split, st))
        mark("attended")
        dist.all_gather_into_tensor(self.gathered2, self.msg2, group=self.group)
        mark("gathered2")
        n2 = self.msg2.numel()
        check(L.fq_lse_merge_strided(
            ptr(self.gathered2), n2 // 2, ctypes.c_void_p(self.gathered2.data_ptr() + self.o_bytes), n2 // 4,
            dtype_code(self.O), self.world, B * Hq, D, ptr(self.O), ptr(self.lse), st))
        mark("merged")
        return self.O.unsqueeze(2), self.lse.unsqueeze(2)

    def local_mask(self) -> torch.Tensor:
        """The bool mask (B,H_q,1,P_local) of the pages this rank attended in the last step (a view of the
        scratch buffer; the layout is the one fq_ctx_scratch_bytes sums up)."""
        pad = lambda x: (x + 255) // 256 * 256
        rows, n, pl = self.B * self.Hq, self.world * self.k_c, max(self.P_local, 1)
        off = pad(rows * pl * 4) + pad(rows * self.k_c * 4) + 2 * pad(rows * n * 4) + pad(rows * n)
        return self.scratch[off: off + rows * self.P_local].view(self.B, self.Hq, 1, self.P_local).bool()

    def capture(self, *args, **kwargs):
        """CUDA graph of step(*args) for static input tensors (collectives included); returns replay()
        -> (O, lse).  One ordinary step runs first (lazy kernel attributes, NCCL set-up)."""
        self.step(*args, **kwargs)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            out = self.step(*args, **kwargs)

        def replay():
            graph.replay()
            return out

        replay.graph = graph
        return replay
