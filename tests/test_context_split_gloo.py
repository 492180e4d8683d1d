"""Context split over 2 (and 3) CPU ranks with the gloo backend: the exchange protocol with the
oracle as the local primitive must reproduce the single-process page set and attention output."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle
from tests._util import make_kv, make_q


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _ops(use_compact=False):
    from flashquest_b200.eager.context_split import ContextSplitOps

    def top_k_mask(scores, k):
        return oracle.select_pages_vectorized(scores, 1.0, 0, 0, k_max_static=k)

    def merge(O_parts, lse_parts):
        return oracle.lse_merge(O_parts, lse_parts)

    return ContextSplitOps(top_k_mask=top_k_mask, merge=merge,
                           compact=oracle.build_compact_selection if use_compact else None)


def _worker(rank, world, port, case, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flashquest_b200.eager import context_split as cs
        oracle.set_num_threads(1)
        B, Hq, Hkv, S, D, page, retention, sinks, window, ties = case
        P = S // page
        k = make_kv(7, (B, Hkv, S, D), torch.float16)
        v = make_kv(9, (B, Hkv, S, D), torch.float16)
        q = make_q(8, (B, Hq, 1, D), torch.float16)
        Kp, Ks, Km = oracle.quantize_k_int4(k, page)
        Vp, Vs, Vm = oracle.quantize_v_int4(v)
        scores = oracle.page_scores_int4_fast(q, Ks, Km)                     # (B,Hq,1,P)
        if ties == "inf":
            # -inf and NaN scores: a page whose score is -inf must still beat an empty candidate slot of a rank
            # that has fewer pages than slots, and a NaN ranks above everything (as in torch.topk)
            scores = scores.clone()
            scores[..., 3:] = float("-inf")
            scores[..., 1] = float("nan")
        elif ties:
            scores = (scores * 2).round() / 2                                # many equal scores
        ref_mask = oracle.select_pages_vectorized(scores, retention, sinks, window)
        lo, hi = cs.page_range(rank, world, P)
        ops = _ops(use_compact=(world == 3))      # 3 ranks: candidate ids from the compact list; 2 ranks: from the sort
        mask = cs.select_pages_context_split(scores[..., lo:hi].contiguous(), P_global=P, retention=retention,
                                             num_sinks=sinks, window_pages=window, ops=ops)
        ok_mask = torch.equal(mask, ref_mask[..., lo:hi])
        # local attention over the local page range, then the merge
        sl = slice(lo * page, hi * page)
        bucket = max(1, hi - lo)
        compact = oracle.build_compact_selection(mask, bucket)
        sm = 1.0 / D ** 0.5
        O_r, lse_r = oracle.sparse_attn_int4(q, Kp[:, :, sl].contiguous(), Ks[:, :, lo:hi].contiguous(),
                                             Km[:, :, lo:hi].contiguous(), Vp[:, :, sl].contiguous(),
                                             Vs[:, :, sl].contiguous(), Vm[:, :, sl].contiguous(),
                                             selected_page_ids=compact, page_size=page, sm_scale=sm)
        O, lse = cs.merge_context_split(O_r, lse_r, ops=ops)
        ref_compact = oracle.build_compact_selection(ref_mask, P)
        O_ref, lse_ref = oracle.sparse_attn_int4(q, Kp, Ks, Km, Vp, Vs, Vm, selected_page_ids=ref_compact, page_size=page, sm_scale=sm)
        err = (O.float() - O_ref.float()).abs().max().item()
        err_l = (lse.float() - lse_ref.float()).abs().max().item()
        out_q.put((rank, ok_mask, err, err_l, int(mask.sum())))
    finally:
        dist.destroy_process_group()


CASES = [
    # B, Hq, Hkv, S, D, page, retention, sinks, window, ties
    (1, 4, 2, 1024, 64, 16, 0.25, 1, 1, False),
    (2, 4, 2, 800, 64, 16, 0.5, 4, 2, True),       # P = 50 does not divide by 3; forced pages span ranks
    (1, 2, 1, 256, 64, 16, 1.0, 0, 0, False),      # everything selected
    (1, 2, 1, 256, 64, 16, 0.0, 2, 1, True),       # only forced pages: most ranks attend nothing
    (1, 2, 1, 112, 64, 16, 0.7, 0, 0, "inf"),      # P = 7, k = 5: more slots than pages on one rank, -inf and NaN scores
]


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("case", CASES)
def test_context_split_matches_single_process(world, case):
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = sorted(out_q.get(timeout=5) for _ in range(world))
    for rank, ok_mask, err, err_l, _ in results:
        assert ok_mask, f"rank {rank}: local mask differs from the single-process mask"
        assert err <= 1e-5 and err_l <= 1e-5, (rank, err, err_l)


def test_page_range_and_k():
    from flashquest_b200.eager import context_split as cs
    for P in (0, 1, 7, 50, 2048):
        for G in (1, 2, 3, 8):
            r = [cs.page_range(i, G, P) for i in range(G)]
            assert r[0][0] == 0 and r[-1][1] == P
            assert all(r[i][1] == r[i + 1][0] for i in range(G - 1))
    assert cs.global_k(0.25, 2048) == 512
    assert cs.global_k(0.2, 2048) == int(oracle.k_per_head(0.2, 1, 2048)[0])
    assert cs.global_k(1.0, 10, 4) == 4
    with pytest.raises(ValueError):
        cs.global_k(1.5, 10)
