"""Context split on 2 GPUs (NCCL): page set and attention output equal the single-GPU run.
Skipped on a box with one GPU; the protocol itself is covered on CPU ranks by the gloo tests."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_q):
    import datetime
    import traceback
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    # a short collective timeout: a rank that fails must not leave its peer waiting for minutes
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    try:
        _worker_body(rank, world, out_q, dist)
    except Exception:
        out_q.put((rank + 1000, False, traceback.format_exc(), 0.0))
        raise
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _worker_body(rank, world, out_q, dist):
    if True:
        from flashquest_b200.eager import context_split as cs
        from flashquest_b200.eager.criticality import page_scores_int4_fast
        from flashquest_b200.eager.selection import build_compact_selection, select_pages_vectorized
        from flashquest_b200.kernel.kv_quant import quantize_k_int4, quantize_v_int4
        from flashquest_b200.kernel.sparse_int4_fwd_compact import flash_attn_sparse_int4_fwd_compact
        B, Hq, Hkv, S, D, page = 1, 8, 2, 16 * 1000 + 5, 128, 16
        P = S // page
        g = torch.Generator(device="cuda").manual_seed(3)
        k = torch.randn(B, Hkv, S, D, device="cuda", generator=g).half()
        v = torch.randn(B, Hkv, S, D, device="cuda", generator=g).half()
        q = torch.randn(B, Hq, 1, D, device="cuda", generator=g).half()
        kc, vc = k[:, :, :P * page], v[:, :, :P * page]
        Kp, Ks, Km = quantize_k_int4(kc, page)
        Vp, Vs, Vm = quantize_v_int4(vc)
        kt, vt = k[:, :, P * page:].contiguous(), v[:, :, P * page:].contiguous()
        kw = dict(retention=0.25, num_sinks=1, window_pages=1)
        # single GPU
        scores = page_scores_int4_fast(q, Ks, Km)
        ref_mask = select_pages_vectorized(scores, kw["retention"], 1, 1)
        comp = build_compact_selection(ref_mask, P)
        O_ref, lse_ref = flash_attn_sparse_int4_fwd_compact(q, Kp, Ks, Km, Vp, Vs, Vm, selected_page_ids=comp,
                                                            page_size=page, K_partial=kt, V_partial=vt)
        # context split
        lo, hi = cs.page_range(rank, world, P)
        sl = slice(lo * page, hi * page)
        local_mask = cs.select_pages_context_split(scores[..., lo:hi].contiguous(), P_global=P, **kw)
        last = rank == world - 1
        O, lse = cs.decode_context_split_int4(
            q, Kp[:, :, sl].contiguous(), Ks[:, :, lo:hi].contiguous(), Km[:, :, lo:hi].contiguous(),
            Vp[:, :, sl].contiguous(), Vs[:, :, sl].contiguous(), Vm[:, :, sl].contiguous(),
            P_global=P, page_size=page, K_partial=kt if last else None, V_partial=vt if last else None, **kw)
        torch.cuda.synchronize()
        out_q.put((rank, bool(torch.equal(local_mask, ref_mask[..., lo:hi])),
                   (O.float() - O_ref.float()).abs().max().item(), (lse - lse_ref).abs().max().item()))
        # the preallocated, graph-captured form of the same step
        dec = cs.ContextSplitInt4(batch_size=B, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D, page_size=page, P_global=P,
                                  q_dtype=torch.float16, device="cuda", **kw)
        loc = (q, Kp[:, :, sl].contiguous(), Ks[:, :, lo:hi].contiguous(), Km[:, :, lo:hi].contiguous(),
               Vp[:, :, sl].contiguous(), Vs[:, :, sl].contiguous(), Vm[:, :, sl].contiguous())
        tail = dict(K_partial=kt if last else None, V_partial=vt if last else None)
        O2, lse2 = dec.step(*loc, **tail)
        torch.cuda.synchronize()
        ok2 = bool(torch.equal(dec.local_mask(), ref_mask[..., lo:hi]))
        e2 = ((O2.float() - O_ref.float()).abs().max().item(), (lse2 - lse_ref).abs().max().item())
        replay = dec.capture(*loc, **tail)
        for _ in range(3):
            O3, lse3 = replay()
        torch.cuda.synchronize()
        out_q.put((rank + 100, ok2 and bool(torch.equal(O3, O2)) and bool(torch.equal(lse3, lse2)), e2[0], e2[1]))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_context_split_matches_single_gpu():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in range(4):
            item = out_q.get(timeout=150)
            assert item[0] < 1000, f"rank {item[0] - 1000} raised:\n{item[2]}"
            results.append(item)
        for p in procs:
            p.join(60)
            assert p.exitcode == 0
    finally:
        for p in procs:                      # never leave a worker behind on the GPUs
            if p.is_alive():
                p.kill()
                p.join(10)
    for rank, ok, err, err_l in sorted(results):
        assert ok, f"rank {rank % 100}: {'graph-captured step: page set or replay' if rank >= 100 else 'mask'} differs"
        assert err <= 2e-3 and err_l <= 1e-3, (rank, err, err_l)   # fp16 partial outputs
