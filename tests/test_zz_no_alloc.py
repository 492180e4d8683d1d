"""The workspace-free attention entry point, fq_sparse_decode_int4_static.

Some callers of the C ABI cannot provide device memory at call time: a binding from a
runtime that has no CUDA allocator of its own, a serving loop that keeps away from
cudaMalloc/cudaFree because they stall the device, a plugin that is handed nothing but its
inputs and outputs.  For them the split-K scratch sits in a fixed 4 MiB array inside the
library.  This test drives that entry point straight through ctypes and checks that it
returns what fq_sparse_decode_int4 returns with a caller-provided workspace, twice in a row
(the second call finds the array dirty from the first), that one of the shapes also agrees
with the CPU oracle, and that a request larger than the array is refused.  Collected last on purpose (file name), and independent of the other tests.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
O_TOL, LSE_TOL = 2e-3, 1e-3      # same tolerances as tests/test_gpu_attention_int4.py


def _case(seed, B, Hq, Hkv, S, D, page, bucket):
    from flashquest_b200.kernel.kv_quant import quantize_k_int4, quantize_v_int4
    g = torch.Generator(device="cuda").manual_seed(seed)
    K = torch.randn(B, Hkv, S, D, device="cuda", generator=g).half()
    V = torch.randn(B, Hkv, S, D, device="cuda", generator=g).half()
    Q = torch.randn(B, Hq, D, device="cuda", generator=g).half()
    Kp, Ks, Km = quantize_k_int4(K, page)
    Vp, Vs, Vm = quantize_v_int4(V)
    comp = torch.stack([torch.randperm(S // page, device="cuda", generator=g)[:bucket]
                        for _ in range(B * Hq)]).reshape(B, Hq, bucket).int().contiguous()
    comp[:, :, -2:] = -1                                   # a couple of sentinels
    tail = torch.randn(2, B, Hkv, 5, D, device="cuda", generator=g).half()
    return Q, Kp, Ks, Km, Vp, Vs.squeeze(-1).contiguous(), Vm.squeeze(-1).contiguous(), comp, tail


def _call(lib, static, t, B, Hq, Hkv, S, D, page, n_split, ws=None):
    Q, Kp, Ks, Km, Vp, Vs, Vm, comp, tail = t
    O = torch.empty(B, Hq, D, dtype=torch.float16, device="cuda")
    lse = torch.empty(B, Hq, dtype=torch.float32, device="cuda")
    P = S // page
    vp = ctypes.c_void_p
    common = [vp(Q.data_ptr()), 1, Q.stride(0), Q.stride(1),
              vp(Kp.data_ptr()), Kp.stride(0), Kp.stride(1),
              vp(Ks.data_ptr()), vp(Km.data_ptr()), Ks.stride(0), Ks.stride(1), Ks.stride(2),
              vp(Vp.data_ptr()), Vp.stride(0), Vp.stride(1),
              vp(Vs.data_ptr()), vp(Vm.data_ptr()), Vs.stride(0), Vs.stride(1),
              vp(comp.data_ptr()), comp.stride(0), comp.stride(1), comp.shape[-1],
              vp(tail[0].data_ptr()), vp(tail[1].data_ptr()), 1, tail[0].stride(0), tail[0].stride(1), tail[0].stride(2),
              tail.shape[3],
              B, Hq, Hkv, S, P, D, page, 1.0 / math.sqrt(D),
              vp(O.data_ptr()), O.stride(0), O.stride(1), vp(lse.data_ptr())]
    stream = vp(torch.cuda.current_stream().cuda_stream)
    if static:
        rc = lib.fq_sparse_decode_int4_static(*common, n_split, stream)
    else:
        rc = lib.fq_sparse_decode_int4(*common, vp(ws.data_ptr()), ws.numel(), n_split, stream)
    torch.cuda.synchronize()
    return rc, O, lse


def test_static_scratch_entry_matches_workspace_entry():
    from flashquest_b200 import _lib
    lib = _lib.lib()
    shapes = [  # (B, Hq, Hkv, S, D, page, bucket, n_split): second call uses another layout
        (2, 6, 2, 2048, 128, 16, 60, 4),
        (3, 8, 4, 1024, 128, 16, 40, 7),
    ]
    for i, (B, Hq, Hkv, S, D, page, bucket, n_split) in enumerate(shapes):
        t = _case(100 + i, B, Hq, Hkv, S, D, page, bucket)
        ws = torch.zeros(lib.fq_sparse_decode_workspace_bytes(B, Hq, D, n_split), dtype=torch.uint8, device="cuda")
        rc0, O_ref, lse_ref = _call(lib, False, t, B, Hq, Hkv, S, D, page, n_split, ws)
        assert rc0 == 0, lib.fq_last_error_string()
        for rep in range(2):            # twice in a row on the shared, now dirty, array
            rc, O, lse = _call(lib, True, t, B, Hq, Hkv, S, D, page, n_split)
            assert rc == 0, lib.fq_last_error_string()
            assert (O.float() - O_ref.float()).abs().max().item() <= O_TOL, (i, rep)
            assert (lse - lse_ref).abs().max().item() <= LSE_TOL, (i, rep)
        assert lib.fq_device_status() == 0
        if i == 0:
            # and against the CPU oracle, so that the check does not rest on the other entry point alone
            import oracle
            Q, Kp, Ks, Km, Vp, Vs, Vm, comp, tail = (x.cpu() for x in t)
            Ow, lw = oracle.sparse_attn_int4(Q.unsqueeze(2), Kp, Ks, Km, Vp, Vs.unsqueeze(-1), Vm.unsqueeze(-1),
                                             selected_page_ids=comp.unsqueeze(2), page_size=page,
                                             K_partial=tail[0], V_partial=tail[1])
            err = (O.float().cpu() - Ow.squeeze(2)).abs()
            assert (err <= O_TOL + 2 ** -11 * Ow.squeeze(2).abs()).all(), float(err.max())
            assert (lse.cpu() - lw.squeeze(2)).abs().max().item() <= LSE_TOL
    # default split count (n_split <= 0) also works
    rc, O, lse = _call(lib, True, t, B, Hq, Hkv, S, D, page, 0)
    assert rc == 0 and (O.float() - O_ref.float()).abs().max().item() <= O_TOL


def test_static_scratch_entry_rejects_oversized_requests():
    from flashquest_b200 import _lib
    lib = _lib.lib()
    B, Hq, Hkv, S, D, page, bucket = 2, 6, 2, 2048, 128, 16, 60
    t = _case(7, B, Hq, Hkv, S, D, page, bucket)
    # pretend a batch whose partials cannot fit in 4 MiB; nothing may be launched or written
    big_B = 4096
    assert lib.fq_sparse_decode_workspace_bytes(big_B, Hq, D, 8) > (4 << 20)
    Q, Kp, Ks, Km, Vp, Vs, Vm, comp, tail = t
    rc, _, _ = _call(lib, True, t, big_B, Hq, Hkv, S, D, page, 8)
    assert rc == -6                                        # FQ_ERR_WORKSPACE
    msg = lib.fq_last_error_string().decode()
    assert "built-in array" in msg and "4194304" in msg
    rc, _, _ = _call(lib, True, t, B, Hq, Hkv, S, D, page, 2000)
    assert rc == -1 and "n_split" in lib.fq_last_error_string().decode()
