"""Generate golden fixtures by running the REFERENCE implementation on CPU.

Run once, in a container that has the reference checkout (it is never needed at test
time):

    python tests/golden/make_golden.py --reference /path/to/flashquest

The reference's eager functions are imported from ``<reference>/src`` and
``<reference>/scripts/profile_contribution.py`` and executed on seeded CPU tensors; inputs
and outputs are written to ``tests/golden/*.npz`` (bf16 tensors as their uint16 bit
patterns).  One shim is needed: ``kernel/kv_quant.py`` creates its codebook with
``device="cuda"`` at import time, which is redirected to the CPU while importing.

``golden.json`` also holds the literal known-answer vectors found in the
reference's own test files (cited there), copied by hand.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import json
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(root: str):
    sys.path.insert(0, os.path.join(root, "src"))
    real_tensor = torch.tensor

    def cpu_tensor(*a, **kw):
        if str(kw.get("device", "cpu")).startswith("cuda"):
            kw["device"] = "cpu"
        return real_tensor(*a, **kw)

    torch.tensor = cpu_tensor
    try:
        import flashquest.kernel.kv_quant as kvq
    finally:
        torch.tensor = real_tensor
    import flashquest.kernel.wht as wht
    import flashquest.eager.criticality as crit
    import flashquest.eager.selection as sel
    sys.path.insert(0, os.path.join(root, "scripts"))  # profile_contribution imports its siblings
    spec = importlib.util.spec_from_file_location(
        "profile_contribution", os.path.join(root, "scripts", "profile_contribution.py"))
    pc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(pc)
    patch = None
    turbo = None
    try:
        import flashquest.eager.llama_persistent_patch as patch  # noqa: F811
        import flashquest.kernel.sparse_turbo_fwd as turbo  # noqa: F811
    except Exception as e:  # transformers / triton import trouble: tail+turbo goldens skipped
        print("WARNING: could not import dispatcher/turbo modules:", repr(e))
    return kvq, wht, crit, sel, pc, patch, turbo


def bits(t: torch.Tensor) -> np.ndarray:
    """numpy view of a tensor; bf16 -> uint16 bit pattern."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype == torch.bool:
        return t.numpy().astype(np.uint8)
    return t.numpy().copy()


def make_kv(gen, shape, dtype, outlier_channels=(3, 17, 64, 100), const_channel=None):
    x = torch.randn(shape, generator=gen, dtype=torch.float32)
    D = shape[-1]
    for c in outlier_channels:
        if c < D:
            x[..., c] *= 8.0
    if const_channel is not None and const_channel < D:
        x[..., const_channel] = 0.75
    return x.to(dtype)


def golden_quant(ref, out):
    kvq, wht = ref[0], ref[1]
    cases = []
    cfgs = [
        ("bf16_p16", torch.bfloat16, (2, 2, 80, 128), 16),
        ("fp16_p16", torch.float16, (2, 2, 80, 128), 16),
        ("fp32_p16", torch.float32, (1, 2, 48, 128), 16),
        ("bf16_p16_ragged", torch.bfloat16, (1, 2, 75, 128), 16),
        ("fp16_p8_d64", torch.float16, (1, 3, 40, 64), 8),
        ("bf16_p64", torch.bfloat16, (1, 1, 128, 128), 64),
    ]
    for i, (name, dt, shape, page) in enumerate(cfgs):
        g = torch.Generator().manual_seed(100 + i)
        K = make_kv(g, shape, dt, const_channel=5)
        V = make_kv(g, shape, dt, outlier_channels=())
        if name == "bf16_p16":
            K[0, 0, :16, 7] = 0.0      # an all-zero channel in one page: scale hits the eps clamp
            V[0, 0, 3, :] = 1.5        # a constant token: V scale hits the eps clamp
        Kp, Ks, Km = kvq.quantize_k_int4(K, page)
        Vp, Vs, Vm = kvq.quantize_v_int4(V)
        Kd = kvq.dequantize_k_int4(Kp, Ks, Km, page)
        Vd = kvq.dequantize_v_int4(Vp, Vs, Vm)
        out[f"q_{name}_K"] = bits(K)
        out[f"q_{name}_V"] = bits(V)
        out[f"q_{name}_Kp"], out[f"q_{name}_Ks"], out[f"q_{name}_Km"] = bits(Kp), bits(Ks), bits(Km)
        out[f"q_{name}_Vp"], out[f"q_{name}_Vs"], out[f"q_{name}_Vm"] = bits(Vp), bits(Vs), bits(Vm)
        out[f"q_{name}_Kd"], out[f"q_{name}_Vd"] = bits(Kd), bits(Vd)
        cases.append({"name": name, "dtype": str(dt).split(".")[-1], "shape": list(shape), "page": page})
    return cases


def golden_turbo(ref, out):
    kvq, wht = ref[0], ref[1]
    cases = []
    cfgs = [
        ("bf16", torch.bfloat16, (2, 2, 64, 128), 16),
        ("fp16", torch.float16, (1, 2, 48, 128), 16),
        ("fp32", torch.float32, (1, 1, 32, 128), 16),
        ("bf16_d64", torch.bfloat16, (1, 2, 32, 64), 8),
    ]
    for i, (name, dt, shape, page) in enumerate(cfgs):
        g = torch.Generator().manual_seed(200 + i)
        K = make_kv(g, shape, dt)
        # heavy-tailed channels (Student-t, df=3) on 8 dims
        tdims = [1, 9, 20, 33, 47, 58, 61, 63]
        chi = torch.randn((*shape[:-1], 8, 3), generator=g).pow(2).sum(-1) / 3.0
        K = K.float()
        K[..., tdims] = (torch.randn((*shape[:-1], 8), generator=g) / chi.sqrt())
        K = K.to(dt)
        V = make_kv(g, shape, dt, outlier_channels=())
        W = wht.wht_along_head_dim(K)
        Km, Kl, Kst, Ksr, Kmr = kvq.quantize_k_turbo(K, page)
        Vm, Vl, Vst = kvq.quantize_v_turbo(V)
        Kd = kvq.dequantize_k_turbo(Km, Kl, Kst, head_dim=shape[-1])
        out[f"t_{name}_K"], out[f"t_{name}_V"], out[f"t_{name}_W"] = bits(K), bits(V), bits(W)
        out[f"t_{name}_Kmsb"], out[f"t_{name}_Klsb"], out[f"t_{name}_Kst"] = bits(Km), bits(Kl), bits(Kst)
        out[f"t_{name}_Ksr"], out[f"t_{name}_Kmr"] = bits(Ksr), bits(Kmr)
        out[f"t_{name}_Vmsb"], out[f"t_{name}_Vlsb"], out[f"t_{name}_Vst"] = bits(Vm), bits(Vl), bits(Vst)
        out[f"t_{name}_Kd"] = bits(Kd)
        cases.append({"name": name, "dtype": str(dt).split(".")[-1], "shape": list(shape), "page": page})
    return cases


def golden_chain(ref, out):
    """score -> select -> compact -> fp32 attention (+ bf16 tail and LSE merge)."""
    kvq, wht, crit, sel, pc, patch, turbo = ref
    cases = []
    cfgs = [
        # name, dtype, B, Hq, Hkv, S_completed, tail, D, page, retention, sinks, window
        ("c_bf16", torch.bfloat16, 2, 6, 2, 320, 5, 128, 16, 0.25, 1, 1),
        ("c_fp16", torch.float16, 1, 6, 2, 256, 0, 128, 16, 0.25, 1, 1),
        ("c_p64", torch.bfloat16, 1, 4, 2, 512, 63, 128, 64, 0.20, 4, 2),
        ("c_d64", torch.bfloat16, 1, 4, 4, 128, 3, 64, 8, 0.5, 0, 0),
    ]
    for i, (name, dt, B, Hq, Hkv, S, tail, D, page, r, sinks, window) in enumerate(cfgs):
        g = torch.Generator().manual_seed(300 + i)
        K = make_kv(g, (B, Hkv, S + tail, D), dt)
        V = make_kv(g, (B, Hkv, S + tail, D), dt, outlier_channels=())
        Q = torch.randn((B, Hq, 1, D), generator=g).to(dt)
        Kp, Ks, Km = kvq.quantize_k_int4(K[:, :, :S], page)
        Vp, Vs, Vm = kvq.quantize_v_int4(V[:, :, :S])
        P = S // page
        scores = crit.page_scores_int4_fast(Q, Ks, Km)
        k_max_static = math.ceil(r * ((S + 64) // page))
        mask = sel.select_pages_vectorized(scores, r, sinks, window, k_max_static=k_max_static)
        bucket = k_max_static + sinks + window
        comp = sel.build_compact_selection(mask, bucket)
        # per-head retention variant (retention 0 on odd heads)
        r_head = torch.tensor([r if h % 2 == 0 else 0.0 for h in range(Hq)])
        mask_ph = sel.select_pages_vectorized(scores, r_head, sinks, window)
        Kx = pc.exact_dequant(Kp, Ks, Km, page_size=page)
        Vx = pc.exact_dequant(Vp, Vs, Vm)
        tmask = pc.token_mask(mask, S, 0, page)
        O, lse = pc.exact_attention(Q, Kx, Vx, tmask)
        # fp32 oracle over completed pages + the raw tail tokens in one softmax
        if tail:
            Kall = torch.cat([Kx, K[:, :, S:].float()], dim=2)
            Vall = torch.cat([Vx, V[:, :, S:].float()], dim=2)
            Oall, lse_all = pc.exact_attention(Q, Kall, Vall, pc.token_mask(mask, S, tail, page))
        else:
            Oall, lse_all = O, lse
        for k_, v_ in (("Ktail", K[:, :, S:]), ("Vtail", V[:, :, S:]), ("Q", Q), ("Kp", Kp), ("Ks", Ks), ("Km", Km), ("Vp", Vp),
                       ("Vs", Vs), ("Vm", Vm), ("scores", scores), ("mask", mask), ("comp", comp),
                       ("mask_ph", mask_ph), ("O", O), ("lse", lse), ("Oall", Oall), ("lse_all", lse_all)):
            out[f"{name}_{k_}"] = bits(v_)
        # the reference's own bf16 tail attention + two-way merge (bf16-only dispatcher path)
        if patch is not None and tail and dt == torch.bfloat16:
            Ot, lset = patch._bf16_dense_attn_with_lse(Q, K[:, :, S:], V[:, :, S:])
            Om = patch._merge_two_attentions(O.to(torch.bfloat16), lse, Ot, lset)
            out[f"{name}_Otail"], out[f"{name}_lsetail"], out[f"{name}_Omerged"] = bits(Ot), bits(lset), bits(Om)
        cases.append({"name": name, "dtype": str(dt).split(".")[-1], "B": B, "Hq": Hq, "Hkv": Hkv, "S": S,
                      "tail": tail, "D": D, "page": page, "retention": r, "sinks": sinks, "window": window,
                      "k_max_static": k_max_static, "bucket": bucket})
    return cases


def golden_turbo_attn(ref, out):
    kvq, wht, crit, sel, pc, patch, turbo = ref
    if turbo is None:
        return []
    cases = []
    B, Hq, Hkv, S, D, page = 1, 6, 2, 128, 128, 16
    g = torch.Generator().manual_seed(400)
    K = make_kv(g, (B, Hkv, S, D), torch.bfloat16)
    V = make_kv(g, (B, Hkv, S, D), torch.bfloat16, outlier_channels=())
    Q = torch.randn((B, Hq, 1, D), generator=g).to(torch.bfloat16)
    Km, Kl, Kst, Ksr, Kmr = kvq.quantize_k_turbo(K, page)
    Vm, Vl, Vst = kvq.quantize_v_turbo(V)
    scores = crit.page_scores_int4_fast(Q, Ksr, Kmr)
    mask = sel.select_pages_vectorized(scores, 0.5, 1, 1)
    turbo.K_TURBO_CODEBOOK = kvq.K_TURBO_CODEBOOK
    O, lse = turbo._flash_attn_sparse_turbo_fwd_reference(
        Q, Km, Kl, Kst, Vm, Vl, Vst, selection_mask=mask, page_size=page)
    for k_, v_ in (("K", K), ("V", V), ("Q", Q), ("Kmsb", Km), ("Klsb", Kl), ("Kst", Kst), ("Ksr", Ksr),
                   ("Kmr", Kmr), ("Vmsb", Vm), ("Vlsb", Vl), ("Vst", Vst), ("scores", scores),
                   ("mask", mask), ("O", O), ("lse", lse)):
        out[f"ta_{k_}"] = bits(v_)
    cases.append({"name": "ta", "B": B, "Hq": Hq, "Hkv": Hkv, "S": S, "D": D, "page": page,
                  "retention": 0.5, "sinks": 1, "window": 1})
    return cases


def golden_config0(ref):
    """BASELINE config 0 (S=4096, page 16, 24/8 heads, retention 0.25, 1 sink + 1 window
    page): too large to commit, so inputs come from numpy's PCG64 stream (seeded) and only
    digests + small outputs are stored."""
    kvq, wht, crit, sel, pc, patch, turbo = ref
    res = {}
    for dt_name, dt in (("fp16", torch.float16), ("bf16", torch.bfloat16)):
        rng = np.random.default_rng(0)
        K = torch.from_numpy(rng.standard_normal((1, 8, 4096, 128), dtype=np.float32))
        V = torch.from_numpy(rng.standard_normal((1, 8, 4096, 128), dtype=np.float32))
        Q = torch.from_numpy(rng.standard_normal((1, 24, 1, 128), dtype=np.float32))
        for c in (3, 17, 64, 100):
            K[..., c] *= 8.0
        K, V, Q = K.to(dt), V.to(dt), Q.to(dt)
        Kp, Ks, Km = kvq.quantize_k_int4(K, 16)
        Vp, Vs, Vm = kvq.quantize_v_int4(V)
        scores = crit.page_scores_int4_fast(Q, Ks, Km)
        mask = sel.select_pages_vectorized(scores, 0.25, 1, 1, k_max_static=64)
        Kx = pc.exact_dequant(Kp, Ks, Km, page_size=16)
        Vx = pc.exact_dequant(Vp, Vs, Vm)
        O, lse = pc.exact_attention(Q, Kx, Vx, pc.token_mask(mask, 4096, 0, 16))
        sha = lambda t: hashlib.sha256(bits(t).tobytes()).hexdigest()  # noqa: E731
        # distance of the k-th score to the (k+1)-th per head: how close selection is to a tie
        top = scores.squeeze(2).sort(dim=-1, descending=True).values
        margin = (top[..., 63] - top[..., 64]).min().item()
        res[dt_name] = {
            "input_sha256": {"K": sha(K), "V": sha(V), "Q": sha(Q)},
            "sha256": {"K_packed": sha(Kp), "K_scale": sha(Ks), "K_mn": sha(Km), "V_packed": sha(Vp),
                       "V_scale": sha(Vs), "V_mn": sha(Vm), "mask": sha(mask)},
            "pages_selected_per_head": mask.sum(-1).flatten().tolist(),
            "min_topk_margin": margin,
            "O": O.flatten().tolist(), "lse": lse.flatten().tolist(),
            "scores_head0_first8": scores[0, 0, 0, :8].tolist(),
        }
    return res


HANDWRITTEN = {
    # tests/test_profile_contribution.py:20-28 — bytes -> codes, low nibble = even channel
    "nibble_unpack": {"bytes": [[0xF0, 0xA5], [0x21, 0x43]],
                      "codes": [[0, 15, 5, 10], [1, 2, 3, 4]]},
    # tests/test_kv_quant_int4.py:26-31 — high bits of the inputs are masked off when packing
    "pack_masks_high": {"input": [0, 15, 16, 255], "unpacked": [0, 15, 0, 15]},
    # tests/test_eager_selection.py:22-44
    "select_zero_retention": {"P": 8, "retention": 0.0, "sinks": 1, "window": 2,
                              "mask": [1, 0, 0, 0, 0, 0, 1, 1]},
    "select_topk": {"scores": [0.1, 0.9, 0.2, 0.8, 0.3, 0.7], "retention": 0.5,
                    "mask": [0, 1, 0, 1, 0, 1]},
    "select_round_up": {"scores": [0.1, 0.4, 0.2, 0.3], "retention": 0.1, "mask": [0, 1, 0, 0]},
    # tests/test_build_compact_selection.py:10-72
    "compact_basic": {"P": 8, "selected": [1, 3, 5], "buckets": [4, 8, 16]},
    "compact_small_P": {"mask": [1, 0, 1, 1], "bucket": 8, "selected": [0, 2, 3]},
    # kernel/kv_quant.py:225-229 and tests/test_kv_quant_turbo.py (codebook symmetry, nearest)
    "turbo_codebook": [-2.1519, -1.3439, -0.7560, -0.2451, 0.2451, 0.7560, 1.3439, 2.1519],
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a flashquest checkout")
    args = ap.parse_args()
    torch.set_num_threads(1)  # one thread: reduction order of the golden run is fixed
    ref = import_reference(args.reference)
    meta = {"torch": torch.__version__, "numpy": np.__version__}
    out = {}
    meta["quant"] = golden_quant(ref, out)
    np.savez_compressed(os.path.join(HERE, "quant_int4.npz"), **out)
    out = {}
    meta["turbo"] = golden_turbo(ref, out)
    meta["turbo_attn"] = golden_turbo_attn(ref, out)
    np.savez_compressed(os.path.join(HERE, "turbo.npz"), **out)
    out = {}
    meta["chain"] = golden_chain(ref, out)
    np.savez_compressed(os.path.join(HERE, "chain.npz"), **out)
    meta["config0"] = golden_config0(ref)
    meta["handwritten"] = HANDWRITTEN
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(meta, f, indent=1)
    for fn in sorted(os.listdir(HERE)):
        print(fn, os.path.getsize(os.path.join(HERE, fn)))


if __name__ == "__main__":
    main()
