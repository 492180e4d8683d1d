"""Golden fixtures of the INT8 KV variant, produced by running the REFERENCE on CPU (same recipe and
helpers as make_golden.py; writes tests/golden/int8.npz and int8.json only).

    python tests/golden/make_golden_int8.py --reference /path/to/flashquest
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from make_golden import HERE, bits, import_reference, make_kv


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    torch.set_num_threads(1)
    kvq, wht, crit, sel, pc, patch, turbo = import_reference(args.reference)
    out, cases = {}, []
    cfgs = [("bf16", torch.bfloat16, (2, 2, 70, 64), 16), ("fp16", torch.float16, (1, 2, 64, 128), 16),
            ("fp32", torch.float32, (1, 1, 33, 32), 8), ("bf16_p64", torch.bfloat16, (1, 2, 200, 128), 64)]
    for i, (name, dt, shape, page) in enumerate(cfgs):
        gen = torch.Generator().manual_seed(800 + i)
        K = make_kv(gen, shape, dt, const_channel=5)
        V = make_kv(gen, shape, dt, outlier_channels=())
        Ku, Ks, Km = kvq.quantize_k(K, page)
        Vu, Vs, Vm = kvq.quantize_v(V)
        Kd, Vd = kvq.dequantize_k(Ku, Ks, Km, page), kvq.dequantize_v(Vu, Vs, Vm)
        B, H, S, D = shape
        Q = torch.randn(B, 2 * H, 1, D, generator=gen).to(torch.bfloat16 if dt == torch.float32 else dt)
        sc_fast = crit.page_scores_int8_fast(Q, Ks, Km)
        sc_slow = crit.page_scores_int8(Q, Ks, Km)
        for k, t in (("K", K), ("V", V), ("Ku", Ku), ("Ks", Ks), ("Km", Km), ("Vu", Vu), ("Vs", Vs), ("Vm", Vm), ("Kd", Kd), ("Vd", Vd),
                     ("Q", Q), ("scores", sc_fast), ("scores_slow", sc_slow)):
            out[f"i8_{name}_{k}"] = bits(t.float() if t.dtype == torch.float16 and k in ("K", "V", "Q") else t)
        cases.append({"name": name, "dtype": str(dt).split(".")[-1], "shape": list(shape), "page": page,
                      "q_dtype": str(Q.dtype).split(".")[-1]})
    np.savez_compressed(os.path.join(HERE, "int8.npz"), **out)
    with open(os.path.join(HERE, "int8.json"), "w") as f:
        json.dump({"torch": torch.__version__, "cases": cases}, f, indent=1)
    print("int8.npz", os.path.getsize(os.path.join(HERE, "int8.npz")))


if __name__ == "__main__":
    main()
