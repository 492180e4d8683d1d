"""Dense causal attention of the prefill branch (fq_prefill_attention: the tcgen05 kernel for head_dim 128 with at
least one full query tile, the mma.sync kernel otherwise) against an fp32 restatement of
scaled_dot_product_attention(q, K, V, is_causal=True, enable_gqa=True) — the call it replaces in the reference's
patched forward (eager/llama_persistent_patch.py:196-201); top-left causal alignment as torch uses when S_q != S_kv.

Tolerance: the probabilities are rounded to the operand dtype before P.V and the output once more: 2e-3 (fp16) /
1.6e-2 (bf16) absolute on outputs of magnitude <= 1."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, K, V, scale):
    B, Hq, Sq, D = q.shape
    Hkv, Skv = K.shape[1], K.shape[2]
    Kf = K.float().repeat_interleave(Hq // Hkv, 1)
    Vf = V.float().repeat_interleave(Hq // Hkv, 1)
    s = (q.float() @ Kf.transpose(-1, -2)) * scale
    mask = torch.ones(Sq, Skv, dtype=torch.bool, device=q.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    return torch.softmax(s, -1) @ Vf


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,D", [(1, 6, 2, 300, 300, 128), (2, 4, 4, 128, 128, 128), (1, 3, 1, 517, 517, 128),
                                               (1, 2, 1, 130, 260, 128), (1, 2, 2, 1024, 1024, 128), (1, 4, 2, 100, 100, 128),
                                               (1, 4, 2, 200, 200, 64), (1, 24, 8, 2048, 2048, 128)])
def test_prefill_attention_matches_fp32_reference(dtype, B, Hq, Hkv, Sq, Skv, D):
    from flashquest_b200 import _lib
    from flashquest_b200.kernel.prefill_attn import prefill_causal_attention
    g = torch.Generator(device="cuda").manual_seed(Sq + D)
    q = torch.randn(B, Hq, Sq, D, device="cuda", generator=g).to(dtype)
    K = torch.randn(B, Hkv, Skv, D, device="cuda", generator=g).to(dtype)
    K[..., [3, 17, 64, 100] if D == 128 else [3, 17, 40]] *= 4.0
    V = torch.randn(B, Hkv, Skv, D, device="cuda", generator=g).to(dtype)
    scale = D ** -0.5
    want = _ref(q, K, V, scale)
    tol = 2e-3 if dtype == torch.float16 else 1.6e-2
    got = prefill_causal_attention(q, K, V)
    assert got.shape == (B, Hq, Sq, D) and got.dtype == dtype
    err = (got.float() - want).abs().max().item()
    assert err <= tol, err
    # (B, S, H, D) output layout and strided (non-contiguous) inputs, as the patched forward hands them over
    qs = q.transpose(1, 2).contiguous().transpose(1, 2)
    got2 = prefill_causal_attention(qs, K, V, out_bshd=True)
    assert got2.shape == (B, Sq, Hq, D)
    assert (got2.transpose(1, 2).float() - want).abs().max().item() <= tol
    torch.cuda.synchronize()
    assert _lib.lib().fq_device_status() == 0
