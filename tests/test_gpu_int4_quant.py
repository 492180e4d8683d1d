"""INT4 pack-on-append kernels vs the oracle and the reference goldens (bit-exact)."""
import pytest
import torch

import oracle
from tests._util import DTYPES, bit_equal, make_kv

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kvq():
    from flashquest_b200.kernel import kv_quant
    return kv_quant


def test_quant_matches_reference_goldens(golden, kvq):
    for case in golden.meta["quant"]:
        n, dt = case["name"], DTYPES[case["dtype"]]
        K = golden.get("quant_int4", f"q_{n}_K", dtype=dt).cuda()
        V = golden.get("quant_int4", f"q_{n}_V", dtype=dt).cuda()
        Kp, Ks, Km = kvq.quantize_k_int4(K, case["page"])
        Vp, Vs, Vm = kvq.quantize_v_int4(V)
        for got, key in ((Kp, "Kp"), (Ks, "Ks"), (Km, "Km"), (Vp, "Vp"), (Vs, "Vs"), (Vm, "Vm")):
            assert bit_equal(got.cpu(), golden.get("quant_int4", f"q_{n}_{key}")), f"{n}:{key}"
        Kd = kvq.dequantize_k_int4(Kp, Ks, Km, case["page"])
        Vd = kvq.dequantize_v_int4(Vp, Vs, Vm)
        assert bit_equal(Kd.cpu(), golden.get("quant_int4", f"q_{n}_Kd")), n
        assert bit_equal(Vd.cpu(), golden.get("quant_int4", f"q_{n}_Vd")), n


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape,page", [((2, 8, 512, 128), 16), ((1, 3, 200, 64), 8), ((1, 2, 130, 128), 64),
                                        ((1, 2, 64, 32), 64), ((1, 1, 33, 256), 16)])
def test_quant_matches_oracle(kvq, dtype, shape, page):
    K = make_kv(11, shape, dtype)
    V = make_kv(12, shape, dtype, outliers=())
    K[0, 0, : min(page, shape[2]), 1] = 0.25      # constant channel -> eps clamp
    V[0, 0, 0, :] = -3.0                          # constant token -> eps clamp
    want = oracle.quantize_k_int4(K, page) + oracle.quantize_v_int4(V)
    got = kvq.quantize_k_int4(K.cuda(), page) + kvq.quantize_v_int4(V.cuda())
    for g, w, name in zip(got, want, ("Kp", "Ks", "Km", "Vp", "Vs", "Vm")):
        assert bit_equal(g.cpu(), w), name


def test_quant_strided_input_and_output(kvq):
    """Inputs that are views (transposed projections) and outputs written into cache slices."""
    B, H, S, D, page = 2, 4, 96, 128, 16
    x = make_kv(5, (B, S, H, D), torch.bfloat16)
    K = x.cuda().transpose(1, 2)                     # (B,H,S,D) view, token stride H*D
    want = oracle.quantize_k_int4(x.transpose(1, 2).contiguous(), page)
    got = kvq.quantize_k_int4(K, page)
    for g, w in zip(got, want):
        assert bit_equal(g.cpu(), w)
    S_max = 256
    Kp = torch.zeros(3, B, H, S_max, D // 2, dtype=torch.uint8, device="cuda")
    Ks = torch.zeros(3, B, H, S_max // page, D, dtype=torch.bfloat16, device="cuda")
    Km = torch.zeros_like(Ks)
    kvq.quantize_kv_int4_into(K, None, page, S, K_packed=Kp[1, :, :, 32:], K_scale=Ks[1, :, :, 2:], K_mn=Km[1, :, :, 2:])
    assert bit_equal(Kp[1, :, :, 32:32 + S].cpu(), want[0])
    assert bit_equal(Ks[1, :, :, 2:2 + S // page].cpu(), want[1])
    assert (Kp[0] == 0).all() and (Kp[2] == 0).all() and (Kp[1, :, :, :32] == 0).all() and (Kp[1, :, :, 32 + S:] == 0).all()


def test_odd_head_dim_rejected(kvq):
    with pytest.raises(ValueError, match="even head_dim"):
        kvq.quantize_k_int4(torch.randn(1, 2, 64, 65, dtype=torch.bfloat16, device="cuda"), 64)
    with pytest.raises(ValueError, match="even head_dim"):
        kvq.quantize_v_int4(torch.randn(1, 2, 64, 65, dtype=torch.bfloat16, device="cuda"))


def test_full_size_roundtrip_properties(kvq):
    """BASELINE config 1 size (one layer): the reference's own round-trip bound
    |dequant - x| <= scale + 1e-2 (tests/test_kv_quant_int4.py:46-54; fp16 inputs are coded
    with fp16 metadata and decoded with its bf16 rounding) and mn + 15*scale ~ page max."""
    B, H, S, D, page = 1, 8, 32768, 128, 16
    g = torch.Generator(device="cuda").manual_seed(3)
    K = torch.randn(B, H, S, D, device="cuda", generator=g)
    K[..., [3, 17, 64, 100]] *= 8
    K = K.half()
    Kp, Ks, Km = kvq.quantize_k_int4(K, page)
    Kd = kvq.dequantize_k_int4(Kp, Ks, Km, page).float()
    sc = Ks.float().repeat_interleave(page, dim=2)
    err = (Kd - K.float()).abs()
    assert (err <= sc + 1e-2).all(), float((err - sc).max())
    pmax = K.float().view(B, H, S // page, page, D).max(dim=3).values
    assert torch.allclose(Km.float() + 15 * Ks.float(), pmax, atol=0.25, rtol=2e-2)
    V = torch.randn(B, H, S, D, device="cuda", generator=g).half()
    Vp, Vs, Vm = kvq.quantize_v_int4(V)
    Vd = kvq.dequantize_v_int4(Vp, Vs, Vm).float()
    assert ((Vd - V.float()).abs() <= Vs.float() + 1e-2).all()
    # a sample of pages against the oracle, bit for bit
    idx = slice(4096, 4096 + 64)
    w = oracle.quantize_k_int4(K[:, :, idx].cpu(), page)
    assert bit_equal(Kp[:, :, idx].cpu(), w[0]) and bit_equal(Ks[:, :, 256:260].cpu(), w[1])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_quotients_on_and_next_to_rounding_ties(kvq, dtype):
    """Scale exactly 1 (values span 0..15): x = k + 0.5 divides to an exact tie (round half to
    even), and the neighbouring representable values fall just beside it.  Also a large sample
    of fp32 values whose quotients crowd the half-integers under an awkward scale."""
    B, H, S, D, page = 1, 2, 64, 128, 16
    g = torch.Generator().manual_seed(5)
    base = torch.randint(0, 15, (B, H, S, D), generator=g).float() + 0.5          # k + 0.5
    eps = {torch.float16: 2.0 ** -8, torch.bfloat16: 2.0 ** -5, torch.float32: 2.0 ** -21}[dtype]
    jitter = torch.randint(-1, 2, (B, H, S, D), generator=g).float() * eps         # -eps, 0, +eps
    X = base + jitter
    X[..., 0] = 0.0      # every token / every page sees the full range 0..15
    X[..., 1] = 15.0
    X[:, :, 0::16, :] = 0.0
    X[:, :, 1::16, :] = 15.0
    X = X.to(dtype)
    want = oracle.quantize_k_int4(X, page) + oracle.quantize_v_int4(X)
    got = kvq.quantize_k_int4(X.cuda(), page) + kvq.quantize_v_int4(X.cuda())
    for a, b in zip(got, want):
        assert bit_equal(a.cpu(), b)
    if dtype == torch.float32:
        # scale 0.7 / 15: many quotients within a few ulps of k + 0.5
        k = torch.randint(0, 15, (1, 1, 4096, 128), generator=g).float() + 0.5
        Y = (k * torch.tensor(0.7 / 15, dtype=torch.float32))
        Y = torch.nextafter(Y, torch.where(torch.rand(Y.shape, generator=g) < 0.5, torch.zeros(()), torch.ones(()) * 10))
        Y[..., 0] = 0.0
        Y[..., 1] = 0.7
        want = oracle.quantize_v_int4(Y)
        got = kvq.quantize_v_int4(Y.cuda())
        for a, b in zip(got, want):
            assert bit_equal(a.cpu(), b)
