"""AWQ W4A16 GEMV through the C ABI against the CPU oracle (AutoAWQ GEMM format restated;
the reference's call sites are kernel/fused_proj.py:18-53)."""
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def _make_linear(K, N, group, seed, interleaved=True, bias=False):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(0, 16, (K, N), generator=g, dtype=torch.int32)
    zeros = torch.randint(0, 16, (K // group, N), generator=g, dtype=torch.int32)
    scales = (torch.rand(K // group, N, generator=g) * 0.02 + 0.002).half()
    qweight = oracle.awq_pack(codes, interleaved)
    qzeros = oracle.awq_pack(zeros, interleaved)
    b = (torch.randn(N, generator=g) * 0.1).half() if bias else None
    return qweight, scales, qzeros, b


def _to_dev(lin, group, interleaved):
    from flashquest_b200.quant import AWQLinear
    qw, sc, qz, b = lin
    return AWQLinear(qw.cuda(), sc.cuda(), qz.cuda(), b.cuda() if b is not None else None,
                     group_size=group, interleaved=interleaved)


def _check(y_dev, x, lin, group, interleaved):
    qw, sc, qz, b = lin
    ref = oracle.awq_gemv(x, qw, sc, qz, group_size=group, interleaved=interleaved)
    if b is not None:
        ref = ref + b.float()
    got = y_dev.float().cpu().reshape(ref.shape)
    # fp32 accumulation in another order + one rounding to fp16
    tol = 2e-3 * ref.abs().max().item() + 1e-3
    assert (got - ref).abs().max().item() <= tol


@pytest.mark.parametrize("M", [1, 2, 3, 8])
@pytest.mark.parametrize("interleaved", [True, False])
def test_qkv_llama3b_shapes(M, interleaved):
    from flashquest_b200.kernel.fused_proj import fused_qkv_proj
    K, group = 3072, 128
    lins = [_make_linear(K, N, group, 10 + i, interleaved) for i, N in enumerate((3072, 1024, 1024))]
    x = (torch.randn(1, M, K, generator=torch.Generator().manual_seed(M)) * 0.5).half()
    outs = fused_qkv_proj(x.cuda(), *[_to_dev(l, group, interleaved) for l in lins])
    assert outs[0].shape == (1, M, 3072) and outs[1].shape == (1, M, 1024)
    for y, l in zip(outs, lins):
        _check(y, x.reshape(M, K), l, group, interleaved)


def test_gate_up_and_single_with_bias():
    from flashquest_b200.kernel.fused_proj import fused_gate_up_proj
    K, group = 3072, 128
    lins = [_make_linear(K, 8192, group, 20 + i, True, bias=(i == 1)) for i in range(2)]
    x = (torch.randn(1, 1, K, generator=torch.Generator().manual_seed(5)) * 0.5).half()
    devs = [_to_dev(l, group, True) for l in lins]
    gate, up = fused_gate_up_proj(x.cuda(), *devs)
    _check(gate, x.reshape(1, K), lins[0], group, True)
    _check(up, x.reshape(1, K), lins[1], group, True)
    # a single projection, called twice in a row (ticket words must be back at zero)
    for _ in range(2):
        _check(devs[1](x.cuda()), x.reshape(1, K), lins[1], group, True)


def test_down_proj_long_k_and_odd_sizes():
    # K = 8192 (down projection), N not a multiple of the CTA tile, group 64
    for K, N, group in ((8192, 3072, 128), (512, 136, 64)):
        lin = _make_linear(K, N, group, 31, True)
        x = (torch.randn(2, K, generator=torch.Generator().manual_seed(6)) * 0.5).half()
        y = _to_dev(lin, group, True)(x.cuda())
        _check(y, x, lin, group, True)


def test_rejects_bad_arguments():
    from flashquest_b200.kernel.fused_proj import awq_gemv_fused
    lin = _make_linear(256, 64, 128, 1)
    dev = _to_dev(lin, 128, True)
    with pytest.raises(NotImplementedError):
        awq_gemv_fused(torch.zeros(9, 256, dtype=torch.float16, device="cuda"), (dev,))
    with pytest.raises(NotImplementedError):
        awq_gemv_fused(torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda"), (dev,))
    with pytest.raises(ValueError):
        awq_gemv_fused(torch.zeros(1, 128, dtype=torch.float16, device="cuda"), (dev,))


def _sep_ops():
    """The separate operators the fused launch must reproduce (fq_add_rmsnorm, fq_swiglu, fq_rope)."""
    from flashquest_b200._lib import check, lib, ptr, stream_ptr
    L = lib()
    dev = torch.device("cuda")

    def add_rmsnorm(x, delta, w, eps):
        s, y = torch.empty_like(x), torch.empty_like(x)
        check(L.fq_add_rmsnorm(ptr(x), ptr(delta), ptr(w), eps, x.shape[0], x.shape[1], ptr(s), ptr(y), stream_ptr(dev)))
        return s, y

    def swiglu(g, u):
        a = torch.empty_like(g)
        check(L.fq_swiglu(ptr(g), ptr(u), g.numel(), ptr(a), stream_ptr(dev)))
        return a

    def rope(q, Hq, k, Hkv, D, pos, theta):
        q, k = q.clone(), k.clone()
        check(L.fq_rope(ptr(q), Hq * D, D, Hq, ptr(k), Hkv * D, D, Hkv, q.shape[0], D, pos, theta, stream_ptr(dev)))
        return q, k
    return add_rmsnorm, swiglu, rope


@pytest.mark.parametrize("M", [1, 3, 8])
def test_fused_norm_qkv_rope(M):
    """add + RMSNorm in front of the fused QKV launch and the rotary embedding behind it: the separate
    operators on the same inputs give the same bits, except where the row's sum of squares (another
    summation order) moves the normalised value by an fp16 ulp; the residual sum is exact."""
    from flashquest_b200.kernel.fused_proj import awq_gemv_fused
    add_rmsnorm, _, rope = _sep_ops()
    K, group, D, theta, pos = 3072, 128, 128, 500000.0, 4321
    lins = [_make_linear(K, N, group, 70 + i, True, bias=(i == 1)) for i, N in enumerate((3072, 1024, 1024))]
    devs = [_to_dev(l, group, True) for l in lins]
    g = torch.Generator().manual_seed(100 + M)
    x = (torch.randn(M, K, generator=g) * 0.7).half().cuda()
    delta = (torch.randn(M, K, generator=g) * 0.3).half().cuda()
    w = (1.0 + 0.1 * torch.randn(K, generator=g)).half().cuda()
    s_ref, normed = add_rmsnorm(x, delta, w, 1e-5)
    q0, k0, v0 = awq_gemv_fused(normed, devs)
    q0, k0 = rope(q0, 24, k0, 8, D, pos, theta)
    pos_dev = torch.tensor([pos], dtype=torch.int32, device="cuda")
    for kw in (dict(pos=pos), dict(pos_dev=pos_dev)):
        q1, k1, v1, s1 = awq_gemv_fused(x, devs, add=delta, norm_weight=w, eps=1e-5, return_sum=True,
                                        rope=dict(mask=3, theta=theta, head_dim=D, **kw))
        assert torch.equal(s1, s_ref)
        for a, b in ((q1, q0), (k1, k0), (v1, v0)):
            err = (a.float() - b.float()).abs()
            assert err.max().item() <= 2e-3 * b.float().abs().max().item() + 1e-3
            assert (err > 0).float().mean().item() < 0.2
    # without the addition and without the sum: plain RMSNorm of x
    _, normed_x = add_rmsnorm(x, None, w, 1e-5)
    (v2,) = awq_gemv_fused(x, devs[2:], norm_weight=w, eps=1e-5)
    (v3,) = awq_gemv_fused(normed_x, devs[2:])
    assert (v2.float() - v3.float()).abs().max().item() <= 2e-3 * v3.float().abs().max().item() + 1e-3
    # against the oracle end to end
    _check(v3, normed_x.cpu(), lins[2], group, True)


@pytest.mark.parametrize("M", [1, 4])
def test_fused_swiglu_down(M):
    from flashquest_b200.kernel.fused_proj import awq_gemv_fused
    _, swiglu, _ = _sep_ops()
    K, N, group = 8192, 3072, 128
    lin = _make_linear(K, N, group, 81, True)
    dev = _to_dev(lin, group, True)
    g = torch.Generator().manual_seed(200 + M)
    gate = (torch.randn(M, K, generator=g) * 1.5).half().cuda()
    up = (torch.randn(M, K, generator=g) * 0.5).half().cuda()
    act = swiglu(gate, up)
    (y0,) = awq_gemv_fused(act, (dev,))
    (y1,) = awq_gemv_fused(gate, (dev,), swiglu_up=up)
    assert torch.equal(y0, y1)            # same inputs, same summation order: same bits
    _check(y1, act.cpu(), lin, group, True)
    for ks in (1, 2, 4, 8):
        (y2,) = awq_gemv_fused(gate, (dev,), swiglu_up=up, k_split=ks)
        _check(y2, act.cpu(), lin, group, True)
    with pytest.raises(ValueError):
        awq_gemv_fused(gate, (dev,), swiglu_up=up, norm_weight=up[0])
    with pytest.raises(ValueError, match="k_split"):
        awq_gemv_fused(gate, (dev,), k_split=3)


def _check_gemm(y_dev, x, lin, group, interleaved):
    """Tensor-core path: weights rounded once to fp16 (as AutoAWQ's GEMM kernels do), fp32 accumulation."""
    qw, sc, qz, b = lin
    ref = oracle.awq_gemv(x, qw, sc, qz, group_size=group, interleaved=interleaved)
    if b is not None:
        ref = ref + b.float()
    got = y_dev.float().cpu().reshape(ref.shape)
    tol = 2e-3 * ref.abs().max().item() + 1e-3
    err = (got - ref).abs().max().item()
    assert err <= tol, (err, tol)


@pytest.mark.parametrize("M", [16, 200, 256, 1000])
@pytest.mark.parametrize("interleaved", [True, False])
def test_gemm_fused_qkv(M, interleaved):
    """The tcgen05 dequant-GEMM on the fused QKV shape of BASELINE config 3, ragged and full row tiles,
    both nibble orders, row by row against the oracle's dequant-matmul."""
    from flashquest_b200 import _lib
    from flashquest_b200.kernel.fused_proj import fused_qkv_proj
    K, group = 3072, 128
    lins = [_make_linear(K, N, group, 40 + i, interleaved, bias=(i == 2)) for i, N in enumerate((3072, 1024, 1024))]
    x = (torch.randn(M, K, generator=torch.Generator().manual_seed(M)) * 0.5).half()
    outs = fused_qkv_proj(x.cuda(), *[_to_dev(l, group, interleaved) for l in lins])
    torch.cuda.synchronize()
    assert _lib.lib().fq_device_status() == 0
    assert outs[0].shape == (M, 3072) and outs[2].shape == (M, 1024)
    rows = sorted(r for r in {0, 1, 127, 128, M // 2, M - 1} if r < M)
    for y, l in zip(outs, lins):
        _check_gemm(y[rows], x[rows], l, group, interleaved)


def test_gemm_gate_up_down_and_group64():
    from flashquest_b200.kernel.fused_proj import awq_gemm_fused, fused_gate_up_proj
    K, group, M = 3072, 128, 300
    lins = [_make_linear(K, 8192, group, 50 + i, True) for i in range(2)]
    x = (torch.randn(M, K, generator=torch.Generator().manual_seed(9)) * 0.5).half()
    gate, up = fused_gate_up_proj(x.cuda(), *[_to_dev(l, group, True) for l in lins])
    rows = [0, 255, 256, 299]
    _check_gemm(gate[rows], x[rows], lins[0], group, True)
    _check_gemm(up[rows], x[rows], lins[1], group, True)
    for K, N, group in ((8192, 3072, 128), (512, 128, 64)):
        lin = _make_linear(K, N, group, 61, True)
        x = (torch.randn(40, K, generator=torch.Generator().manual_seed(6)) * 0.5).half()
        (y,) = awq_gemm_fused(x.cuda(), (_to_dev(lin, group, True),))
        _check_gemm(y, x, lin, group, True)
    with pytest.raises(NotImplementedError):
        awq_gemm_fused(torch.zeros(16, 256, dtype=torch.float16, device="cuda"), (_to_dev(_make_linear(256, 64, 128, 1), 128, True),))
