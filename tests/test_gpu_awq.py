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
