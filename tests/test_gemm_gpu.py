"""GPU parity of the tcgen05 block-scaled FP4 matmul against the fp64 oracle.

Tolerance: the kernel accumulates exact FP4 x FP4 x scale products in fp32 and rounds once to
bf16, the oracle computes in fp64 and rounds to bf16; they may differ by one bf16 ulp of the
result plus fp32 accumulation error, so |got - want| <= 2^-7 |want| + 2^-10 max|want|."""
import pytest
import torch

from oracle import fp4
from tests import inputs

pytestmark = pytest.mark.gpu

REL, ABS = 2.0 ** -7, 2.0 ** -10


def _random_operands(M, N, K, fmt, seed):
    g = 16 if fmt == "nvfp4" else 32
    gen = torch.Generator().manual_seed(seed)
    a = torch.randint(0, 256, (M, K // 2), generator=gen, dtype=torch.uint8)
    b = torch.randint(0, 256, (N, K // 2), generator=gen, dtype=torch.uint8)
    lo, hi = (118, 132) if fmt == "mxfp4" else (0x20, 0x50)
    sa = torch.randint(lo, hi, (M, K // g), generator=gen, dtype=torch.uint8)
    sb = torch.randint(lo, hi, (N, K // g), generator=gen, dtype=torch.uint8)
    return a, b, sa, sb


def _check(got, want):
    got, want = got.float(), want.float()
    tol = REL * want.abs() + ABS * want.abs().max()
    bad = (got - want).abs() > tol
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} outputs off; worst {(got - want).abs().max().item()}"


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("shape", [(128, 128, 64), (128, 256, 256), (1, 256, 256), (16, 1024, 512),
                                   (130, 384, 320), (257, 640, 1088), (300, 1024, 4096), (512, 136, 256)])
def test_gemm_random_codes_and_scales(cuda_device, fmt, shape):
    from fpq_b200 import ops

    M, N, K = shape
    a, b, sa, sb = _random_operands(M, N, K, fmt, seed=M * 7 + N * 3 + K)
    alpha = torch.tensor([0.37])
    want = fp4.fp4_matmul(a, b, sa, sb, 0.37, fmt)
    d = cuda_device
    got = ops.gemm_fp4(a.to(d), b.to(d), ops.swizzle_scales(sa.to(d)), ops.swizzle_scales(sb.to(d)), alpha.to(d), fmt)
    ops.check_device_errors(d)
    _check(got.cpu(), want)


# The W4A4 linear shapes of a Qwen3-8B block (K, N) at the token counts where the entry point leaves the
# large-M kernel: M = 1 and 16 take the swap-AB split-K kernel (the cluster size and the K depth per CTA
# change with K = 12288), M = 128 the single-CTA or the CTA-pair kernel depending on N.
QWEN3_8B_LINEARS = [(4096, 4096), (4096, 12288), (12288, 4096), (4096, 1024)]


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("kn", QWEN3_8B_LINEARS)
@pytest.mark.parametrize("M", [1, 16, 128])
def test_gemm_small_m_at_model_shapes(cuda_device, fmt, kn, M):
    from fpq_b200 import ops

    K, N = kn
    a, b, sa, sb = _random_operands(M, N, K, fmt, seed=M + 3 * N + 5 * K)
    d = cuda_device
    got = ops.gemm_fp4(a.to(d), b.to(d), ops.swizzle_scales(sa.to(d)), ops.swizzle_scales(sb.to(d)),
                       torch.tensor([0.25], device=d), fmt)
    ops.check_device_errors(d)
    assert got.shape == (M, N)
    # every row, a sample of the output features (first and last tile included)
    gen = torch.Generator().manual_seed(N + K)
    cols = torch.cat([torch.arange(0, 64), torch.arange(N - 64, N), torch.randperm(N, generator=gen)[:256]]).unique()
    want = fp4.fp4_matmul(a, b[cols], sa, sb[cols], 0.25, fmt)
    _check(got[:, cols.to(d)].cpu(), want)


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
def test_gemm_with_bias(cuda_device, fmt):
    from fpq_b200 import ops

    M, N, K = 96, 512, 512
    a, b, sa, sb = _random_operands(M, N, K, fmt, seed=5)
    bias = inputs.normal_weight(1, N, seed=9, std=50.0)[0]
    want = (fp4.fp4_matmul(a, b, sa, sb, 1.0, fmt).float() + bias.float())
    d = cuda_device
    got = ops.gemm_fp4(a.to(d), b.to(d), ops.swizzle_scales(sa.to(d)), ops.swizzle_scales(sb.to(d)),
                       torch.ones(1, device=d), fmt, bias=bias.to(d))
    ops.check_device_errors(d)
    got, want = got.cpu().float(), want
    tol = 2.0 ** -6 * want.abs() + ABS * want.abs().max()
    assert not ((got - want).abs() > tol).any()


@pytest.mark.parametrize("fmt,hgroup", [("mxfp4", 32), ("nvfp4", 16), ("nvfp4", 128)])
@pytest.mark.parametrize("M", [1, 16, 128, 2048])
def test_quantize_then_gemm_matches_oracle_pipeline(cuda_device, fmt, hgroup, M):
    """The W4A4 linear of the benchmark: rotate + quantise activations on the GPU (swizzled
    scales straight from the kernel), multiply with pre-quantised weights, compare with the
    oracle pipeline run on the CPU end to end."""
    from fpq_b200 import ops

    K, N = 1024, 768
    x = inputs.outlier_activations(M, K, seed=1)
    w = inputs.normal_weight(N, K, seed=3)
    d = cuda_device
    gs_a = gs_w = None
    alpha = 1.0 / 9.0
    xr, wr = fp4.fwht_butterfly(x, hgroup), fp4.fwht_butterfly(w, hgroup)
    if fmt == "nvfp4":
        gs_a, gs_w = fp4.nvfp4_global_scale(xr.abs().max()), fp4.nvfp4_global_scale(wr.abs().max())
        alpha = 1.0 / float(gs_a * gs_w)
    xq, xs, _ = fp4.quantize(xr, fmt, gs_a)
    wq, ws, _ = fp4.quantize(wr, fmt, gs_w)
    want = fp4.fp4_matmul(xq, wq, xs, ws, alpha, fmt)

    dq, dsb, _ = ops.quantize(x.to(d), fmt, hgroup, None if gs_a is None else gs_a.to(d), swizzled=True)
    dwq, dws, _ = ops.quantize(w.to(d), fmt, hgroup, None if gs_w is None else gs_w.to(d), swizzled=True)
    assert torch.equal(dq.cpu(), xq) and torch.equal(dwq.cpu(), wq)
    got = ops.gemm_fp4(dq, dwq, dsb, dws, torch.tensor([alpha], device=d), fmt)
    ops.check_device_errors(d)
    _check(got.cpu(), want)
    # and the result approximates the unquantised product
    exact = x.float() @ w.float().t()
    rel = (got.cpu().float() - exact).norm() / exact.norm()
    assert rel < 0.25


def test_gemm_rejects_bad_shapes(cuda_device):
    from fpq_b200 import ops, _cabi as C

    d = cuda_device
    a = torch.zeros(4, 48, dtype=torch.uint8, device=d)     # K = 96: not a multiple of 64
    b = torch.zeros(128, 48, dtype=torch.uint8, device=d)
    sa = torch.zeros(128, 4, dtype=torch.uint8, device=d)
    with pytest.raises(C.FpqError):
        ops.gemm_fp4(a, b, sa, sa, torch.ones(1, device=d), "mxfp4")
