"""The benchmark's full sizes, checked on samples the CPU oracle can afford: rows of the quantiser and
rows x columns of the GEMM are independent of the rest of the problem, and a column slab of X^T X needs
only those columns of X.  The sampled entries must meet the same bar as the small cases (bit-exact
codes and scale bytes; GEMM within bf16 rounding of the fp64 oracle; Hessian 1e-5 relative)."""
import pytest
import torch

from oracle import fp4
from tests import inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt,hgroup", [("mxfp4", 32), ("nvfp4", 16)])
def test_quantize_8192x12288_sampled_rows(cuda_device, fmt, hgroup):
    from fpq_b200 import ops

    M, K = 8192, 12288
    x = inputs.outlier_activations(M, K, seed=11)
    gs = torch.tensor([7.25]) if fmt == "nvfp4" else None
    codes, sbytes, _ = ops.quantize(x.to(cuda_device), fmt, hgroup, None if gs is None else gs.to(cuda_device),
                                    swizzled=False)
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:96]
    want_codes, want_sb, _ = fp4.quantize(fp4.fwht_butterfly(x[rows], hgroup), fmt, gs)
    assert torch.equal(codes[rows.to(cuda_device)].cpu(), want_codes)
    assert torch.equal(sbytes.view(torch.uint8)[rows.to(cuda_device)].cpu()[:, : K // (32 if fmt == "mxfp4" else 16)],
                       want_sb.view(torch.uint8))


@pytest.mark.parametrize("shape", [(8192, 12288, 4096), (8192, 4096, 12288)])
@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
def test_gemm_full_size_sampled(cuda_device, fmt, shape):
    from fpq_b200 import ops

    M, N, K = shape
    g = 16 if fmt == "nvfp4" else 32
    gen = torch.Generator().manual_seed(M + N + K)
    a = torch.randint(0, 256, (M, K // 2), generator=gen, dtype=torch.uint8)
    b = torch.randint(0, 256, (N, K // 2), generator=gen, dtype=torch.uint8)
    lo, hi = (118, 132) if fmt == "mxfp4" else (0x20, 0x50)
    sa = torch.randint(lo, hi, (M, K // g), generator=gen, dtype=torch.uint8)
    sb = torch.randint(lo, hi, (N, K // g), generator=gen, dtype=torch.uint8)
    d = cuda_device
    got = ops.gemm_fp4(a.to(d), b.to(d), ops.swizzle_scales(sa.to(d)), ops.swizzle_scales(sb.to(d)),
                       torch.tensor([0.5], device=d), fmt)
    ops.check_device_errors(d)
    rows = torch.randperm(M, generator=gen)[:40]
    cols = torch.randperm(N, generator=gen)[:320]
    want = fp4.fp4_matmul(a[rows], b[cols], sa[rows], sb[cols], 0.5, fmt).float()
    sub = got[rows.to(d)][:, cols.to(d)].cpu().float()
    tol = 2.0 ** -7 * want.abs() + 2.0 ** -10 * want.abs().max()
    bad = (sub - want).abs() > tol
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} sampled outputs off"


@pytest.mark.parametrize("tokens,d", [(5000, 3336), (2048, 14336)])
def test_hessian_large_column_slab(cuda_device, tokens, d):
    from fpq_b200 import ops

    x = inputs.correlated_activations(tokens, d, seed=3)
    H = torch.zeros(d, d, device=cuda_device)
    ops.hessian_accumulate(H, x.to(cuda_device), alpha=0.5, beta=0.0)
    ops.check_device_errors(cuda_device)
    cols = torch.randperm(d, generator=torch.Generator().manual_seed(2))[:48]
    want = (x.double().t() @ x[:, cols].double()) * 0.5
    got = H[:, cols.to(cuda_device)].cpu().double()
    assert ((got - want).norm() / want.norm()).item() < 1e-5
    assert torch.equal(H, H.t())
