"""GPU parity of the tcgen05 MXFP8 matmul (`matmul_mxf8_bf16_tn_op`, the GEMM of the reference's quantised
backward pass, inference_lib/src/fp_quant/module/qutlass_ops.py:171-189) against the fp64 oracle.

Tolerance as for the FP4 matmul: exact products accumulated in fp32 and one rounding to bf16 against fp64
rounded to bf16: |got - want| <= 2^-7 |want| + 2^-10 max|want|.  QuTLASS itself is not available, so this
pins the arithmetic contract (E4M3 x E4M3, one E8M0 scale per 32 elements of K), not QuTLASS' bits."""
import pytest
import torch

from oracle import fp4

pytestmark = pytest.mark.gpu

REL, ABS = 2.0 ** -7, 2.0 ** -10


def _random_operands(M, N, K, seed):
    gen = torch.Generator().manual_seed(seed)

    def e4m3_bytes(rows):
        x = torch.randint(0, 256, (rows, K), generator=gen, dtype=torch.uint8)
        x[(x & 0x7F) == 0x7F] = 0x38            # the two NaN patterns become 1.0
        return x

    a, b = e4m3_bytes(M), e4m3_bytes(N)
    sa = torch.randint(120, 131, (M, K // 32), generator=gen, dtype=torch.uint8)
    sb = torch.randint(120, 131, (N, K // 32), generator=gen, dtype=torch.uint8)
    return a, b, sa, sb


def _check(got, want):
    got, want = got.float(), want.float()
    tol = REL * want.abs() + ABS * want.abs().max()
    bad = (got - want).abs() > tol
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} outputs off; worst {(got - want).abs().max().item()}"


@pytest.mark.parametrize("shape", [(128, 256, 128), (256, 256, 32), (1, 256, 256), (16, 1024, 512), (130, 384, 320),
                                   (257, 640, 1088), (300, 1024, 4096), (512, 136, 256), (1024, 4096, 2048)])
def test_mxf8_gemm_random_bytes_and_scales(cuda_device, shape):
    from fpq_b200 import ops

    M, N, K = shape
    a, b, sa, sb = _random_operands(M, N, K, seed=M * 7 + N * 3 + K)
    want = fp4.mxfp8_matmul(a, b, sa, sb, 2.0 ** -9)
    d = cuda_device
    got = ops.gemm_mxf8(a.to(d).view(torch.float8_e4m3fn), b.to(d), ops.swizzle_scales(sa.to(d)),
                        ops.swizzle_scales(sb.to(d)), torch.tensor([2.0 ** -9], device=d))
    ops.check_device_errors(d)
    assert got.shape == (M, N) and got.dtype == torch.bfloat16
    _check(got.cpu(), want)


def test_mxf8_gemm_every_scale_byte_position(cuda_device):
    """One 32-element group of K at a time carries data (scale 2^j for group j): every one of the four scale
    bytes a stage holds per row, in every stage of the ring, must be the one the instruction applies."""
    from fpq_b200 import ops

    M, N, K = 256, 256, 1024
    d = cuda_device
    gen = torch.Generator().manual_seed(5)
    a = torch.full((M, K), 0x38, dtype=torch.uint8)                       # 1.0 everywhere
    b = torch.randint(0x30, 0x40, (N, K), generator=gen, dtype=torch.uint8)   # 0.5 .. 1.875
    sb = torch.full((N, K // 32), 127, dtype=torch.uint8)
    for j in range(K // 32):
        sa = torch.zeros(M, K // 32, dtype=torch.uint8)                   # 2^-127: the other groups vanish in bf16
        sa[:, j] = 127 + (j % 7)
        got = ops.gemm_mxf8(a.to(d), b.to(d), ops.swizzle_scales(sa.to(d)), ops.swizzle_scales(sb.to(d)),
                            torch.ones(1, device=d))
        want = fp4.mxfp8_matmul(a, b, sa, sb, 1.0)
        ops.check_device_errors(d)
        assert torch.equal(got.cpu(), want), j


def test_mxf8_op_takes_row_major_scales(cuda_device):
    """The reference-named op: row-major E8M0 scales (float8_e8m0fnu), swizzled per call like `to_blocked`."""
    from fpq_b200.fp_quant.module.qutlass_ops import matmul_mxf8_bf16_tn_op

    M, N, K = 384, 512, 512
    a, b, sa, sb = _random_operands(M, N, K, seed=11)
    d = cuda_device
    got = matmul_mxf8_bf16_tn_op(a.to(d).view(torch.float8_e4m3fn), b.to(d).view(torch.float8_e4m3fn),
                                 sa.to(d).view(torch.float8_e8m0fnu), sb.to(d).view(torch.float8_e8m0fnu),
                                 torch.tensor([0.5], device=d))
    _check(got.cpu(), fp4.mxfp8_matmul(a, b, sa, sb, 0.5))


def test_mxf8_gemm_matches_the_vendor_library(cuda_device):
    """cuBLASLt's block-scaled MXFP8 GEMM through torch on the same bytes and the same swizzled scales (the
    layout is thereby pinned independently of the oracle).  Skipped where torch rejects the call."""
    from fpq_b200 import ops

    M, N, K = 512, 768, 1024
    a, b, sa, sb = _random_operands(M, N, K, seed=3)
    d = cuda_device
    sa_sw, sb_sw = ops.swizzle_scales(sa.to(d)), ops.swizzle_scales(sb.to(d))
    got = ops.gemm_mxf8(a.to(d), b.to(d), sa_sw, sb_sw, torch.ones(1, device=d))
    try:
        lib = torch._scaled_mm(a.to(d).view(torch.float8_e4m3fn), b.to(d).view(torch.float8_e4m3fn).t(),
                               sa_sw.view(torch.float8_e8m0fnu), sb_sw.view(torch.float8_e8m0fnu),
                               out_dtype=torch.bfloat16)
    except Exception as exc:      # noqa: BLE001
        pytest.skip(f"torch._scaled_mm rejects MXFP8 here: {exc}")
    _check(got.cpu(), lib.cpu())


def test_mxf8_gemm_rejects_bad_shapes(cuda_device):
    from fpq_b200 import ops

    d = cuda_device
    a = torch.zeros(128, 48, dtype=torch.uint8, device=d)           # K not a multiple of 32
    with pytest.raises(Exception):
        ops.gemm_mxf8(a, a, torch.zeros(128, 4, dtype=torch.uint8, device=d),
                      torch.zeros(128, 4, dtype=torch.uint8, device=d), torch.ones(1, device=d))
