"""Shape and dtype contracts of the reference-named custom ops, checked on the meta device (no GPU, no kernels):
what `torch.compile` sees when it traces through them.  The expected shapes are the ones the reference's fake
implementations return (inference_lib/src/fp_quant/module/qutlass_ops.py:54-71, :87-105, :165-212, :229-245,
:260-274, :285-304, :315-330 of IST-DASLab/FP-Quant)."""
import torch

from fpq_b200.fp_quant.module import qutlass_ops  # noqa: F401  (registers the ops)


def _up(n, m):
    return -(-n // m) * m


def _meta(*shape, dtype=torch.bfloat16):
    return torch.empty(*shape, dtype=dtype, device="meta")


NS = getattr(torch.ops, qutlass_ops.NAMESPACE)


def test_forward_ops_on_meta_tensors():
    M, K, N = 200, 256, 384
    x, h = _meta(M, K), _meta(32, 32)
    q, s, mask = NS.fused_quantize_mx_op(x, h, "quest", True)
    assert q.shape == (M, K // 2) and q.dtype == torch.uint8
    assert s.shape == (_up(M, 128), _up(K // 32, 4)) and s.dtype == torch.float8_e8m0fnu
    assert mask.shape == (M, K // 8) and mask.dtype == torch.uint8
    q2, s2 = NS.fused_quantize_nv_op(x, _meta(16, 16), _meta(1, dtype=torch.float32))
    assert q2.shape == (M, K // 2) and s2.shape == (_up(M, 128), _up(K // 16, 4)) and s2.dtype == torch.float8_e4m3fn
    w = _meta(N, K // 2, dtype=torch.uint8)
    ws = _meta(_up(N, 128), _up(K // 32, 4), dtype=torch.float8_e8m0fnu)
    y = NS.matmul_mxf4_bf16_tn_op(q, w, s, ws, _meta(1, dtype=torch.float32))
    assert y.shape == (M, N) and y.dtype == torch.bfloat16


def test_backward_ops_on_meta_tensors():
    m, n = 256, 384
    x, h = _meta(m, n), _meta(32, 32)
    # transpose + rotate + quantise: [m, n] -> codes [n, m/2], scales along m
    q, s = NS.backward_t_bf16(x, h)
    assert q.shape == (n, m // 2) and q.dtype == torch.uint8 and s.dtype == torch.float8_e8m0fnu
    assert s.shape[0] >= n and s.shape[1] >= m // 32
    xq, xs = _meta(m, n // 2, dtype=torch.uint8), _meta(_up(m, 128), _up(n // 32, 4), dtype=torch.float8_e8m0fnu)
    q2, s2 = NS.backward_qt_bf16(xq, xs, h, _meta(1, dtype=torch.float32))
    assert q2.shape == (n, m // 2) and s2.shape[0] >= n and s2.shape[1] >= m // 32
    # one E4M3 tensor with scales along either axis; the row count is padded to 128
    g = _meta(200, n)
    g8, rs, cs = NS.backward_bf16_square_double_mxfp8(g)
    assert g8.shape == (256, n) and g8.dtype == torch.float8_e4m3fn
    assert rs.shape == (256, n // 32) and cs.shape == (n, 256 // 32) and rs.dtype == cs.dtype == torch.float8_e8m0fnu
    t8, ts = NS.mxfp4_transpose_mxfp8(_meta(200, n // 2, dtype=torch.uint8), _meta(256, _up(n // 32, 4), dtype=torch.float8_e8m0fnu))
    assert t8.shape == (n, 256) and ts.shape == (n, 8)
    # the two MXFP8 products: tn [M, K] x [N, K] -> [M, N]; nn takes its first operand as [K, M]
    a, b = _meta(256, n, dtype=torch.float8_e4m3fn), _meta(512, n, dtype=torch.float8_e4m3fn)
    sa, sb = _meta(256, n // 32, dtype=torch.float8_e8m0fnu), _meta(512, n // 32, dtype=torch.float8_e8m0fnu)
    alpha = _meta(1, dtype=torch.float32)
    assert NS.matmul_mxf8_bf16_tn_op(a, b, sa, sb, alpha).shape == (256, 512)
    at = _meta(n, 256, dtype=torch.float8_e4m3fn)          # [K, M]
    out = NS.matmul_mxf8_bf16_nn_op(at, b, sa, sb, alpha)
    assert out.shape == (256, 512) and out.dtype == torch.bfloat16
