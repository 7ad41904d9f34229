"""The MXFP8 backward pass (`FPQuant4x8MasterFn`, inference_lib/src/fp_quant/module/linear_fns.py:232-350):
its two re-quantisation kernels against the CPU restatement (oracle/mxfp8.py, bit for bit), the `nn` form of
the GEMM, and the gradients of an `FPQuantLinear` against the exact products of the operands the backward
pass is defined on.  QuTLASS, whose kernels the reference calls here, is not available: what is pinned is
this repository's definition of the arithmetic and the reference's interface and data flow."""
import pytest
import torch

from oracle import fp4, mxfp8

pytestmark = pytest.mark.gpu


def _bf16_matrix(rows, cols, seed, spread=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    if spread:      # rows and column bands of very different magnitude, some exact zeros
        x = x * torch.exp2(torch.randint(-12, 6, (rows, 1), generator=g).float())
        x[:, : cols // 4] *= 2.0 ** -9
        x[torch.rand(rows, cols, generator=g) < 0.05] = 0.0
    return x.bfloat16()


@pytest.mark.parametrize("shape", [(128, 32), (100, 256), (257, 288), (1, 64), (640, 1024)])
def test_square_quantize_matches_the_oracle(cuda_device, shape):
    from fpq_b200 import ops

    rows, cols = shape
    x = _bf16_matrix(rows, cols, seed=rows + cols)
    if rows > 64:
        x[32:64, :32] = 0.0                                   # an all-zero square
    want, want_rs, want_cs = mxfp8.square_quantize(x)
    got, rs, cs = ops.quantize_mxfp8_square(x.to(cuda_device))
    assert got.shape == want.shape and rs.shape == want_rs.shape and cs.shape == want_cs.shape
    assert torch.equal(rs.cpu(), want_rs) and torch.equal(cs.cpu(), want_cs)
    assert torch.equal(got.view(torch.uint8).cpu(), want)
    # what the scales mean: the same bytes dequantise to the same values along either axis
    a = mxfp8.dequantize_mxfp8(want, want_rs)
    b = mxfp8.dequantize_mxfp8(want.t().contiguous(), want_cs).t()
    assert torch.equal(a, b)
    ref = x.double()
    assert float((a[:rows] - ref).norm() / ref.norm()) < 0.04
    # the forms the backward pass uses: scales in the GEMM's tile layout, bytes in both orientations
    got2, rs2, cs2, got_t = ops.quantize_mxfp8_square(x.to(cuda_device), swizzled=True, transposed=True)
    assert torch.equal(got2.view(torch.uint8).cpu(), want) and torch.equal(got_t.view(torch.uint8).cpu(), want.t())
    assert torch.equal(rs2.cpu().flatten(), fp4.swizzle_scales(want_rs).flatten())
    assert torch.equal(cs2.cpu().flatten(), fp4.swizzle_scales(want_cs).flatten())


def test_square_quantize_extremes(cuda_device):
    """Largest and smallest bf16 magnitudes, a square of bf16 subnormals, values that saturate at 448."""
    from fpq_b200 import ops

    x = torch.zeros(128, 128, dtype=torch.bfloat16)
    x[:32, :32] = 3.0e38
    x[:32, 32:64] = torch.tensor(1e-40).bfloat16()            # subnormal in bf16
    x[32:64, :32] = torch.linspace(-500, 500, 32).bfloat16()  # 2^8 <= amax < 2^9: scaled values reach past 448
    x[32:64, 32:64] = torch.tensor(9.2e-41).bfloat16()
    x[64:96, 0] = 1.0
    want, want_rs, want_cs = mxfp8.square_quantize(x)
    got, rs, cs = ops.quantize_mxfp8_square(x.to(cuda_device))
    assert torch.equal(rs.cpu(), want_rs) and torch.equal(cs.cpu(), want_cs)
    assert torch.equal(got.view(torch.uint8).cpu(), want)


@pytest.mark.parametrize("shape", [(128, 128), (70, 256), (257, 96), (512, 1024)])
def test_fp4_transpose_matches_the_oracle(cuda_device, shape):
    from fpq_b200 import ops

    rows, cols = shape
    g = torch.Generator().manual_seed(rows * 3 + cols)
    codes = torch.randint(0, 256, (rows, cols // 2), generator=g, dtype=torch.uint8)
    sb = torch.randint(110, 135, (rows, cols // 32), generator=g, dtype=torch.uint8)
    sb[::7] = 90                                              # rows 2^-20 and more below their neighbours: rounded
    sb[3::11] = 2
    want, want_s = mxfp8.fp4_transpose_fp8(codes, sb)
    got, got_s = ops.mxfp4_transpose_mxfp8(codes.to(cuda_device), sb.to(cuda_device))
    assert torch.equal(got_s.cpu(), want_s)
    assert torch.equal(got.view(torch.uint8).cpu(), want)
    got2, got_s2 = ops.mxfp4_transpose_mxfp8(codes.to(cuda_device), sb.to(cuda_device), swizzled=True)
    assert torch.equal(got2.view(torch.uint8).cpu(), want)
    assert torch.equal(got_s2.cpu().flatten(), fp4.swizzle_scales(want_s).flatten())


def test_fp4_transpose_is_exact_for_real_operands(cuda_device):
    """Operands as the forward pass makes them (Hadamard 32 + MXFP4 abs_max of activations with outlier
    channels): the MXFP8 transpose dequantises to exactly the transposed MXFP4 values."""
    from fpq_b200 import ops
    from tests import inputs

    x = inputs.outlier_activations(300, 512, seed=4)
    d = cuda_device
    q, sb, _ = ops.quantize(x.to(d), "mxfp4", 32)
    t, ts = ops.mxfp4_transpose_mxfp8(q, sb)
    want = fp4.dequantize(fp4.unpack_codes(q.cpu()), fp4.decode_scale_bytes(sb.cpu(), "mxfp4"), 32).double()
    got = mxfp8.dequantize_mxfp8(t.view(torch.uint8).cpu(), ts.cpu())
    assert torch.equal(got[:, :300], want.t()) and float(got[:, 300:].abs().max()) == 0.0


def test_nn_form_equals_tn_form(cuda_device):
    from fpq_b200.fp_quant.module.qutlass_ops import matmul_mxf8_bf16_nn_op, matmul_mxf8_bf16_tn_op

    d = cuda_device
    g = torch.Generator().manual_seed(2)
    K, M, N = 256, 384, 512
    a = torch.randint(0, 0x7E, (K, M), generator=g, dtype=torch.uint8)       # stored [K, M]
    b = torch.randint(0, 0x7E, (N, K), generator=g, dtype=torch.uint8)
    sa = torch.randint(120, 130, (M, K // 32), generator=g, dtype=torch.uint8)
    sb = torch.randint(120, 130, (N, K // 32), generator=g, dtype=torch.uint8)
    alpha = torch.tensor([0.25], device=d)
    e8 = torch.float8_e8m0fnu
    nn = matmul_mxf8_bf16_nn_op(a.to(d).view(torch.float8_e4m3fn), b.to(d).view(torch.float8_e4m3fn),
                                sa.to(d).view(e8), sb.to(d).view(e8), alpha)
    tn = matmul_mxf8_bf16_tn_op(a.t().contiguous().to(d).view(torch.float8_e4m3fn), b.to(d).view(torch.float8_e4m3fn),
                                sa.to(d).view(e8), sb.to(d).view(e8), alpha)
    assert nn.shape == (M, N) and torch.equal(nn, tn)
    want = fp4.mxfp8_matmul(a.t().contiguous(), b, sa, sb, 0.25)
    assert float((nn.cpu().float() - want.float()).abs().max()) <= 2.0 ** -7 * float(want.float().abs().max())


@pytest.mark.parametrize("method", ["abs_max", "quest"])
@pytest.mark.parametrize("bias,N", [(False, 384), (True, 384), (False, 320)])
def test_mxfp8_backward_gradients(cuda_device, method, bias, N):
    """`FPQuantLinear(backward_dtype=MXFP8, store_master_weights=True)`: the forward equals the bf16-backward
    configuration's; grad_input and grad_weight are compared with the exact (fp64) products of the gradient
    with the dequantised MXFP4 operands, clip masks applied, rotated back -- the quantity the backward pass
    estimates.  The only error is the E4M3 rounding of the gradient (3 mantissa bits: 2-3 % in norm)."""
    from fpq_b200.fp_quant import FPQuantConfig, FPQuantDtype, FPQuantLinear
    from fpq_b200.fp_quant.module.linear_fns import _unpack_mask, forward_quantize
    from tests import inputs

    d = cuda_device
    tokens, K, h = 200, 256, 32            # N = 320: an output width that is not a multiple of the 128-row padding
    cfg = dict(forward_dtype=FPQuantDtype.MXFP4, forward_method=method, hadamard_group_size=h, store_master_weights=True)
    layer = FPQuantLinear(K, N, FPQuantConfig(backward_dtype=FPQuantDtype.MXFP8, **cfg), bias=bias, device=d, dtype=torch.bfloat16)
    twin = FPQuantLinear(K, N, FPQuantConfig(backward_dtype=FPQuantDtype.BF16, **cfg), bias=bias, device=d, dtype=torch.bfloat16)
    w = inputs.normal_weight(N, K, seed=1).to(d)
    for m in (layer, twin):
        m.weight.data.copy_(w)
        if bias:
            m.bias.data.copy_(torch.linspace(-1, 1, N))
        m.pre_forward()
    # (quest with a 2-D input: like the reference, the function asks for the activation's clip mask only when
    # the flattened input itself requires grad, which a flattened view of a 3-D input does not, linear_fns.py:27-40)
    x = inputs.outlier_activations(tokens, K, seed=2).to(d)
    x = (x if method == "quest" else x.view(4, 50, K)).requires_grad_(True)
    y = layer(x)
    with torch.no_grad():
        y_twin = twin(x.detach())
        if bias:      # the twin adds the bias to the fp32 accumulator, this path to the rounded product
            assert torch.allclose(y.float(), y_twin.float(), rtol=2.0 ** -6, atol=2.0 ** -6)   # one bf16 ulp of the product before the bias cancels it
        else:
            assert torch.equal(y, y_twin)
    gy = (torch.randn(tokens, N, generator=torch.Generator().manual_seed(3)) * 0.01).bfloat16().to(d).view(y.shape)
    y.backward(gy)

    # reference: exact products on the operands the forward pass used
    H = layer.forward_hadamard_matrix
    with torch.no_grad():      # (tensors that require grad: that is what makes forward_quantize return the masks)
        xq, xs, xm = forward_quantize(x.detach().flatten(end_dim=-2).requires_grad_(True), H, layer.act_global_scale,
                                      FPQuantDtype.MXFP4, method)
        wq, ws, wm = forward_quantize(layer.weight, H, layer.weight_global_scale, FPQuantDtype.MXFP4, method)

    def dq(q, s, rows):
        sb = s.view(torch.uint8)[:rows, : K // 32].cpu()
        return fp4.dequantize(fp4.unpack_codes(q.cpu()), fp4.decode_scale_bytes(sb, "mxfp4"), 32).double()

    x_eff = dq(xq, xs, tokens) / float(layer.act_global_scale)
    w_eff = dq(wq, ws, N) / float(layer.weight_global_scale)
    g = gy.flatten(end_dim=-2).cpu().double()
    Hd = H.cpu().double()
    gi = g @ w_eff
    gw = g.t() @ x_eff
    if method == "quest":
        assert xm is not None and wm is not None
        gi = gi * _unpack_mask(xm).cpu().double()
        gw = gw * _unpack_mask(wm).cpu().double()
    gi = (gi.view(-1, h) @ Hd.t()).view(tokens, K)
    gw = (gw.view(-1, h) @ Hd.t()).view(N, K)

    def rel(a, b):
        return float((a.cpu().double() - b).norm() / b.norm())

    ri, rw = rel(x.grad.flatten(end_dim=-2), gi), rel(layer.weight.grad, gw)
    print(f"{method} bias={bias}: grad_input {ri:.4f}, grad_weight {rw:.4f} relative to the exact products")
    assert ri < 0.04 and rw < 0.04
    if bias:
        assert torch.allclose(layer.bias.grad.float().cpu(), g.sum(0).float(), rtol=2e-2, atol=1e-3)
    # and close to the plain bf16 gradient of the twin (straight-through estimate of the same quantity)
    x2 = x.detach().clone().requires_grad_(True)
    twin(x2).backward(gy)
    print(f"   against the bf16 backward of the unquantised operands: grad_input {rel(x.grad, x2.grad.cpu().double()):.3f}, "
          f"grad_weight {rel(layer.weight.grad, twin.weight.grad.cpu().double()):.3f}")


def test_mxfp8_backward_without_master_weights_raises(cuda_device):
    from fpq_b200.fp_quant import FPQuantConfig, FPQuantDtype, FPQuantLinear

    d = cuda_device
    layer = FPQuantLinear(128, 128, FPQuantConfig(forward_dtype=FPQuantDtype.MXFP4, forward_method="abs_max",
                                                   backward_dtype=FPQuantDtype.MXFP8, hadamard_group_size=32,
                                                   store_master_weights=False), bias=False, device=d, dtype=torch.bfloat16)
    layer.pre_forward()
    x = torch.randn(64, 128, device=d, dtype=torch.bfloat16, requires_grad=True)
    y = layer(x)
    assert y.shape == (64, 128)
    with pytest.raises(NotImplementedError):
        y.sum().backward()


# ------------------------------------------------------------------------------------------- MXFP4 backward
@pytest.mark.parametrize("shape", [(128, 128), (70, 256), (257, 96), (96, 1024)])
def test_fp4_transpose_dequant_matches_the_oracle(cuda_device, shape):
    from fpq_b200 import ops

    rows, cols = shape
    g = torch.Generator().manual_seed(rows + 5 * cols)
    codes = torch.randint(0, 256, (rows, cols // 2), generator=g, dtype=torch.uint8)
    sb = torch.randint(100, 140, (rows, cols // 32), generator=g, dtype=torch.uint8)
    sb[::5, 0] = 3                                            # extreme exponents take the kernel's general path
    sb[1::5, -1] = 250
    for alpha in (3.0, 1.0, 0.37):
        want = mxfp8.fp4_transpose_dequant(codes, sb, alpha)
        got = ops.mxfp4_transpose_dequant(codes.to(cuda_device), sb.to(cuda_device), torch.tensor([alpha], device=cuda_device))
        assert got.shape == (cols, rows)
        assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16)), alpha


def test_backward_requantisation_ops(cuda_device):
    """`backward_t_bf16` and `backward_qt_bf16` (qutlass_ops.py:218-274) are the transposes followed by the
    forward quantiser: same codes and scales as transposing on the host and calling `fused_quantize_mx_op`."""
    from fpq_b200 import ops
    from fpq_b200.fp_quant.module.qutlass_ops import backward_qt_bf16_op, backward_t_bf16_op, fused_quantize_mx_op
    from tests import inputs

    d = cuda_device
    m, n = 256, 384
    H = (fp4_hadamard(32) * torch.tensor([1.0, -1.0] * 16)).bfloat16().to(d)       # column signs: a dense rotation
    x = inputs.outlier_activations(m, n, seed=8).to(d)
    q, s = backward_t_bf16_op(x, H)
    q_ref, s_ref, _ = fused_quantize_mx_op(x.t().contiguous(), H, "abs_max", False)
    assert q.shape == (n, m // 2) and torch.equal(q, q_ref) and torch.equal(s.view(torch.uint8), s_ref.view(torch.uint8))

    xq, xs, _ = fused_quantize_mx_op(x, H, "abs_max", False)
    q2, s2 = backward_qt_bf16_op(xq, xs, H, torch.tensor([3.0], device=d))
    xt = mxfp8.fp4_transpose_dequant(xq.cpu(), xs.view(torch.uint8)[:m, : n // 32].cpu(), 3.0).to(d)
    q2_ref, s2_ref, _ = fused_quantize_mx_op(xt, H, "abs_max", False)
    assert q2.shape == (n, m // 2) and torch.equal(q2, q2_ref) and torch.equal(s2.view(torch.uint8), s2_ref.view(torch.uint8))


def fp4_hadamard(g):
    from fpq_b200.rotation import sylvester

    return (sylvester(g) * g ** -0.5).float()


@pytest.mark.parametrize("method", ["abs_max", "quest"])
def test_mxfp4_backward_gradients(cuda_device, method):
    """`FPQuantLinear(backward_dtype=MXFP4, store_master_weights=True)` (FPQuant4x4MasterFn): gradients against
    the exact products of the upstream gradient with the dequantised forward operands.  Every operand of the
    two gradient GEMMs passes through a second MXFP4 quantisation here, so the estimate carries FP4 noise
    (about 10 % per operand in norm); the bound checks the scaling and the data flow, the printed figures
    give the size of the noise."""
    from fpq_b200.fp_quant import FPQuantConfig, FPQuantDtype, FPQuantLinear
    from fpq_b200.fp_quant.module.linear_fns import _unpack_mask, forward_quantize
    from tests import inputs

    d = cuda_device
    tokens, K, N, h = 200, 256, 384, 32
    layer = FPQuantLinear(K, N, FPQuantConfig(forward_dtype=FPQuantDtype.MXFP4, forward_method=method, hadamard_group_size=h,
                                              store_master_weights=True, backward_dtype=FPQuantDtype.MXFP4),
                          bias=True, device=d, dtype=torch.bfloat16)
    layer.weight.data.copy_(inputs.normal_weight(N, K, seed=1).to(d))
    layer.pre_forward()
    x = inputs.outlier_activations(tokens, K, seed=2).to(d).requires_grad_(True)
    y = layer(x)
    gy = (torch.randn(tokens, N, generator=torch.Generator().manual_seed(3)) * 0.01).bfloat16().to(d)
    torch.manual_seed(0)
    y.backward(gy)

    H = layer.forward_hadamard_matrix
    with torch.no_grad():
        xq, xs, xm = forward_quantize(x.detach().requires_grad_(True), H, layer.act_global_scale, FPQuantDtype.MXFP4, method)
        wq, ws, wm = forward_quantize(layer.weight, H, layer.weight_global_scale, FPQuantDtype.MXFP4, method)

    def dq(q, s, rows):
        sb = s.view(torch.uint8)[:rows, : K // 32].cpu()
        return fp4.dequantize(fp4.unpack_codes(q.cpu()), fp4.decode_scale_bytes(sb, "mxfp4"), 32).double()

    g = gy.cpu().double()
    gi = g @ (dq(wq, ws, N) / float(layer.weight_global_scale))
    gw = g.t() @ (dq(xq, xs, tokens) / float(layer.act_global_scale))
    if method == "quest":
        gi, gw = gi * _unpack_mask(xm).cpu().double(), gw * _unpack_mask(wm).cpu().double()
    Hd = H.cpu().double()
    gi, gw = (gi.view(-1, h) @ Hd.t()).view(tokens, K), (gw.view(-1, h) @ Hd.t()).view(N, K)

    def rel(a, b):
        return float((a.cpu().double() - b).norm() / b.norm())

    ri, rw = rel(x.grad, gi), rel(layer.weight.grad, gw)
    cos_i = float((x.grad.cpu().double() * gi).sum() / (x.grad.cpu().double().norm() * gi.norm()))
    print(f"{method}: grad_input {ri:.3f} (cosine {cos_i:.4f}), grad_weight {rw:.3f} relative to the exact products")
    assert ri < 0.3 and rw < 0.3 and cos_i > 0.95
    assert torch.allclose(layer.bias.grad.float().cpu(), g.sum(0).float(), rtol=2e-2, atol=1e-3)


@pytest.mark.parametrize("group", [0, 16, 32])
@pytest.mark.parametrize("shape", [(256, 384), (200, 320), (1000, 1032), (33, 8)])
def test_transposing_quantiser_equals_quantising_the_transpose(cuda_device, shape, group):
    """`fpq_quantize_transposed` (the one-pass form of `backward_t_bf16`, qutlass_ops.py:218-245): same codes and
    scale bytes as zero-padding the token axis, transposing on the host and quantising, in both scale layouts."""
    from fpq_b200 import ops
    from tests import inputs

    t, n = shape
    d = cuda_device
    x = inputs.outlier_activations(t, n, seed=t + n).to(d)
    tp = -(-t // 128) * 128
    xt = torch.zeros(n, tp, dtype=torch.bfloat16, device=d)
    xt[:, :t] = x.t()
    want_q, want_s, _ = ops.quantize(xt, "mxfp4", group)
    got_q, got_s = ops.quantize_transposed(x, group, pad_to=128)
    assert got_q.shape == (n, tp // 2) and torch.equal(got_q, want_q) and torch.equal(got_s, want_s)
    want_q2, want_s2, _ = ops.quantize(xt, "mxfp4", group, swizzled=True)
    got_q2, got_s2 = ops.quantize_transposed(x, group, pad_to=128, swizzled=True)
    assert torch.equal(got_q2, want_q2) and torch.equal(got_s2.flatten(), want_s2.flatten())


def test_backward_t_op_takes_the_one_pass_form_for_the_hadamard_matrix(cuda_device):
    from fpq_b200.fp_quant.module.qutlass_ops import backward_t_bf16_op, fused_quantize_mx_op
    from tests import inputs

    d = cuda_device
    H = fp4_hadamard(32).bfloat16().to(d)
    x = inputs.outlier_activations(256, 384, seed=9).to(d)
    q, s = backward_t_bf16_op(x, H)
    q_ref, s_ref, _ = fused_quantize_mx_op(x.t().contiguous(), H, "abs_max", False)
    assert torch.equal(q, q_ref) and torch.equal(s.view(torch.uint8), s_ref.view(torch.uint8))


def test_transposing_dequantiser_pads_the_contraction_axis(cuda_device):
    from fpq_b200 import ops

    g = torch.Generator().manual_seed(12)
    codes = torch.randint(0, 256, (200, 64), generator=g, dtype=torch.uint8)
    sb = torch.randint(110, 135, (200, 4), generator=g, dtype=torch.uint8)
    got = ops.mxfp4_transpose_dequant(codes.to(cuda_device), sb.to(cuda_device), torch.tensor([3.0], device=cuda_device), pad_to=128)
    want = mxfp8.fp4_transpose_dequant(codes, sb, 3.0)
    assert got.shape == (128, 256)
    assert torch.equal(got[:, :200].cpu().view(torch.int16), want.view(torch.int16)) and float(got[:, 200:].abs().max()) == 0.0
