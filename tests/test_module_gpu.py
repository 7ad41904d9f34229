"""GPU tests of the Python API mirror: Quantizer, HadamardTransform, FPQuantLinear and the op layer."""
import pytest
import torch

from oracle import fp4
from tests import inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt,group,prec", [("nvfp", 16, "e4m3"), ("mxfp", 32, "e8m0")])
def test_quantizer_api_matches_oracle(cuda_device, fmt, group, prec):
    from fpq_b200.quantization import Quantizer
    from fpq_b200.quantization.quant_ops import cast_scales_to_eXmY, pack_fp4_to_uint8

    w = inputs.normal_weight(96, 512, seed=2, dtype=torch.float32)
    q = Quantizer(bits=4, format=fmt, granularity="group", group_size=group, scale_precision=prec)
    wd = w.to(cuda_device)
    scales, zeros = q.get_quantization_params(wd)
    kfmt = "nvfp4" if fmt == "nvfp" else "mxfp4"
    gs = fp4.nvfp4_global_scale(w.abs().max()) if fmt == "nvfp" else None
    want_codes, want_sb, want_s = fp4.quantize(w, kfmt, gs)
    assert torch.equal(scales.cpu(), want_s) and not zeros.any()
    if fmt == "nvfp":
        assert torch.equal(q.global_scale.cpu(), gs)
    grid = q.quantize(wd, scales, zeros)
    assert torch.equal(pack_fp4_to_uint8(grid).cpu(), want_codes)
    dq = q.dequantize(grid, scales, zeros)
    want_dq = fp4.dequantize(fp4.unpack_codes(want_codes), want_s, group)
    assert torch.equal(dq.cpu(), want_dq)
    assert torch.equal(q(wd, scales, zeros).cpu(), w + (want_dq - w))
    stored = cast_scales_to_eXmY(scales * q.global_scale.to(cuda_device), prec)
    assert torch.equal(stored.cpu(), want_sb)
    # running minimum of the tensor scale, then frozen
    if fmt == "nvfp":
        q.get_quantization_params(wd * 4)
        assert torch.equal(q.global_scale.cpu(), fp4.nvfp4_global_scale((w * 4).abs().max()))
        q._track_global_scale = False
        q.get_quantization_params(wd * 100)
        assert torch.equal(q.global_scale.cpu(), fp4.nvfp4_global_scale((w * 4).abs().max()))


def test_quantizer_column_mode(cuda_device):
    """group_size=None with one scale per element: the call GPTQ makes per column."""
    from fpq_b200.quantization import Quantizer

    q = Quantizer(bits=4, format="nvfp", granularity="group", group_size=16, scale_precision="e4m3")
    q.group_size = None
    g = torch.Generator().manual_seed(1)
    col = torch.randn(256, generator=g)
    s = torch.rand(256, generator=g) + 0.1
    want = fp4.code_values(fp4.e2m1_codes(col.unsqueeze(-1), s.unsqueeze(-1), 1).squeeze(-1))
    got = q.quantize(col.to(cuda_device), s.to(cuda_device))
    assert torch.equal(got.cpu(), want)


def test_unsupported_configurations_raise():
    from fpq_b200.quantization import Quantizer

    with pytest.raises(NotImplementedError):
        Quantizer(bits=4, format="int", granularity="group", group_size=128)
    with pytest.raises(NotImplementedError):
        Quantizer(bits=4, format="nvfp", granularity="group", group_size=32, scale_precision="e4m3")
    with pytest.raises(NotImplementedError):
        Quantizer(bits=4, format="mxfp", granularity="channel", scale_precision="e8m0")
    Quantizer(bits=4, format="nvfp", granularity="group", group_size=16, scale_precision="e4m3", observer="mse")


@pytest.mark.parametrize("group", [16, 32, 64, 128])
def test_hadamard_transform_module(cuda_device, group):
    from fpq_b200.transforms import HadamardTransform, build_transform, get_transform_matrix

    x = inputs.normal_weight(8, 256, seed=4, std=1.0).view(2, 4, 256)
    t = build_transform("hadamard", group_size=group, size=256, device=cuda_device)
    assert isinstance(t, HadamardTransform)
    y = t(x.to(cuda_device), inv_t=True)
    assert torch.equal(y.cpu(), fp4.fwht_butterfly(x, group).bfloat16())
    m = get_transform_matrix("hadamard", group, cuda_device, torch.float32).cpu()
    assert torch.allclose(m, fp4.hadamard_matrix(group), atol=1e-7)


@pytest.mark.parametrize("dtype_name,hgroup", [("mxfp4", 32), ("mxfp4", 128), ("nvfp4", 16), ("nvfp4", 64)])
@pytest.mark.parametrize("bias", [False, True])
def test_fpquant_linear_forward(cuda_device, dtype_name, hgroup, bias):
    from fpq_b200.fp_quant import FPQuantConfig, FPQuantDtype, FPQuantLinear

    K, N = 512, 384
    fd = FPQuantDtype.MXFP4 if dtype_name == "mxfp4" else FPQuantDtype.NVFP4
    cfg = FPQuantConfig(forward_dtype=fd, forward_method="abs_max", backward_dtype=FPQuantDtype.BF16,
                        hadamard_group_size=hgroup)
    layer = FPQuantLinear(K, N, cfg, bias=bias, device=cuda_device, dtype=torch.bfloat16)
    w = inputs.normal_weight(N, K, seed=3)
    b = inputs.normal_weight(1, N, seed=8, std=0.1)[0]
    layer.weight.data.copy_(w)
    if bias:
        layer.bias.data.copy_(b)
    layer.pre_forward()
    assert layer.weight is None and layer.qweight.shape == (N, K // 2)
    x = inputs.outlier_activations(2 * 37, K, seed=1).view(2, 37, K)
    y = layer(x.to(cuda_device))
    assert y.shape == (2, 37, N) and y.dtype == torch.bfloat16

    gs = torch.tensor([3.0])
    xr, wr = fp4.fwht_butterfly(x.view(-1, K), hgroup), fp4.fwht_butterfly(w, hgroup)
    xq, xs, _ = fp4.quantize(xr, dtype_name, gs)
    wq, ws, _ = fp4.quantize(wr, dtype_name, gs)
    assert torch.equal(layer.qweight.cpu(), wq)
    g = 16 if dtype_name == "nvfp4" else 32
    assert torch.equal(layer.scales.view(torch.uint8).cpu()[:N, : K // g], ws)
    # alpha with the reference's rounding order: 1 / (3 * 3) in the bf16 of the buffers, then fp32
    alpha = float((1.0 / (torch.tensor([3.0]).bfloat16() * torch.tensor([3.0]).bfloat16())).float())
    assert alpha == 0.111328125 and float(layer._gemm_alpha()) == alpha
    want = fp4.fp4_matmul(xq, wq, xs, ws, alpha, dtype_name).float()
    if bias:
        want = (want.bfloat16() + b).float()
    got = y.cpu().float().view(-1, N)
    tol = 2.0 ** -6 * want.abs() + 2.0 ** -9 * want.abs().max()
    assert not ((got - want).abs() > tol).any()


def test_reference_named_ops_keep_row_major_contract(cuda_device):
    from fpq_b200.fp_quant.module.linear_fns import forward_gemm, forward_quantize
    from fpq_b200.fp_quant.module.linear import get_hadamard_matrix
    from fpq_b200.fp_quant import FPQuantDtype

    M, K, N = 70, 256, 128
    x = inputs.outlier_activations(M, K, seed=5).to(cuda_device)
    w = inputs.normal_weight(N, K, seed=6).to(cuda_device)
    h = get_hadamard_matrix(32, torch.bfloat16, cuda_device)
    gs = torch.tensor([3.0], device=cuda_device)
    for dt, g, st in ((FPQuantDtype.MXFP4, 32, torch.float8_e8m0fnu), (FPQuantDtype.NVFP4, 16, torch.float8_e4m3fn)):
        xq, xs, mask = forward_quantize(x, h, gs, dt, "abs_max")
        wq, ws, _ = forward_quantize(w, h, gs, dt, "abs_max")
        assert xq.shape == (M, K // 2) and xs.shape == (128, K // g) and xs.dtype == st and mask is None
        y = forward_gemm(xq, wq, xs, ws, torch.tensor([1 / 9.0], device=cuda_device), dt)
        assert y.shape == (M, N) and y.dtype == torch.bfloat16
        fmt = "mxfp4" if dt == FPQuantDtype.MXFP4 else "nvfp4"
        xr, wr = fp4.fwht_butterfly(x.cpu(), 32), fp4.fwht_butterfly(w.cpu(), 32)
        oq, os_, _ = fp4.quantize(xr, fmt, torch.tensor([3.0]))
        wq_o, ws_o, _ = fp4.quantize(wr, fmt, torch.tensor([3.0]))
        assert torch.equal(xs.view(torch.uint8).cpu()[:M], os_)
        want = fp4.fp4_matmul(oq, wq_o, os_, ws_o, 1 / 9.0, fmt).float()
        tol = 2.0 ** -7 * want.abs() + 2.0 ** -10 * want.abs().max()
        assert not ((y.cpu().float() - want).abs() > tol).any()


def test_gsr_and_identity_rotations(cuda_device):
    from fpq_b200.fp_quant.module.linear import get_gsr_matrix, get_identity_matrix
    from fpq_b200.fp_quant.module.qutlass_ops import fused_quantize_blocked_op

    x = inputs.outlier_activations(64, 256, seed=7)
    xd = x.to(cuda_device)
    gs = torch.tensor([3.0], device=cuda_device)
    eye = get_identity_matrix(32, torch.bfloat16, cuda_device)
    q, sb = fused_quantize_blocked_op(xd, eye, gs, False)
    oq, os_, _ = fp4.quantize(x.float(), "mxfp4")
    assert torch.equal(q.cpu(), oq) and torch.equal(sb.cpu(), fp4.swizzle_scales(os_))
    gsr = get_gsr_matrix(32, torch.bfloat16, cuda_device)
    q, sb = fused_quantize_blocked_op(xd, gsr, gs, False)
    xr = fp4.rotate_dense(x, gsr.cpu())
    oq, os_, _ = fp4.quantize(xr, "mxfp4")
    assert torch.equal(q.cpu(), oq) and torch.equal(sb.cpu(), fp4.swizzle_scales(os_))


def test_pseudoquant_linear(cuda_device):
    from fpq_b200.fp_quant import FPQuantConfig, FPQuantDtype, FPQuantLinear

    K, N = 256, 128
    cfg = FPQuantConfig(forward_dtype=FPQuantDtype.NVFP4, forward_method="abs_max", backward_dtype=FPQuantDtype.BF16,
                        hadamard_group_size=16, pseudoquantization=True)
    layer = FPQuantLinear(K, N, cfg, bias=False, device=cuda_device, dtype=torch.bfloat16)
    w = inputs.normal_weight(N, K, seed=3)
    layer.weight.data.copy_(w)
    layer.pre_forward()
    wr = fp4.fwht_butterfly(w, 16)
    q, sb, s = fp4.quantize(wr, "nvfp4", torch.tensor([3.0]))
    assert torch.equal(layer.dqweight.cpu(), fp4.dequantize(fp4.unpack_codes(q), s, 16).bfloat16())
    x = inputs.outlier_activations(32, K, seed=1)
    y = layer(x.to(cuda_device))
    exact = x.float() @ w.float().t()
    assert (y.cpu().float() - exact).norm() / exact.norm() < 0.25


@pytest.mark.parametrize("bias", [False, True])
def test_fpquant_linear_with_the_default_quest_method(cuda_device, bias):
    """FPQuantConfig's defaults (MXFP4, forward_method = "quest", Hadamard 32) with a bf16 backward: the
    configuration a user gets without arguments (inference_lib/src/fp_quant/utils/config.py:17-27).  Weight
    codes and scale bytes bit-exact against the oracle's QuEST rule, tensor scales 1.0 (linear.py:190-196),
    output within bf16 rounding of the fp64 product of the decoded operands."""
    from fpq_b200.fp_quant import FPQuantConfig, FPQuantDtype, FPQuantLinear

    K, N = 512, 384
    cfg = FPQuantConfig(backward_dtype=FPQuantDtype.BF16)
    assert cfg.forward_method == "quest" and cfg.forward_dtype == FPQuantDtype.MXFP4 and cfg.hadamard_group_size == 32
    layer = FPQuantLinear(K, N, cfg, bias=bias, device=cuda_device, dtype=torch.bfloat16)
    w = inputs.normal_weight(N, K, seed=3)
    b = inputs.normal_weight(1, N, seed=8, std=0.1)[0]
    layer.weight.data.copy_(w)
    if bias:
        layer.bias.data.copy_(b)
    layer.pre_forward()
    assert float(layer.weight_global_scale) == 1.0 and float(layer.act_global_scale) == 1.0
    wq, ws, _, _ = fp4.quest_quantize(fp4.fwht_butterfly(w, 32))
    assert torch.equal(layer.qweight.cpu(), wq)
    assert torch.equal(layer.scales.view(torch.uint8).cpu()[:N, : K // 32], ws)
    x = inputs.outlier_activations(2 * 37, K, seed=1).view(2, 37, K)
    y = layer(x.to(cuda_device))
    xq, xs, _, _ = fp4.quest_quantize(fp4.fwht_butterfly(x.view(-1, K), 32))
    want = fp4.fp4_matmul(xq, wq, xs, ws, 1.0, "mxfp4").float()
    if bias:
        want = (want.bfloat16() + b).float()
    got = y.cpu().float().view(-1, N)
    tol = 2.0 ** -6 * want.abs() + 2.0 ** -9 * want.abs().max()
    assert not ((got - want).abs() > tol).any()
    exact = x.view(-1, K).float() @ w.float().t() + (b.float() if bias else 0.0)
    assert (got - exact).norm() / exact.norm() < 0.3


def test_quest_mask_and_pseudoquant_through_the_reference_api(cuda_device):
    """`forward_quantize(..., "quest")` hands back the packed clip mask when the input requires grad
    (linear_fns.py:34-40), and `forward_pseudoquantize` returns the element-wise one (pseudoquant_linear_fns.py:
    19-34); both are the oracle's."""
    from fpq_b200.fp_quant import FPQuantDtype
    from fpq_b200.fp_quant.module.linear import get_hadamard_matrix
    from fpq_b200.fp_quant.module.linear_fns import forward_quantize
    from fpq_b200.fp_quant.module.pseudoquant_linear_fns import forward_pseudoquantize

    M, K = 70, 256
    x = inputs.outlier_activations(M, K, seed=5)
    h = get_hadamard_matrix(64, torch.bfloat16, cuda_device)
    gs = torch.tensor([1.0], device=cuda_device)
    want_codes, want_sb, want_s, want_mask = fp4.quest_quantize(fp4.fwht_butterfly(x, 64))
    q, s, mask = forward_quantize(x.to(cuda_device).requires_grad_(True), h, gs, FPQuantDtype.MXFP4, "quest")
    assert s.dtype == torch.float8_e8m0fnu and s.shape == (128, 8) and mask.shape == (M, K // 8)
    assert torch.equal(q.cpu(), want_codes) and torch.equal(s.view(torch.uint8).cpu()[:M], want_sb)
    assert torch.equal(mask.cpu(), fp4.pack_clip_mask(want_mask))
    _, _, none = forward_quantize(x.to(cuda_device), h, gs, FPQuantDtype.MXFP4, "quest")
    assert none is None
    y, m = forward_pseudoquantize(x.to(cuda_device), h, gs, FPQuantDtype.MXFP4, "quest")
    assert torch.equal(y.cpu().float(), fp4.dequantize(fp4.unpack_codes(want_codes), want_s, 32).bfloat16().float())
    assert torch.equal(m.cpu(), want_mask)
    with pytest.raises(AssertionError):
        forward_pseudoquantize(x.to(cuda_device), h, gs, FPQuantDtype.NVFP4, "quest")


def test_ops_live_in_the_reference_namespace_and_trace_under_torch_compile(cuda_device):
    """The reference registers its operators as torch custom ops `fp_quant::*` with fake implementations so that
    torch.compile(fullgraph=True) traces through a quantised layer (README.md:39; qutlass_ops.py:36, :54, :111).
    Same names here; `torch.library.opcheck` validates schema and fake kernels, and a layer compiled with
    fullgraph=True (graph capture and fake-tensor propagation; backend aot_eager, so no code generator is
    involved) returns what the eager layer returns."""
    from fpq_b200.fp_quant import FPQuantConfig, FPQuantDtype, FPQuantLinear
    from fpq_b200.fp_quant.module import qutlass_ops
    from fpq_b200.fp_quant.module.linear import get_hadamard_matrix

    assert qutlass_ops.NAMESPACE == "fp_quant"
    for name in ("fused_quantize_mx_op", "fused_quantize_nv_op", "matmul_mxf4_bf16_tn_op", "matmul_nvf4_bf16_tn_op"):
        assert hasattr(torch.ops.fp_quant, name), name
    x = inputs.outlier_activations(70, 256, seed=5).to(cuda_device)
    h = get_hadamard_matrix(32, torch.bfloat16, cuda_device)
    gs = torch.tensor([3.0], device=cuda_device)
    checks = ("test_schema", "test_faketensor", "test_autograd_registration")
    torch.library.opcheck(torch.ops.fp_quant.fused_quantize_mx_op.default, (x, h, "abs_max", False), test_utils=checks)
    torch.library.opcheck(torch.ops.fp_quant.fused_quantize_mx_op.default, (x, h, "quest", True), test_utils=checks)
    torch.library.opcheck(torch.ops.fp_quant.fused_quantize_nv_op.default, (x, h, gs), test_utils=checks)
    torch.library.opcheck(torch.ops.fpq_b200.fused_quantize_blocked_op.default, (x, h, gs, False, 0, False), test_utils=checks)
    q, s, _ = torch.ops.fp_quant.fused_quantize_mx_op(x, h, "abs_max", False)
    wq, ws, _ = torch.ops.fp_quant.fused_quantize_mx_op(inputs.normal_weight(128, 256, seed=3).to(cuda_device), h, "abs_max", False)
    alpha = torch.tensor([1 / 9.0], device=cuda_device)
    # (the schema check perturbs its inputs with arithmetic that torch does not implement for float8_e8m0fnu)
    torch.library.opcheck(torch.ops.fp_quant.matmul_mxf4_bf16_tn_op.default, (q, wq, s, ws, alpha), test_utils=checks[1:])

    for method in ("abs_max", "quest"):
        cfg = FPQuantConfig(forward_method=method, backward_dtype=FPQuantDtype.BF16)
        layer = FPQuantLinear(256, 128, cfg, bias=True, device=cuda_device, dtype=torch.bfloat16)
        layer.weight.data.copy_(inputs.normal_weight(128, 256, seed=3))
        layer.bias.data.copy_(inputs.normal_weight(1, 128, seed=8, std=0.1)[0])
        layer.pre_forward()
        with torch.no_grad():
            eager = layer(x)
            compiled = torch.compile(layer, fullgraph=True, backend="aot_eager")(x)
        assert torch.equal(eager, compiled)


@pytest.mark.parametrize("dtype_name,hgroup", [("mxfp4", 32), ("nvfp4", 128)])
def test_gated_mlp_with_fused_activation(cuda_device, dtype_name, hgroup):
    """`fuse_gated_mlp_activation` on a Llama-style MLP whose linears are real-quantised FPQuantLinear layers:
    the patched module returns bit for bit what the unpatched one (separate SiLU * up kernel, then the
    down-projection's own rotate + quantise) returns."""
    import torch.nn as nn

    from fpq_b200.fp_quant import (FPQuantConfig, FPQuantDtype, fuse_gated_mlp_activation,
                                   replace_quantize_with_fp_quant_linear)

    class MLP(nn.Module):
        def __init__(self, d, f):
            super().__init__()
            self.gate_proj, self.up_proj = nn.Linear(d, f, bias=False), nn.Linear(d, f, bias=False)
            self.down_proj = nn.Linear(f, d, bias=True)
            self.act_fn = nn.SiLU()

        def forward(self, x):
            return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))

    torch.manual_seed(0)
    mlp = MLP(256, 512).to(device=cuda_device, dtype=torch.bfloat16)
    fd = FPQuantDtype.MXFP4 if dtype_name == "mxfp4" else FPQuantDtype.NVFP4
    cfg = FPQuantConfig(forward_dtype=fd, forward_method="abs_max", backward_dtype=FPQuantDtype.BF16,
                        hadamard_group_size=hgroup, modules_to_not_convert=[])
    replace_quantize_with_fp_quant_linear(mlp, cfg)
    x = inputs.outlier_activations(2 * 70, 256, seed=1).view(2, 70, 256).to(cuda_device)
    with torch.no_grad():
        want = mlp(x)
        assert fuse_gated_mlp_activation(mlp) == 1
        got = mlp(x)
        compiled = torch.compile(mlp, fullgraph=True, backend="aot_eager")(x)
    assert torch.equal(got, want) and torch.equal(compiled, want)
