"""GPU parity of the fused rotate + FP4 quantise kernels against the CPU oracle (bit-exact)."""
import os
import pytest
import torch

from oracle import fp4
from tests import inputs

pytestmark = pytest.mark.gpu


def _oracle_quant(y, fmt, gs=None):
    return fp4.quantize(y, fmt, gs)


def _global_scale(y):
    return fp4.nvfp4_global_scale(y.abs().max())


@pytest.mark.parametrize("group", [16, 32, 64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rotate_matches_butterfly(cuda_device, group, dtype):
    from fpq_b200 import ops

    x = inputs.normal_weight(67, 512, seed=3, std=1.0, dtype=dtype)
    want = fp4.fwht_butterfly(x, group)
    got = ops.rotate_hadamard(x.to(cuda_device), group, out_dtype=torch.float32).cpu()
    assert torch.equal(got, want)
    got_same = ops.rotate_hadamard(x.to(cuda_device), group).cpu()
    assert torch.equal(got_same, want.to(dtype))


@pytest.mark.parametrize("group", [16, 64])
def test_rotate_dense_matches_sequential_sum(cuda_device, group):
    from fpq_b200 import ops

    x = inputs.normal_weight(33, 256, seed=5, std=1.0)
    perm = fp4.gsr_permutation(group)
    m = fp4.hadamard_matrix(group)[:, perm].bfloat16()
    want = fp4.rotate_dense(x, m)
    got = ops.rotate_dense(x.to(cuda_device), m.to(cuda_device), out_dtype=torch.float32).cpu()
    assert torch.equal(got, want)


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("hgroup", [0, 16, 32, 64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 128), (3, 256), (130, 384), (512, 4096)])
def test_quantize_bit_exact(cuda_device, fmt, hgroup, dtype, shape):
    from fpq_b200 import ops

    x = inputs.outlier_activations(*shape, seed=11, dtype=dtype)
    y = fp4.fwht_butterfly(x, hgroup) if hgroup else x.float()
    gs = _global_scale(y) if fmt == "nvfp4" else None
    want_codes, want_sb, want_s = _oracle_quant(y, fmt, gs)
    q, sb, sf = ops.quantize(x.to(cuda_device), fmt, hgroup, None if gs is None else gs.to(cuda_device),
                             scales_f32=True)
    assert torch.equal(sf.cpu(), want_s)
    assert torch.equal(sb.cpu(), want_sb)
    assert torch.equal(q.cpu(), want_codes)
    # same call writing the swizzled layout
    q2, sbz, _ = ops.quantize(x.to(cuda_device), fmt, hgroup, None if gs is None else gs.to(cuda_device),
                              swizzled=True)
    assert torch.equal(q2.cpu(), want_codes)
    assert torch.equal(sbz.cpu(), fp4.swizzle_scales(want_sb))
    assert torch.equal(ops.swizzle_scales(sb).cpu(), fp4.swizzle_scales(want_sb))


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
def test_quantize_edge_cases(cuda_device, fmt):
    """Ties, signed zeros, zero groups, maxima just below powers of two, extreme magnitudes."""
    from fpq_b200 import ops

    x = inputs.edge_case_rows(128)
    gs = torch.tensor([3.0]) if fmt == "nvfp4" else None
    want_codes, want_sb, want_s = _oracle_quant(x, fmt, gs)
    q, sb, sf = ops.quantize(x.to(cuda_device), fmt, 0, None if gs is None else gs.to(cuda_device), scales_f32=True)
    assert torch.equal(sf.cpu(), want_s)
    assert torch.equal(sb.cpu(), want_sb)
    assert torch.equal(q.cpu(), want_codes)


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("hgroup", [16, 32, 64, 128])
def test_rounding_boundaries_through_the_rotation(cuda_device, fmt, hgroup):
    """The edge rows above reach the quantiser unrotated.  These rows are built backwards from the rotated
    values (tests/inputs.py::rotation_boundary_probes), so the rotation is exact and every probe lands on or
    within a few grid steps of one of the seven E2M1 rounding boundaries after the kernel's own butterfly:
    this is where the MXFP4 single-multiply path (multiplier not a power of two for groups 32 and 128) could
    differ from the reference's division."""
    from fpq_b200 import ops

    x, t = inputs.rotation_boundary_probes(hgroup)
    y = fp4.fwht_butterfly(x, hgroup)
    assert torch.equal(y, t * torch.tensor(hgroup ** -0.5, dtype=torch.float32))      # the construction holds
    assert torch.equal(ops.rotate_hadamard(x.to(cuda_device), hgroup).cpu(), y)
    gs = _global_scale(y) if fmt == "nvfp4" else None
    want_codes, want_sb, want_s = _oracle_quant(y, fmt, gs)
    q, sb, sf = ops.quantize(x.to(cuda_device), fmt, hgroup, None if gs is None else gs.to(cuda_device),
                             scales_f32=True)
    assert torch.equal(sf.cpu(), want_s)
    assert torch.equal(sb.cpu(), want_sb)
    assert torch.equal(q.cpu(), want_codes)
    if fmt == "mxfp4":      # every code of the grid is hit, so both sides of every boundary were probed
        seen = set(fp4.unpack_codes(want_codes).flatten().tolist())
        assert seen >= set(range(1, 8)) | set(range(8, 16))


@pytest.mark.parametrize("fmt,hgroup", [("nvfp4", 128), ("mxfp4", 128), ("mxfp4", 32)])
def test_weight_round_trip_4096(cuda_device, fmt, hgroup):
    """The 4096 x 4096 N(0, 0.02^2) weight: codes, scales, global scale and MSE."""
    from fpq_b200 import ops

    w = inputs.normal_weight(4096, 4096, seed=0)
    y = fp4.fwht_butterfly(w, hgroup)
    wd = w.to(cuda_device)
    gs_d = None
    gs = None
    if fmt == "nvfp4":
        bits = ops.absmax_bits(wd, hgroup)
        gs_d = torch.full((1,), float("inf"), device=cuda_device)
        ops.global_scale_update(bits, gs_d)
        gs = _global_scale(y)
        assert torch.equal(gs_d.cpu(), gs)
    want_codes, want_sb, want_s = _oracle_quant(y, fmt, gs)
    q, sb, sf = ops.quantize(wd, fmt, hgroup, gs_d, scales_f32=True)
    assert torch.equal(sb.cpu(), want_sb)
    assert torch.equal(q.cpu(), want_codes)
    g = 16 if fmt == "nvfp4" else 32
    dq = ops.fake_quantize(wd, fmt, hgroup, gs_d).cpu().float()
    want_dq = fp4.dequantize(fp4.unpack_codes(want_codes), want_s, g)
    assert torch.equal(dq, want_dq.bfloat16().float())
    mse = ((want_dq - y) ** 2).mean().item()
    assert 1e-6 < mse < 1e-5


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("ste", [False, True])
def test_fake_quantize_fp32(cuda_device, fmt, ste):
    from fpq_b200 import ops

    x = inputs.outlier_activations(64, 512, seed=21, dtype=torch.float32)
    y = fp4.fwht_butterfly(x, 64)
    gs = _global_scale(y) if fmt == "nvfp4" else None
    codes, _, s = _oracle_quant(y, fmt, gs)
    dq = fp4.dequantize(fp4.unpack_codes(codes), s, 16 if fmt == "nvfp4" else 32)
    want = y + (dq - y) if ste else dq
    got = ops.fake_quantize(x.to(cuda_device), fmt, 64, None if gs is None else gs.to(cuda_device), ste=ste).cpu()
    assert torch.equal(got, want)


@pytest.mark.parametrize("group", [16, 32, 128])
def test_apply_scales_and_pack(cuda_device, group):
    from fpq_b200 import ops, _cabi as C

    x = inputs.outlier_activations(40, 256, seed=31, dtype=torch.float32)
    g = torch.Generator().manual_seed(32)
    s = torch.rand(40, 256 // group, generator=g) + 0.05
    codes = fp4.e2m1_codes(x, s, group)
    grid = fp4.code_values(codes)
    xd, sd = x.to(cuda_device), s.to(cuda_device)
    assert torch.equal(ops.apply_scales(xd, sd, group, C.OUT_CODES).cpu(), fp4.pack_codes(codes))
    got_grid = ops.apply_scales(xd, sd, group, C.OUT_GRID)
    assert torch.equal(got_grid.cpu(), grid)
    dq = fp4.dequantize(codes, s, group)
    assert torch.equal(ops.apply_scales(xd, sd, group, C.OUT_DEQUANT).cpu(), dq)
    assert torch.equal(ops.apply_scales(xd, sd, group, C.OUT_DEQUANT_STE).cpu(), x + (dq - x))
    assert torch.equal(ops.pack_grid(got_grid).cpu(), fp4.pack_codes(codes))


def test_bad_arguments_raise(cuda_device):
    from fpq_b200 import ops, _cabi as C

    x = torch.zeros(4, 48, device=cuda_device)
    with pytest.raises(C.FpqError):
        ops.quantize(x, "mxfp4", 32)
    with pytest.raises(RuntimeError):
        ops.quantize(torch.zeros(4, 64), "mxfp4", 32)
    with pytest.raises(C.FpqError):
        ops.quantize(torch.zeros(4, 64, device=cuda_device), "mxfp4", 24)


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_mse_observer_scales_match_the_reference(cuda_device, fmt):
    """fpq_mse_scales through Quantizer(observer="mse") against the golden scales of the unmodified reference
    (tests/golden/mse_<fmt>.npz).  The search compares sums of |x - xq| ** 2.4 over 100 candidates; the device
    powf and the summation order differ from torch-CPU in the last bits, which can only matter between two
    candidates whose errors agree to ~1e-6: at least 99.5 % of the groups must get the identical scale (all of
    them do on this tensor; the fraction is printed).  The all-zero group must come out as the reference's."""
    import numpy as np

    from fpq_b200.quantization import Quantizer

    d = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"mse_{fmt}.npz"))
    y, want = torch.from_numpy(d["rotated"]), torch.from_numpy(d["scales"])
    name, prec, group = ("nvfp", "e4m3", 16) if fmt == "nvfp4" else ("mxfp", "e8m0", 32)
    q = Quantizer(bits=4, format=name, granularity="group", observer="mse", group_size=group, scale_precision=prec)
    got, zeros = q.get_quantization_params(y.to(cuda_device))
    got = got.float().cpu()
    assert got.shape == want.shape and not bool(zeros.any())
    if fmt == "nvfp4":
        assert torch.equal(q.global_scale.cpu(), torch.from_numpy(d["global_scale"]))
    same = got == want
    frac = same.float().mean().item()
    print(f"{fmt}: MSE-observer scales identical to the reference on {frac:.5f} of the groups")
    assert frac >= 0.995
    assert torch.equal(got[3, 32 // group:64 // group], want[3, 32 // group:64 // group])       # the all-zero group

    def err(s):
        g = y.reshape(64, -1, group)
        codes = fp4.e2m1_codes(y, s, group)
        return (g - (fp4.code_values(codes).reshape(g.shape) * s.unsqueeze(-1))).abs().pow(2.4).sum(-1)

    e_got = err(got)
    # the observer must actually lower the error it searches on, against the min-max scales
    qmm = Quantizer(bits=4, format=name, granularity="group", observer="minmax", group_size=group, scale_precision=prec)
    mm, _ = qmm.get_quantization_params(y.to(cuda_device))
    assert e_got.sum() < err(mm.float().cpu()).sum()
    # and Quantizer.__call__ with those scales works as with any others
    out = q(y.to(cuda_device), got.to(cuda_device)).cpu()
    assert torch.allclose(out, fp4.dequantize(fp4.e2m1_codes(y, got, group), got, group), rtol=1e-6, atol=1e-9)


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("rows", [1, 64, 130])
def test_swizzled_pad_rows_are_written_by_the_kernel(cuda_device, fmt, rows):
    """The scale bytes of the rows between the tensor's end and the next multiple of 128 are zeroed by the
    quantise kernel itself: a buffer pre-filled with 0xFF comes back identical to the oracle's zero-padded
    layout, so callers need no memset before a launch."""
    from fpq_b200 import _cabi as C

    K = 512
    x = inputs.outlier_activations(rows, K, seed=51).to(cuda_device)
    g = 16 if fmt == "nvfp4" else 32
    gs = torch.tensor([5.0], device=cuda_device) if fmt == "nvfp4" else None
    pr = (rows + 127) // 128 * 128
    sb = torch.full((pr, K // g), 0xFF, dtype=torch.uint8, device=cuda_device)
    codes = torch.empty(rows, K // 2, dtype=torch.uint8, device=cuda_device)
    C.call("fpq_quantize", x.data_ptr(), C.DT_BF16, rows, K, 32, C.FMT_NVFP4 if fmt == "nvfp4" else C.FMT_MXFP4,
           None if gs is None else gs.data_ptr(), codes.data_ptr(), sb.data_ptr(), C.SCALES_SWIZZLED, None,
           torch.cuda.current_stream().cuda_stream)
    _, want_sb, _ = _oracle_quant(fp4.fwht_butterfly(x.cpu(), 32), fmt, None if gs is None else gs.cpu())
    assert torch.equal(sb.cpu(), fp4.swizzle_scales(want_sb))


@pytest.mark.parametrize("hgroup", [0, 32, 64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quest_quantize_bit_exact(cuda_device, hgroup, dtype):
    """forward_method = "quest": codes, E8M0 bytes (row-major and swizzled), the packed clip mask and the
    pseudo-quantised output against the oracle's restatement, which tests/test_oracle_cpu.py pins to the
    reference's Triton kernel."""
    from fpq_b200 import ops

    x = inputs.outlier_activations(130, 512, seed=61, dtype=dtype)
    x[3, 32:64] = 0
    x[5, :32] = 1.0
    y = fp4.fwht_butterfly(x, hgroup) if hgroup else x.float()
    want_codes, want_sb, want_s, want_mask = fp4.quest_quantize(y)
    q, sb, mask = ops.quantize_quest(x.to(cuda_device), hgroup, swizzled=False, return_mask=True)
    assert torch.equal(sb.cpu(), want_sb)
    assert torch.equal(q.cpu(), want_codes)
    assert torch.equal(mask.cpu(), fp4.pack_clip_mask(want_mask))
    q2, sbz, none = ops.quantize_quest(x.to(cuda_device), hgroup, swizzled=True)
    assert none is None and torch.equal(q2.cpu(), want_codes)
    assert torch.equal(sbz.cpu(), fp4.swizzle_scales(want_sb))
    dq, m2 = ops.fake_quantize_quest(x.to(cuda_device), hgroup)
    want_dq = fp4.dequantize(fp4.unpack_codes(want_codes), want_s, 32)
    assert torch.equal(dq.cpu().float(), want_dq.to(dtype).float())
    assert m2.dtype == torch.bool and torch.equal(m2.cpu(), want_mask)
    assert 0.5 < want_mask.float().mean().item() < 1.0          # the rule does clip: that is its point


@pytest.mark.parametrize("fmt,hgroup", [("mxfp4", 32), ("nvfp4", 16), ("nvfp4", 128), ("mxfp4", 0)])
@pytest.mark.parametrize("shape", [(3, 256), (130, 1024), (512, 4096)])
def test_fused_silu_mul_quantize(cuda_device, fmt, hgroup, shape):
    """fpq_quantize_silu_mul = fpq_quantize of bf16(bf16(silu(gate)) * up).  Two checks:
      * bit-exact against the two-step device computation (torch's silu and product on the GPU, then the
        quantise kernel): the fused kernel evaluates the activation with the same operations;
      * against the CPU oracle fed torch-CPU's bf16 activation: the two exponentials can differ in the last
        fp32 bit, which moves a bf16 rounding of the activation for a few elements in 10^5; every differing
        code must sit in a scale group whose activation input differs, and such groups must be rare."""
    from fpq_b200 import ops

    gate = inputs.outlier_activations(*shape, seed=71) * 4
    up = inputs.outlier_activations(*shape, seed=73)
    gs = torch.tensor([2.5]) if fmt == "nvfp4" else None
    gs_d = None if gs is None else gs.to(cuda_device)
    q, sb = ops.quantize_silu_mul(gate.to(cuda_device), up.to(cuda_device), fmt, hgroup, gs_d, swizzled=True)
    h_dev = torch.nn.functional.silu(gate.to(cuda_device)) * up.to(cuda_device)
    q2, sb2, _ = ops.quantize(h_dev, fmt, hgroup, gs_d, swizzled=True)
    assert torch.equal(q, q2) and torch.equal(sb, sb2)
    qr, sbr = ops.quantize_silu_mul(gate.to(cuda_device), up.to(cuda_device), fmt, hgroup, gs_d, swizzled=False)
    assert torch.equal(qr, q) and torch.equal(ops.swizzle_scales(sbr), sb)

    h_cpu = torch.nn.functional.silu(gate) * up                                  # bf16 on the CPU
    y = fp4.fwht_butterfly(h_cpu, hgroup) if hgroup else h_cpu.float()
    want_codes, want_sb, _ = _oracle_quant(y, fmt, gs)
    g = 16 if fmt == "nvfp4" else 32
    rot = max(hgroup, g)                      # an input element reaches every output of its rotation group
    in_diff = (h_cpu != h_dev.cpu()).reshape(shape[0], -1, rot).any(-1)
    code_diff = (fp4.unpack_codes(qr.cpu()) != fp4.unpack_codes(want_codes)).reshape(shape[0], -1, rot).any(-1)
    scale_diff = (sbr.cpu() != want_sb).reshape(shape[0], -1, rot // g).any(-1)
    assert not bool(((code_diff | scale_diff) & ~in_diff).any())
    assert in_diff.float().mean().item() < 2e-3
