"""CPU tests: the oracle against the committed golden vectors (made from the unmodified
reference by tests/golden/make_golden.py) and, when the reference tree is present, live."""
import os

import numpy as np
import pytest
import torch

from oracle import fp4, gptq as ogptq, ref_shim
from tests import inputs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FORMATS = {"nvfp4": 16, "mxfp4": 32}


def load(name):
    d = np.load(os.path.join(GOLDEN, name))
    return {k: torch.from_numpy(d[k]) for k in d.files}


@pytest.mark.parametrize("fmt", list(FORMATS))
def test_rtn_round_trip_matches_golden(fmt):
    g = load(f"rtn_{fmt}.npz")
    w = g["weight_bf16"].view(torch.bfloat16)
    assert torch.equal(w, inputs.normal_weight(64, 512, seed=0))          # seeded input is reproducible
    y = fp4.fwht_butterfly(w, 128)
    assert torch.equal(y, g["rotated"])
    gs = fp4.nvfp4_global_scale(y.abs().max()) if fmt == "nvfp4" else None
    if fmt == "nvfp4":
        assert torch.equal(gs, g["global_scale"])
    codes, sb, s = fp4.quantize(y, fmt, gs)
    assert torch.equal(codes, g["codes"]) and torch.equal(sb, g["scale_bytes"]) and torch.equal(s, g["scales"])
    dq = fp4.dequantize(fp4.unpack_codes(codes), s, FORMATS[fmt])
    assert abs(((dq - y) ** 2).mean().item() - g["mse"].item()) <= 1e-12
    # the stored bytes decode to scale * global scale
    gsv = gs if fmt == "nvfp4" else torch.tensor([3.0])
    assert torch.allclose(fp4.decode_scale_bytes(sb, fmt), s * gsv, rtol=1e-6)


@pytest.mark.parametrize("fmt", list(FORMATS))
def test_edge_rows_match_golden(fmt):
    g = load(f"edge_{fmt}.npz")
    x = g["x"]
    assert torch.equal(x, inputs.edge_case_rows(128))
    codes, sb, s = fp4.quantize(x, fmt, torch.tensor([3.0]) if fmt == "nvfp4" else None)
    assert torch.equal(codes, g["codes"]) and torch.equal(s, g["scales"])
    keep = ~g["scale_underflow"]
    assert torch.equal(sb[keep], g["scale_bytes"][keep])


def test_log2_probes_match_golden():
    g = load("log2_probes.npz")
    assert torch.equal(fp4.mx_exponent(g["m"].clamp(min=2.0 ** -126)), g["exponent"])


@pytest.mark.parametrize("fmt", list(FORMATS))
def test_gptq_matches_golden(fmt):
    g = load(f"gptq_{fmt}.npz")
    Hd = ogptq.prepare_hessian(g["hessian"], g["weight"], 0.01)
    assert torch.allclose(Hd, g["damped_hessian"])
    U, ok = ogptq.cholesky_inverse_upper(Hd)
    assert ok and torch.allclose(U, g["u"], rtol=1e-4, atol=1e-6)
    wq, codes = ogptq.gptq_column_loop(g["weight"], g["scales"], g["u"], FORMATS[fmt], 128)
    assert torch.equal(fp4.pack_codes(codes), g["codes"]) and torch.equal(wq, g["dequantized"])
    assert abs(ogptq.relative_mse(wq, g["weight"], g["damped_hessian"]) - g["relative_mse"].item()) < 1e-6
    # GPTQ must beat round-to-nearest on this correlated Hessian
    rtn = fp4.dequantize(fp4.e2m1_codes(g["weight"], g["scales"], FORMATS[fmt]), g["scales"], FORMATS[fmt])
    assert g["relative_mse"].item() < 0.5 * ogptq.relative_mse(rtn, g["weight"], g["damped_hessian"])


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_gptq_activation_order_matches_golden(fmt):
    """quantization_order="activation" (gptq.py:146-155, 170-171, 190-193): permute by falling diag(H),
    keep every column's static scale group, quantise, undo the permutation."""
    g = load(f"gptq_actorder_{fmt}.npz")
    group = FORMATS[fmt]
    perm, perm_inv, gidx = ogptq.activation_order(g["hessian"], group)
    assert torch.equal(perm, g["perm"].long())
    Hd = ogptq.prepare_hessian(g["hessian"][perm][:, perm], g["weight"], 0.01)
    U, ok = ogptq.cholesky_inverse_upper(Hd)
    assert ok and torch.allclose(U, g["u_permuted"], rtol=1e-4, atol=1e-6)
    wq, codes = ogptq.gptq_column_loop(g["weight"][:, perm], g["scales"], g["u_permuted"], group, 128, group_index=gidx)
    assert torch.equal(fp4.pack_codes(codes[:, perm_inv].contiguous()), g["codes"])
    assert torch.equal(wq[:, perm_inv], g["dequantized"].float())
    plain = load(f"gptq_{fmt}.npz")
    assert not torch.equal(g["codes"], plain["codes"])          # the order changes the result


def test_rotation_properties():
    x = inputs.normal_weight(16, 256, seed=9, std=1.0, dtype=torch.float32)
    for g in (16, 32, 64, 128):
        y = fp4.fwht_butterfly(x, g)
        ref = (x.double().view(-1, g) @ fp4.hadamard_matrix(g).double()).view(x.shape)
        assert (y.double() - ref).abs().max() < 1e-5
        assert torch.allclose(fp4.fwht_butterfly(y, g), x, atol=1e-5)      # self-inverse
        m = fp4.hadamard_matrix(g).bfloat16()
        assert torch.allclose(fp4.rotate_dense(x.bfloat16(), m), y, atol=0.05)


def test_swizzle_layout_formula():
    """Byte (r, c) lands at tile (r // 128, c // 4), offset (r % 32) * 16 + ((r // 32) % 4) * 4 + c % 4;
    checked element by element, and against torch's own `to_blocked` helper where it imports."""
    try:
        from torch.testing._internal.common_quantized import to_blocked
    except Exception:
        to_blocked = None
    for rows, cols in ((128, 4), (256, 8), (130, 6), (1, 128)):
        sb = torch.arange(rows * cols, dtype=torch.int64).remainder(251).to(torch.uint8).view(rows, cols)
        mine = fp4.swizzle_scales(sb).flatten()
        tiles_k = (cols + 3) // 4
        for r in range(0, rows, 7):
            for c in range(cols):
                off = ((r // 128) * tiles_k + c // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + c % 4
                assert mine[off] == sb[r, c]
        assert int((mine != 0).sum()) == int((sb != 0).sum())          # padding is zero
        assert torch.equal(fp4.unswizzle_scales(mine, rows, cols), sb)
        if to_blocked is not None:
            assert torch.equal(mine, to_blocked(sb.to(torch.float32)).to(torch.uint8).flatten())


def test_pack_unpack_and_code_values():
    codes = torch.arange(16, dtype=torch.uint8).repeat(4).view(2, 32)
    assert torch.equal(fp4.unpack_codes(fp4.pack_codes(codes)), codes)
    vals = fp4.code_values(torch.arange(16, dtype=torch.uint8))
    assert vals.tolist() == [0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6]
    ties = torch.tensor([[0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, 0.0, -0.0, 7.0, -7.0, 0.26, 0.74, 5.01, -5.0]])
    c = fp4.e2m1_codes(ties, torch.ones(1, 1), 16)
    assert c.tolist() == [[8, 2, 2, 4, 4, 6, 6, 8, 8, 8, 7, 15, 1, 1, 7, 14]]


def test_matmul_oracle_against_dequantised_product():
    gen = torch.Generator().manual_seed(0)
    a = torch.randint(0, 256, (8, 64), generator=gen, dtype=torch.uint8)
    b = torch.randint(0, 256, (12, 64), generator=gen, dtype=torch.uint8)
    for fmt, g, lo, hi in (("mxfp4", 32, 120, 130), ("nvfp4", 16, 0x30, 0x40)):
        sa = torch.randint(lo, hi, (8, 128 // g), generator=gen, dtype=torch.uint8)
        sb = torch.randint(lo, hi, (12, 128 // g), generator=gen, dtype=torch.uint8)
        y = fp4.fp4_matmul(a, b, sa, sb, 0.5, fmt).float()
        ad = fp4.dequantize(fp4.unpack_codes(a), fp4.decode_scale_bytes(sa, fmt), g)
        bd = fp4.dequantize(fp4.unpack_codes(b), fp4.decode_scale_bytes(sb, fmt), g)
        assert torch.allclose(y, 0.5 * ad @ bd.t(), rtol=2 ** -7)


def test_hessian_running_mean_equals_scaled_sum():
    xs = [inputs.correlated_activations(64, 128, seed=20 + i).view(1, 64, 128) for i in range(5)]
    H, n = None, 0
    for x in xs:
        H, n = ogptq.hessian_update(H, n, x)
    exact = ogptq.hessian_exact(xs, 5)
    assert n == 5 and ((H.double() - exact).norm() / exact.norm()).item() < 1e-6


@pytest.mark.skipif(not ref_shim.available(), reason="reference tree not present")
@pytest.mark.parametrize("fmt,name,prec", [("nvfp4", "nvfp", "e4m3"), ("mxfp4", "mxfp", "e8m0")])
def test_oracle_equals_live_reference(fmt, name, prec):
    ref_shim.load()
    from src.quantization.quant_ops import cast_scales_to_eXmY, pack_fp4_to_uint8
    from src.quantization.quantizer import Quantizer

    y = fp4.fwht_butterfly(inputs.outlier_activations(96, 1024, seed=11), 64)
    q = Quantizer(bits=4, format=name, granularity="group", group_size=FORMATS[fmt], scale_precision=prec)
    s, z = q.get_quantization_params(y)
    codes = pack_fp4_to_uint8(q.quantize(y, s, z))
    sb = cast_scales_to_eXmY(s * q.global_scale, prec)
    o_codes, o_sb, o_s = fp4.quantize(y, fmt, q.global_scale if fmt == "nvfp4" else None)
    assert torch.equal(codes, o_codes) and torch.equal(s, o_s)
    keep = o_sb != 0 if fmt == "nvfp4" else torch.ones_like(o_sb, dtype=torch.bool)
    assert torch.equal(sb[keep], o_sb[keep])


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_mse_observer_matches_golden(fmt):
    """Quantizer(observer="mse") of the reference (quantizer.py:117-134): the restated search picks the same
    scale for every group, the all-zero group included; and it differs from the min-max scales."""
    g = load(f"mse_{fmt}.npz")
    y, group = g["rotated"], FORMATS[fmt]
    raw = fp4.mse_observer_raw_scales(y, group)
    if fmt == "nvfp4":
        gs = fp4.nvfp4_global_scale(y.abs().max())
        assert torch.equal(gs, g["global_scale"])
        _, s = fp4.nvfp4_scales_from_raw(raw, gs)
        _, s_minmax = fp4.nvfp4_scales(y, gs)
    else:
        _, s = fp4.mxfp4_scales_from_raw(raw)
        _, s_minmax = fp4.mxfp4_scales(y)
    assert torch.equal(s, g["scales"])
    assert (s != s_minmax).float().mean().item() > 0.03


def test_quest_restatement_matches_the_reference_triton_kernel():
    """oracle/fp4.py::quest_quantize against the UNMODIFIED Triton kernel of the reference run by Triton's
    interpreter (tests/golden/quest_triton.npz, made by tests/golden/make_quest_golden.py): the scale rule,
    the divisor, the clip mask and the rounding must agree on every element except exact ties, which the
    Triton kernel's strict `>` thresholds send toward zero (inference_lib/src/fp_quant/module/triton/mxfp4.py:
    70-104) and this package, like the reference's Quantizer, rounds to even."""
    import numpy as np

    d = np.load(os.path.join(GOLDEN, "quest_triton.npz"))
    x = torch.from_numpy(d["x"])
    want, want_mask = torch.from_numpy(d["quest_dequantized"]), torch.from_numpy(d["quest_mask"])
    codes, sb, s, mask = fp4.quest_quantize(x)
    got = fp4.dequantize(fp4.unpack_codes(codes), s, 32)
    assert torch.equal(mask, want_mask)
    assert torch.equal(sb.to(torch.float32) - 127, torch.log2(s))                  # stored byte = exponent + 127
    v = (x.reshape(64, -1, 32) / s.unsqueeze(-1)).reshape(x.shape)
    tie = torch.zeros_like(v, dtype=torch.bool)
    for t in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        tie |= v.abs() == t
    differ = got != want
    assert int(tie.sum()) > 100 and not bool((differ & ~tie).any())
    assert bool((got[differ].abs() > want[differ].abs()).all())                    # on ties the kernel goes down, we go to even
    # the all-zero group and the constant group (zero variance: divisor 2^floor(log2(1e-8)) = 2^-27)
    assert float(s[3, 1]) == 2.0 ** -27 and float(s[5, 0]) == 2.0 ** -27
    assert torch.equal(got[5, :32], torch.full((32,), 6 * 2.0 ** -27))
    # packed mask layout
    packed = fp4.pack_clip_mask(mask)
    for i in range(8):
        assert torch.equal(((packed >> i) & 1).bool(), mask[:, i::8])


def test_abs_max_triton_kernel_agrees_with_the_quantizer_rule_off_ties():
    """The same golden file holds the Triton kernel's abs_max branch: away from exact ties and all-zero groups
    (where it divides by zero) it must give what the Quantizer chain gives -- the basis for comparing the
    pseudo-quantised forward against the Quantizer rather than bit for bit against Triton."""
    import numpy as np

    d = np.load(os.path.join(GOLDEN, "quest_triton.npz"))
    x = torch.from_numpy(d["x"])
    want = torch.from_numpy(d["absmax_dequantized"])
    codes, _, s = fp4.quantize(x, "mxfp4")
    got = fp4.dequantize(fp4.unpack_codes(codes), s, 32)
    v = (x.reshape(64, -1, 32) / s.unsqueeze(-1)).reshape(x.shape)
    tie = torch.zeros_like(v, dtype=torch.bool)
    for t in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        tie |= v.abs() == t
    ok = (got == want) | tie | want.isnan()
    assert bool(ok.all()), int((~ok).sum())


def test_mxfp8_matmul_known_answer():
    """E4M3 1.0 everywhere, scales (2^0, 2^1) x (2^-1, 2^0) per 32-element group: 32*1*0.5 + 32*2*1 = 80."""
    a = torch.full((1, 64), 0x38, dtype=torch.uint8)
    y = fp4.mxfp8_matmul(a, a, torch.tensor([[127, 128]], dtype=torch.uint8), torch.tensor([[126, 127]], dtype=torch.uint8), 1.0)
    assert y.dtype == torch.bfloat16 and float(y) == 80.0
    b = torch.tensor([[0x40] * 32 + [0xC4] * 32], dtype=torch.uint8)      # 2.0 and -3.0
    y = fp4.mxfp8_matmul(a, b, torch.full((1, 2), 127, dtype=torch.uint8), torch.full((1, 2), 127, dtype=torch.uint8), 0.5)
    assert float(y) == 0.5 * (32 * 2.0 - 32 * 3.0)


def test_mxfp8_square_quantize_known_answers():
    """One E8M0 byte per 32 x 32 square = floor(log2(max|x|)) - 8 + 127; elements x / 2^(byte - 127) on the E4M3
    grid; padding rows zero; the same bytes dequantise identically along rows and along columns."""
    from oracle import mxfp8

    x = torch.zeros(40, 64, dtype=torch.bfloat16)
    x[:32, :32] = 1.0                   # max 1 -> exponent -8 -> byte 119, elements 256 = 0x78
    x[0, 0] = 1.5                       # 1.5 * 256 = 384 = 0x7C
    x[:32, 32:] = 0.0                   # all-zero square: byte 0
    x[32:, :32] = -448.0                # rows 32..39 of the second band: 448 = 1.75 * 2^8 -> exponent 0 -> byte 127
    out, rs, cs = mxfp8.square_quantize(x)
    assert out.shape == (128, 64) and rs.shape == (128, 2) and cs.shape == (64, 4)
    assert int(rs[0, 0]) == 119 and int(rs[0, 1]) == 0 and int(rs[32, 0]) == 127 and int(rs[64, 0]) == 0
    assert int(out[1, 1]) == 0x78 and int(out[0, 0]) == 0x7C and int(out[33, 5]) == 0xFE and int(out[50, 5]) == 0
    assert torch.equal(cs[:32, 0], rs[0, 0].expand(32)) and torch.equal(cs[:32, 1], rs[32, 0].expand(32))
    a = mxfp8.dequantize_mxfp8(out, rs)
    b = mxfp8.dequantize_mxfp8(out.t().contiguous(), cs).t()
    assert torch.equal(a, b) and torch.equal(a[:40], x.double())
    # a value just below a power of two saturates instead of overflowing: 511 / 2 = 255.5 -> scaled past 448
    y = torch.full((32, 32), 0.001, dtype=torch.bfloat16)
    y[3, 3] = 510.0
    out, rs, _ = mxfp8.square_quantize(y)
    assert int(rs[0, 0]) == 127 and int(out[3, 3]) == 0x7E


def test_mxfp4_transposes_are_exact_on_real_operands():
    """MXFP4 -> transposed MXFP8 keeps every value exactly while the exponents of a 32-row band lie within 2^14,
    and the transposing dequantiser returns fp4 * 2^e / alpha rounded once to bf16."""
    from oracle import mxfp8

    y = fp4.fwht_butterfly(torch.randn(70, 128, generator=torch.Generator().manual_seed(4)), 32)
    q, sb, _ = fp4.quantize(y, "mxfp4")
    want = fp4.dequantize(fp4.unpack_codes(q), fp4.decode_scale_bytes(sb, "mxfp4"), 32).double()
    out, os_ = mxfp8.fp4_transpose_fp8(q, sb)
    assert out.shape == (128, 128) and os_.shape == (128, 4)
    got = mxfp8.dequantize_mxfp8(out, os_)
    assert torch.equal(got[:, :70], want.t()) and float(got[:, 70:].abs().max()) == 0.0
    assert int(os_[0, 3]) == 0                                   # a square without source rows
    t = mxfp8.fp4_transpose_dequant(q, sb, 3.0)
    assert t.shape == (128, 70) and t.dtype == torch.bfloat16
    ref = (want.float() / torch.tensor(3.0)).t().to(torch.bfloat16)
    assert torch.equal(t.view(torch.int16), (ref + 0.0).view(torch.int16))
