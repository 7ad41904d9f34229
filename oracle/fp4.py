"""Oracle: rotation, micro-scaled FP4 quantisation, packing, layouts, matmul.

TEST INFRASTRUCTURE ONLY (see the package docstring).  All arithmetic is fp32
IEEE on CPU tensors, written so that every intermediate rounding is explicit.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

# E2M1 magnitudes indexed by the low three code bits
# (reference: src/quantization/quant_ops.py:15-16, FP4_GRID / FP4_BITPACKING_PERM).
E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
E4M3_MAX = 448.0      # quant_ops.py:9
E2M1_MAX = 6.0        # quant_ops.py:8
NVFP_GROUP = 16       # quant_ops.py:10
MXFP_GROUP = 32       # quant_ops.py:11


# --------------------------------------------------------------------------- rotation
def fwht_butterfly(x: torch.Tensor, group: int) -> torch.Tensor:
    """Block-diagonal Sylvester-Hadamard rotation of every contiguous `group`
    elements of the last dim, in fp32, natural ordering, scaled by fl32(1/sqrt(g)).

    Mathematically this is `HadamardTransform.forward`
    (src/transforms/transforms.py:81-84: `hadamard_transform(x.view(-1, g), scale=1/sqrt(g))`)
    and `x.view(-1, g) @ get_hadamard_matrix(g)` (inference_lib/src/fp_quant/module/linear.py:24-30).
    The external FWHT's summation order is not published, so the order is fixed
    here and the CUDA kernel uses the same one: stages with pair distance
    1, 2, 4, ..., g/2; in each stage the element with the distance bit clear
    becomes a+b and its partner a-b; then one fp32 multiply by fl32(1/sqrt(g)).
    Only IEEE add/sub/mul are used, so the result is bit-reproducible.
    """
    assert group >= 1 and (group & (group - 1)) == 0
    shape = x.shape
    assert shape[-1] % group == 0
    y = x.detach().to(torch.float32).reshape(-1, group).clone()
    d = 1
    while d < group:
        v = y.view(-1, group // (2 * d), 2, d)
        a = v[:, :, 0, :].clone()
        b = v[:, :, 1, :].clone()
        v[:, :, 0, :] = a + b
        v[:, :, 1, :] = a - b
        d *= 2
    c = torch.tensor(1.0 / math.sqrt(group), dtype=torch.float32)
    return (y * c).reshape(shape)


def rotate_dense(x: torch.Tensor, matrix: torch.Tensor) -> torch.Tensor:
    """`x.view(-1, g) @ matrix` for an arbitrary g x g rotation, accumulated
    sequentially over k = 0..g-1 in fp32 (acc = fl(acc + x_k * m_kj)).

    Follows the contract of `fusedQuantize*`'s second argument
    (inference_lib/src/fp_quant/module/linear_fns.py:34-48: the matrix is passed
    as bf16, so each product of a bf16 input and a bf16 entry is exact in fp32).
    """
    g = matrix.shape[0]
    assert matrix.shape == (g, g) and x.shape[-1] % g == 0
    xs = x.detach().to(torch.float32).reshape(-1, g)
    m = matrix.detach().to(torch.float32)
    acc = torch.zeros_like(xs)
    for k in range(g):
        acc = acc + xs[:, k:k + 1] * m[k:k + 1, :]
    return acc.reshape(x.shape)


def hadamard_matrix(group: int) -> torch.Tensor:
    """Sylvester-Hadamard matrix / sqrt(g) in fp64 -> fp32
    (inference_lib/src/fp_quant/module/linear.py:24-30)."""
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < group:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return (h * group ** -0.5).to(torch.float32)


def gsr_permutation(group: int) -> torch.Tensor:
    """Column order of the GSR rotation: Hadamard columns sorted by their number
    of sign changes (inference_lib/src/fp_quant/module/linear.py:37-41)."""
    h = hadamard_matrix(group)
    changes = torch.diff(h, dim=0).ne(0).sum(dim=0)
    return torch.argsort(changes)


# --------------------------------------------------------------------------- scales
def group_absmax(y: torch.Tensor, group: int) -> torch.Tensor:
    """max(-min, max) per contiguous group (src/quantization/quantizer.py:107-111)."""
    return y.reshape(*y.shape[:-1], y.shape[-1] // group, group).abs().amax(dim=-1)


def nvfp4_global_scale(tensor_absmax: torch.Tensor) -> torch.Tensor:
    """gs = fl(2688 * fl(1/absmax)), 0 when absmax == 0
    (quantizer.py:10-16 `get_reciprocal`, :146)."""
    a = tensor_absmax.to(torch.float32).reshape(1)
    r = torch.where(a == 0, torch.zeros_like(a), 1.0 / a)
    return (E4M3_MAX * E2M1_MAX) * r


def _e4m3_round(v: torch.Tensor) -> torch.Tensor:
    return v.to(torch.float8_e4m3fn)


def nvfp4_scales(y: torch.Tensor, global_scale: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-16 scales of NVFP4 (quantizer.py:111, :156-160, :168).

    Returns (stored scale bytes uint8 [..., K/16], fp32 scales used for division).
    s0 = fl(fl(2a)/12); u = e4m3_rne(clamp(fl(s0*gs), +-448)); s = fl(float(u) * fl(1/gs));
    s == 0 -> 1.  The stored byte is u (what `cast_scales_to_eXmY(s * gs)` yields,
    quant_ops.py:111-118, whenever float(u)*fl(1/gs)*gs rounds back to u); an
    all-zero group stores byte 0 (the reference would store e4m3(gs), which is not
    a usable scale; see the test-suite's note on zero groups).
    """
    a = group_absmax(y.to(torch.float32), NVFP_GROUP)
    return nvfp4_scales_from_raw((2 * a) / 12.0, global_scale)


def nvfp4_scales_from_raw(s0: torch.Tensor, global_scale: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The E4M3 chain of `nvfp4_scales` applied to given unrounded scales (min-max: fl(fl(2a)/12); MSE
    observer: the best shrunk candidate)."""
    gs = global_scale.to(torch.float32).reshape(())
    u = _e4m3_round((s0 * gs).clamp(-E4M3_MAX, E4M3_MAX))
    rgs = torch.where(gs == 0, torch.zeros_like(gs), 1.0 / gs)
    s = u.to(torch.float32) * rgs
    s = torch.where(s == 0, torch.ones_like(s), s)
    return u.view(torch.uint8), s


def mx_exponent(m: torch.Tensor) -> torch.Tensor:
    """floor(fl32(log2(m))) clamped to [-127, 127] for m >= 2^-126
    (quant_ops.py:94: `x.clamp(min=FP32_MIN_NORMAL).log2().floor().clamp(qmin, qmax)`).

    torch's fp32 log2 rounds to the integer for inputs a few ulps below a power
    of two, which raises the exponent by one there; the restatement is
    "fp64 log2, rounded to fp32, then floor", which reproduces torch-CPU on every
    probe of `tests/golden/make_golden.py`.
    """
    l = torch.log2(m.to(torch.float64)).to(torch.float32)
    return l.floor().clamp(-127, 127)


def mxfp4_scales(y: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-32 scales of MXFP4 (quantizer.py:111, :162-165; quant_ops.py:82-94).

    m = max(fl(6*fl(fl(2a)/12)), 2^-126); e = mx_exponent(m); s = fl(2^(e-2) / 0.75).
    Stored byte = e + 127 (= e8m0(3*s), quant_ops.py:115-117 with global scale 3,
    quantizer.py:64-65).
    """
    a = group_absmax(y.to(torch.float32), MXFP_GROUP)
    return mxfp4_scales_from_raw((2 * a) / 12.0)


def mxfp4_scales_from_raw(s0: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The E8M0 chain of `mxfp4_scales` applied to given unrounded scales."""
    m = (E2M1_MAX * s0).clamp(min=2.0 ** -126)
    e = mx_exponent(m)
    s = torch.pow(torch.tensor(2.0, dtype=torch.float32), e - 2) / 0.75
    s = torch.where(s == 0, torch.ones_like(s), s)
    return (e + 127).to(torch.uint8), s


QUEST_GAUSSIAN_SCALE = 2.92247856 / 6.0      # inference_lib/src/fp_quant/module/pseudoquant_linear_fns.py:20


def quest_scales(y: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-32 scales of the "quest" forward method, the default of FPQuantConfig
    (inference_lib/src/fp_quant/utils/config.py:20).  Its only statement in the reference tree is the Triton
    pseudo-quantisation kernel (inference_lib/src/fp_quant/module/triton/mxfp4.py:51-59):
        std = sqrt(mean(x^2) - mean(x)^2); scale = c * std + 1e-8; divisor = 2^floor(log2(scale))
    with c = 2.92247856 / 6 as an fp32 constant.  Triton does not define the order of its sums; it is fixed
    here (and in the CUDA kernel) as: even and odd elements of the group accumulated separately in index
    order, then even + odd; squares are rounded products added to their accumulator (no fused multiply-add);
    a variance that rounds below zero counts as zero; floor(log2) is the exponent field (scale >= 1e-8 is a
    normal number).  Returns (stored E8M0 byte = exponent + 127, fp32 divisors)."""
    g = y.to(torch.float32).reshape(*y.shape[:-1], y.shape[-1] // MXFP_GROUP, MXFP_GROUP // 2, 2)
    acc = g[..., 0, :].clone()
    acc2 = g[..., 0, :] * g[..., 0, :]
    for j in range(1, MXFP_GROUP // 2):
        acc = acc + g[..., j, :]
        acc2 = acc2 + g[..., j, :] * g[..., j, :]
    mean = (acc[..., 0] + acc[..., 1]) * 0.03125
    mean_sq = (acc2[..., 0] + acc2[..., 1]) * 0.03125
    var = (mean_sq - mean * mean).clamp(min=0.0)
    scale = torch.tensor(QUEST_GAUSSIAN_SCALE, dtype=torch.float32) * var.sqrt() + torch.tensor(1e-8, dtype=torch.float32)
    byte = (scale.view(torch.int32) >> 23) & 0xFF
    divisor = (byte << 23).to(torch.int32).view(torch.float32)
    return byte.to(torch.uint8), divisor


def quest_quantize(y: torch.Tensor):
    """Rotated fp32 tensor -> (packed codes, E8M0 scale bytes, fp32 divisors, clip mask bool): E2M1
    round-to-nearest-even of y / divisor saturating at +-6, zeros packed as 0x8 like every code in this
    package; mask = |y / divisor| < 6 (triton/mxfp4.py:105-110)."""
    sb, s = quest_scales(y)
    codes = e2m1_codes(y, s, MXFP_GROUP)
    v = y.to(torch.float32).reshape(*y.shape[:-1], -1, MXFP_GROUP) / s.unsqueeze(-1)
    return pack_codes(codes), sb, s, (v.abs() < E2M1_MAX).reshape(y.shape)


def pack_clip_mask(mask: torch.Tensor) -> torch.Tensor:
    """bool [.., K] -> uint8 [.., K/8], bit i of byte b = element 8 b + i: the layout `_unpack_mask` reads
    (inference_lib/src/fp_quant/module/linear_fns.py:66-76)."""
    m = mask.reshape(*mask.shape[:-1], mask.shape[-1] // 8, 8).to(torch.int32)
    w = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.int32)
    return (m * w).sum(dim=-1).to(torch.uint8)


def mse_observer_raw_scales(y: torch.Tensor, group: int, iters: int = 100, max_shrink: float = 0.80,
                            norm: float = 2.4) -> torch.Tensor:
    """The MSE observer's search (quantizer.py:117-134): candidates fl(f_i * s0) with
    f_i = 1 - i * max_shrink / iters (a Python float, rounded to fp32 by the multiply), error
    sum_j |x_j - grid(fl(x_j / s)) * s| ** norm over the group, the first strictly smaller error wins.
    The candidate scales are NOT rounded to E4M3 / E8M0 during the search; the chain of the scale
    precision is applied to the winner afterwards.  Returns fp32 [..., K/group]."""
    y = y.to(torch.float32)
    g = y.reshape(*y.shape[:-1], y.shape[-1] // group, group)
    s0 = (2 * g.abs().amax(dim=-1, keepdim=True)) / 12.0
    best = s0.clone()
    best_err = torch.full(g.shape[:-1], float("inf"))
    for i in range(iters):
        s = (1 - i * max_shrink / iters) * s0
        v = g / s                                             # 0 / 0 = NaN for an all-zero group: never "better"
        q = code_values(e2m1_codes(v, torch.ones(*v.shape[:-1], 1), group))
        q = torch.where(v.isnan(), v, q)
        err = (g - q * s).abs_().pow_(norm).sum(dim=-1)
        better = err < best_err
        best_err = torch.where(better, err, best_err)
        best = torch.where(better.unsqueeze(-1), s, best)
    return best.squeeze(-1)


# --------------------------------------------------------------------------- codes
def e2m1_codes(y: torch.Tensor, scales: torch.Tensor, group: int) -> torch.Tensor:
    """4-bit codes of fl(y / s) rounded to nearest-even on the E2M1 grid
    (quant_ops.py:57-68 `cast_to_fp4`, :70-71 `quantize_fp4`) and encoded as
    `pack_fp4_to_uint8` does (quant_ops.py:31-40): magnitude index in bits 0-2,
    sign in bit 3, and every zero (either sign) as 0x8.
    """
    y = y.to(torch.float32)
    v = y.reshape(*y.shape[:-1], y.shape[-1] // group, group) / scales.to(torch.float32).unsqueeze(-1)
    v = v.reshape(y.shape)
    a = v.abs()
    idx = torch.zeros_like(a, dtype=torch.int32)
    idx = torch.where((a > 0.25) & (a < 0.75), 1, idx)
    idx = torch.where((a >= 0.75) & (a <= 1.25), 2, idx)
    idx = torch.where((a > 1.25) & (a < 1.75), 3, idx)
    idx = torch.where((a >= 1.75) & (a <= 2.5), 4, idx)
    idx = torch.where((a > 2.5) & (a < 3.5), 5, idx)
    idx = torch.where((a >= 3.5) & (a <= 5.0), 6, idx)
    idx = torch.where(a > 5.0, 7, idx)
    neg = (v < 0) | (idx == 0)
    return (idx | (neg.to(torch.int32) << 3)).to(torch.uint8)


def pack_codes(codes: torch.Tensor) -> torch.Tensor:
    """Two codes per byte, even element in the low nibble (quant_ops.py:40)."""
    return (codes[..., 1::2] << 4) | codes[..., 0::2]


def unpack_codes(packed: torch.Tensor) -> torch.Tensor:
    out = torch.empty(*packed.shape[:-1], packed.shape[-1] * 2, dtype=torch.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


def code_values(codes: torch.Tensor) -> torch.Tensor:
    """Grid value of each code as fp32 (0x8 and 0x0 are both zero)."""
    mag = torch.tensor(E2M1_MAGNITUDES, dtype=torch.float32)[(codes & 7).long()]
    return torch.where((codes & 8) != 0, -mag, mag)


def dequantize(codes: torch.Tensor, scales: torch.Tensor, group: int) -> torch.Tensor:
    """grid(code) * s in fp32 (quant_ops.py:73-74 `dequantize_fp4`)."""
    v = code_values(codes)
    v = v.reshape(*v.shape[:-1], v.shape[-1] // group, group) * scales.to(torch.float32).unsqueeze(-1)
    return v.reshape(codes.shape)


def decode_scale_bytes(b: torch.Tensor, fmt: str) -> torch.Tensor:
    """Stored scale byte -> fp32 value: E4M3 (nvfp4) or 2^(b-127) (mxfp4)."""
    if fmt == "nvfp4":
        return b.contiguous().view(torch.float8_e4m3fn).to(torch.float32)
    return torch.pow(torch.tensor(2.0, dtype=torch.float64), b.to(torch.float64) - 127).to(torch.float32)


def quantize(y: torch.Tensor, fmt: str, global_scale: Optional[torch.Tensor] = None):
    """Rotated fp32 tensor -> (packed codes, scale bytes row-major, fp32 scales)."""
    if fmt == "nvfp4":
        sb, s = nvfp4_scales(y, global_scale)
        g = NVFP_GROUP
    elif fmt == "mxfp4":
        sb, s = mxfp4_scales(y)
        g = MXFP_GROUP
    else:
        raise ValueError(fmt)
    codes = e2m1_codes(y, s, g)
    return pack_codes(codes), sb, s


# --------------------------------------------------------------------------- layouts
def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def swizzle_scales(sb: torch.Tensor) -> torch.Tensor:
    """Row-major scale bytes [R, C] -> the 128x4-tile layout the block-scaled
    tensor-core matmul reads, padded with zeros to [ceil(R/128)*128, ceil(C/4)*4]
    (shape contract: inference_lib/src/fp_quant/module/qutlass_ops.py:54-71, :87-105;
    the call it replaces: `to_blocked`, qutlass_ops.py:122-123, :334-335).

    Byte (r, c) goes to tile (r // 128, c // 4) -- tiles ordered row-block-major,
    then K-block -- at offset (r % 32) * 16 + ((r // 32) % 4) * 4 + (c % 4) inside
    the 512-byte tile.
    """
    R, C = sb.shape
    Rp, Cp = ceil_div(R, 128) * 128, ceil_div(C, 4) * 4
    p = torch.zeros(Rp, Cp, dtype=torch.uint8)
    p[:R, :C] = sb
    t = p.view(Rp // 128, 4, 32, Cp // 4, 4).permute(0, 3, 2, 1, 4)
    return t.reshape(Rp, Cp).contiguous()


def unswizzle_scales(blocked: torch.Tensor, R: int, C: int) -> torch.Tensor:
    Rp, Cp = ceil_div(R, 128) * 128, ceil_div(C, 4) * 4
    t = blocked.reshape(Rp // 128, Cp // 4, 32, 4, 4).permute(0, 3, 2, 1, 4)
    return t.reshape(Rp, Cp)[:R, :C].contiguous()


# --------------------------------------------------------------------------- matmul
def fp4_matmul(aq, bq, sa, sb, alpha, fmt: str) -> torch.Tensor:
    """Y = alpha * dequant(A) @ dequant(B)^T rounded to bf16; A [M, K/2], B [N, K/2]
    packed codes, sa/sb row-major scale bytes [rows, K/g]
    (contract of `matmul_{mxf4,nvf4}_bf16_tn_op`, qutlass_ops.py:111-168;
    alpha = 1/(weight_global_scale * act_global_scale), linear_fns.py:503-510).
    Computed in fp64, so it is the exact value up to the final rounding.
    """
    g = NVFP_GROUP if fmt == "nvfp4" else MXFP_GROUP
    a = dequantize(unpack_codes(aq), decode_scale_bytes(sa, fmt), g).to(torch.float64)
    b = dequantize(unpack_codes(bq), decode_scale_bytes(sb, fmt), g).to(torch.float64)
    y = (a @ b.t()) * float(alpha)
    return y.to(torch.float32).to(torch.bfloat16)


def mxfp8_matmul(a8, b8, sa, sb, alpha) -> torch.Tensor:
    """Y = alpha * dequant(A) @ dequant(B)^T rounded to bf16 for MXFP8 operands: A [M, K], B [N, K] as E4M3
    bytes (uint8 or float8_e4m3fn, no NaN patterns), sa / sb row-major E8M0 bytes [rows, K/32], element value
    = e4m3 * 2^(byte - 127) (contract of `matmul_mxf8_bf16_tn_op`, qutlass_ops.py:171-189).  fp64 throughout.
    """
    def dq(x, s):
        v = x.view(torch.float8_e4m3fn).to(torch.float64)
        e = torch.pow(torch.tensor(2.0, dtype=torch.float64), s.view(torch.uint8).to(torch.float64) - 127.0)
        return (v.view(v.shape[0], -1, 32) * e.unsqueeze(-1)).view(v.shape)

    y = (dq(a8, sa) @ dq(b8, sb).t()) * float(alpha)
    return y.to(torch.float32).to(torch.bfloat16)
