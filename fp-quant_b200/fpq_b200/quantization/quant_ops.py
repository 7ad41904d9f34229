"""Constants and packing helpers of the quantisation API
(src/quantization/quant_ops.py of IST-DASLab/FP-Quant), backed by the CUDA library."""
from __future__ import annotations

import torch

from .. import ops
from .quant_args import ScalePrecision

FP4_E2M1_MAX = 6
FP8_E4M3_MAX = 448
NVFP_GROUPSIZE = 16
MXFP_GROUPSIZE = 32
FP4_SCALE = 3 / 4
# grid value of each 4-bit code (code = index); 0x0 and 0x8 are both zero, packing emits 0x8
FP4_CODE_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def pack_fp4_to_uint8(x: torch.Tensor) -> torch.Tensor:
    """Tensor of E2M1 grid values [rows, cols] -> uint8 [rows, cols/2], even element in the low
    nibble, zeros encoded as 0x8 (quant_ops.py:31-40)."""
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    return ops.pack_grid(x)


def cast_scales_to_eXmY(scales: torch.Tensor, scale_precision: str) -> torch.Tensor:
    """Scale values -> stored bytes (quant_ops.py:111-118): E4M3 bit pattern, or the E8M0
    biased exponent.  A dtype cast of an already exact value; the fused quantise kernel writes
    the same bytes directly."""
    precision = ScalePrecision(scale_precision)
    if precision == ScalePrecision.E4M3:
        return scales.to(torch.float8_e4m3fn).view(torch.uint8)
    if precision == ScalePrecision.E8M0:
        return scales.to(torch.float8_e8m0fnu).view(torch.uint8)
    return scales


def get_quantization_range(format, bits: int, symmetric: bool):
    if str(format) in ("fp", "nvfp", "mxfp"):
        assert bits == 4, "only 4-bit floating-point formats are supported"
        return -FP4_E2M1_MAX, FP4_E2M1_MAX
    raise NotImplementedError("integer formats are outside the B200 hot path")
