"""CPU restatement (test infrastructure only) of the two MXFP8 re-quantisation steps of the quantised backward
pass, `backward_bf16_square_double_mxfp8` and `mxfp4_transpose_mxfp8`
(inference_lib/src/fp_quant/module/qutlass_ops.py:277-330 of IST-DASLab/FP-Quant bind them from QuTLASS).

PARITY UNPINNED: QuTLASS is an external, un-vendored package; the reference holds neither its source nor a
test or golden vector for these two ops.  What the reference fixes is their interface (shapes, dtypes, the
padding of the row count to 128: the fake implementations at qutlass_ops.py:285-304 and :315-330) and their
use (linear_fns.py:293-332): one E4M3 tensor that is read with scales along its rows by one GEMM and with
scales along its columns by the other, hence one scale per 32 x 32 square.  The arithmetic inside a square
is defined by this repository (OCP-MX style: power-of-two scale from the largest magnitude, round to nearest
even, saturate) and the CUDA kernels are compared with this file bit for bit.
"""
import torch

from . import fp4

E4M3_MAX = 448.0


def _pad_rows(rows: int) -> int:
    return (rows + 127) // 128 * 128


def _to_e4m3_bytes(v: torch.Tensor) -> torch.Tensor:
    """fp32/fp64 values -> E4M3 bytes, round to nearest even, clamped to +-448 first."""
    return v.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float32).to(torch.float8_e4m3fn).view(torch.uint8)


def square_quantize(x_bf16: torch.Tensor):
    """bf16 [rows, cols] -> (E4M3 bytes [rows_pad, cols], row_scales [rows_pad, cols/32], col_scales
    [cols, rows_pad/32]); one E8M0 byte per 32 x 32 square: floor(log2(max|x|)) - 8 + 127 clamped to
    [0, 254], 0 for an all-zero square; elements are x * 2^-(byte - 127)."""
    rows, cols = x_bf16.shape
    rp = _pad_rows(rows)
    x = torch.zeros(rp, cols, dtype=torch.float64)
    x[:rows] = x_bf16.to(torch.float64)
    sq = x.view(rp // 32, 32, cols // 32, 32)
    amax = sq.abs().amax(dim=(1, 3))                               # [rp/32, cols/32]
    _, ex = torch.frexp(amax)                                      # amax = m * 2^ex, m in [0.5, 1)
    e = (ex - 1 - 8).clamp(-127, 127)
    byte = torch.where(amax > 0, e + 127, torch.zeros_like(e)).to(torch.uint8)
    e_used = byte.to(torch.float64) - 127.0
    scaled = sq * torch.pow(torch.tensor(2.0, dtype=torch.float64), -e_used)[:, None, :, None]
    out = _to_e4m3_bytes(scaled.reshape(rp, cols))
    row_scales = byte.repeat_interleave(32, dim=0)                 # [rp, cols/32]
    col_scales = byte.t().repeat_interleave(32, dim=0).contiguous()   # [cols, rp/32]
    return out, row_scales, col_scales


def fp4_transpose_fp8(codes: torch.Tensor, scale_bytes: torch.Tensor):
    """MXFP4 (packed codes [rows, cols/2], E8M0 bytes [rows, cols/32]) -> (E4M3 bytes [cols, rows_pad],
    E8M0 bytes [cols, rows_pad/32]) of the transpose.  Per 32 x 32 square: byte = max(0, emax - 6 + 127) with
    emax the largest source exponent of its (real) rows, 0 for a square without rows; element =
    fp4 * 2^(e_row - (byte - 127)), zeros of either sign as +0."""
    rows, cols = codes.shape[0], codes.shape[1] * 2
    rp = _pad_rows(rows)
    v = fp4.code_values(fp4.unpack_codes(codes)).to(torch.float64)
    e = scale_bytes.view(torch.uint8).to(torch.int64) - 127        # [rows, cols/32]
    e_pad = torch.full((rp, cols // 32), -1000, dtype=torch.int64)
    e_pad[:rows] = e
    emax = e_pad.view(rp // 32, 32, cols // 32).amax(dim=1)         # [rp/32, cols/32]
    e_sq = (emax - 6).clamp(min=-127)
    byte = torch.where(emax > -1000, e_sq + 127, torch.zeros_like(e_sq)).to(torch.uint8)
    vals = torch.zeros(rp, cols, dtype=torch.float64)
    shift = (e - e_sq.repeat_interleave(32, dim=0)[:rows]).to(torch.float64)          # [rows, cols/32]
    vals[:rows] = (v.view(rows, cols // 32, 32) * torch.pow(torch.tensor(2.0, dtype=torch.float64), shift)[:, :, None]).view(rows, cols)
    vals = vals + 0.0                                              # -0 -> +0
    out = _to_e4m3_bytes(vals.t().contiguous())                    # [cols, rp]
    out_scales = byte.t().repeat_interleave(32, dim=0).contiguous()    # [cols, rp/32]
    return out, out_scales


def dequantize_mxfp8(bytes_e4m3: torch.Tensor, scale_bytes: torch.Tensor) -> torch.Tensor:
    """E4M3 bytes [rows, K] with E8M0 bytes [rows, K/32] along K -> fp64 values."""
    v = bytes_e4m3.view(torch.float8_e4m3fn).to(torch.float64)
    s = torch.pow(torch.tensor(2.0, dtype=torch.float64), scale_bytes.view(torch.uint8).to(torch.float64) - 127.0)
    return (v.view(v.shape[0], -1, 32) * s[:, :, None]).view(v.shape)


def fp4_transpose_dequant(codes: torch.Tensor, scale_bytes: torch.Tensor, alpha: float) -> torch.Tensor:
    """MXFP4 (packed codes [rows, cols/2], E8M0 bytes [rows, cols/32]) -> bf16 [cols, rows]: fp32 value
    fp4 * 2^(byte - 127), divided by fl32(alpha) (IEEE fp32 division), rounded once to bf16; zeros of either
    sign come out as +0.  First half of `backward_qt_bf16` (qutlass_ops.py:248-274)."""
    v = fp4.code_values(fp4.unpack_codes(codes))
    s = fp4.decode_scale_bytes(scale_bytes.view(torch.uint8), "mxfp4")
    x = (v.view(v.shape[0], -1, 32) * s.unsqueeze(-1)).view(v.shape)            # exact in fp32
    x = x / torch.tensor(alpha, dtype=torch.float32) + 0.0
    return x.t().contiguous().to(torch.bfloat16)
