"""Tensor-level wrappers over the C ABI: allocate outputs with torch, pass raw
pointers and the current CUDA stream, never synchronise."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _cabi as C
from ._cabi import call as _cabi_call

FORMATS = {"mxfp4": C.FMT_MXFP4, "nvfp4": C.FMT_NVFP4}
GROUP_OF = {"mxfp4": 32, "nvfp4": 16}


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return C.DT_BF16
    if t.dtype == torch.float32:
        return C.DT_F32
    raise ValueError(f"fpq_b200 kernels take bfloat16 or float32 tensors, got {t.dtype}")


def _cuda(t: torch.Tensor, name: str = "tensor") -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: fpq_b200 has no CPU path")
    return t


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def _guard(device: torch.device):
    """Make `device` current for the launch; free when it already is (the common case)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _2d(x: torch.Tensor) -> Tuple[torch.Tensor, int, int]:
    x = _cuda(x, "x").contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    return x, rows, cols


def padded_scale_shape(rows: int, sf_cols: int) -> Tuple[int, int]:
    return ((rows + 127) // 128) * 128, ((sf_cols + 3) // 4) * 4


def rotate_hadamard(x: torch.Tensor, group: int, out_dtype: Optional[torch.dtype] = None,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    x, rows, cols = _2d(x)
    if cols % group != 0:
        raise ValueError(f"last dim ({cols}) must be a multiple of the hadamard group ({group})")
    if cols % 32 != 0 and x.numel() % 32 == 0:
        # groups are contiguous in memory, so any row length that keeps them whole is equivalent
        rows, cols = x.numel() // max(32, group), max(32, group)
    if out is None:
        out = torch.empty_like(x, dtype=out_dtype or x.dtype)
    with _guard(x.device):
        C.call("fpq_rotate_hadamard", x.data_ptr(), _dt(x), out.data_ptr(), _dt(out), rows, cols, group, _stream(x))
    return out


def rotate_dense(x: torch.Tensor, matrix: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    x, rows, cols = _2d(x)
    m = _cuda(matrix, "matrix").to(torch.float32).contiguous()
    out = torch.empty_like(x, dtype=out_dtype or x.dtype)
    with _guard(x.device):
        C.call("fpq_rotate_dense", x.data_ptr(), _dt(x), out.data_ptr(), _dt(out), rows, cols, m.shape[0],
               m.data_ptr(), _stream(x))
    return out


def absmax_bits(x: torch.Tensor, hadamard_group: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """uint32 bit pattern (held in an int32 tensor) of max |rotate(x)|."""
    x, rows, cols = _2d(x)
    if out is None:
        out = torch.zeros(1, dtype=torch.int32, device=x.device)
    with _guard(x.device):
        C.call("fpq_absmax", x.data_ptr(), _dt(x), rows, cols, hadamard_group, out.data_ptr(), _stream(x))
    return out


def global_scale_update(bits: torch.Tensor, global_scale: torch.Tensor,
                        status: Optional[torch.Tensor] = None) -> torch.Tensor:
    assert global_scale.dtype == torch.float32 and global_scale.is_cuda
    with _guard(bits.device):
        C.call("fpq_global_scale_update", bits.data_ptr(), global_scale.data_ptr(), _ptr(status), _stream(bits))
    return global_scale


def quantize(x: torch.Tensor, fmt: str, hadamard_group: int = 0, global_scale: Optional[torch.Tensor] = None,
             codes: bool = True, scale_bytes: bool = True, swizzled: bool = False, scales_f32: bool = False):
    """Returns (codes u8 [rows, cols/2] | None, scale bytes | None, fp32 scales | None)."""
    x, rows, cols = _2d(x)
    g = GROUP_OF[fmt]
    sf_cols = cols // g
    dev = x.device
    q = torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev) if codes else None
    sb = None
    if scale_bytes:
        if swizzled:
            pr, pc = padded_scale_shape(rows, sf_cols)
            alloc = torch.zeros if pc != sf_cols else torch.empty       # pad rows are zeroed by the kernel
            sb = alloc(pr, pc, dtype=torch.uint8, device=dev)
        else:
            sb = torch.empty(rows, sf_cols, dtype=torch.uint8, device=dev)
    sf = torch.empty(rows, sf_cols, dtype=torch.float32, device=dev) if scales_f32 else None
    if fmt == "nvfp4":
        if global_scale is None:
            raise ValueError("nvfp4 needs a global_scale tensor")
        global_scale = _cuda(global_scale, "global_scale").to(torch.float32)
    with _guard(dev):
        C.call("fpq_quantize", x.data_ptr(), _dt(x), rows, cols, hadamard_group, FORMATS[fmt],
               _ptr(global_scale) if fmt == "nvfp4" else None, _ptr(q), _ptr(sb),
               C.SCALES_SWIZZLED if swizzled else C.SCALES_ROWMAJOR, _ptr(sf), _stream(x))
    return q, sb, sf


def quantize_silu_mul(gate: torch.Tensor, up: torch.Tensor, fmt: str, hadamard_group: int = 0,
                      global_scale: Optional[torch.Tensor] = None, swizzled: bool = True):
    """quantize(silu(gate) * up) in one pass: (codes u8 [rows, cols/2], scale bytes).  gate, up: bf16 [.., cols]."""
    gate, rows, cols = _2d(gate)
    up = _cuda(up, "up").contiguous()
    if gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16 or up.numel() != gate.numel():
        raise ValueError("gate and up must be bfloat16 tensors of the same shape")
    sf_cols = cols // GROUP_OF[fmt]
    dev = gate.device
    q = torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev)
    if swizzled:
        pr, pc = padded_scale_shape(rows, sf_cols)
        sb = (torch.zeros if pc != sf_cols else torch.empty)(pr, pc, dtype=torch.uint8, device=dev)
    else:
        sb = torch.empty(rows, sf_cols, dtype=torch.uint8, device=dev)
    if fmt == "nvfp4":
        if global_scale is None:
            raise ValueError("nvfp4 needs a global_scale tensor")
        global_scale = _cuda(global_scale, "global_scale").to(torch.float32)
    with _guard(dev):
        C.call("fpq_quantize_silu_mul", gate.data_ptr(), up.data_ptr(), rows, cols, hadamard_group, FORMATS[fmt],
               _ptr(global_scale) if fmt == "nvfp4" else None, q.data_ptr(), sb.data_ptr(),
               C.SCALES_SWIZZLED if swizzled else C.SCALES_ROWMAJOR, _stream(gate))
    return q, sb


def quantize_quest(x: torch.Tensor, hadamard_group: int = 0, swizzled: bool = False, return_mask: bool = False):
    """MXFP4 with the QuEST scale rule: (codes u8 [rows, cols/2], E8M0 scale bytes, clip mask u8 [rows, cols/8] | None)."""
    x, rows, cols = _2d(x)
    sf_cols = cols // 32
    dev = x.device
    q = torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev)
    if swizzled:
        pr, pc = padded_scale_shape(rows, sf_cols)
        sb = (torch.zeros if pc != sf_cols else torch.empty)(pr, pc, dtype=torch.uint8, device=dev)
    else:
        sb = torch.empty(rows, sf_cols, dtype=torch.uint8, device=dev)
    mask = torch.empty(rows, cols // 8, dtype=torch.uint8, device=dev) if return_mask else None
    with _guard(dev):
        C.call("fpq_quantize_quest", x.data_ptr(), _dt(x), rows, cols, hadamard_group, q.data_ptr(), sb.data_ptr(),
               C.SCALES_SWIZZLED if swizzled else C.SCALES_ROWMAJOR, _ptr(mask), _stream(x))
    return q, sb, mask


def fake_quantize_quest(x: torch.Tensor, hadamard_group: int = 0, return_mask: bool = True):
    """Quantise-dequantise with the QuEST scale rule: (y like x, bool clip mask like x | None)."""
    shape = x.shape
    x, rows, cols = _2d(x)
    y = torch.empty_like(x)
    mask = torch.empty(rows, cols, dtype=torch.bool, device=x.device) if return_mask else None
    with _guard(x.device):
        C.call("fpq_fake_quantize_quest", x.data_ptr(), _dt(x), rows, cols, hadamard_group, y.data_ptr(), _ptr(mask),
               _stream(x))
    return y.view(shape), (mask.view(shape) if mask is not None else None)


def mse_scales(x: torch.Tensor, fmt: str, global_scale: Optional[torch.Tensor] = None, iters: int = 100,
               max_shrink: float = 0.80, error_norm: float = 2.4) -> torch.Tensor:
    """fp32 [rows, cols/g]: the scales the MSE observer picks (quantizer.py:117-134) after the E4M3 / E8M0 chain."""
    x, rows, cols = _2d(x)
    out = torch.empty(rows, cols // GROUP_OF[fmt], dtype=torch.float32, device=x.device)
    if fmt == "nvfp4":
        if global_scale is None:
            raise ValueError("nvfp4 needs a global_scale tensor")
        global_scale = _cuda(global_scale, "global_scale").to(torch.float32)
    with _guard(x.device):
        C.call("fpq_mse_scales", x.data_ptr(), _dt(x), rows, cols, FORMATS[fmt],
               _ptr(global_scale) if fmt == "nvfp4" else None, int(iters), float(max_shrink), float(error_norm),
               out.data_ptr(), _stream(x))
    return out


def fake_quantize(x: torch.Tensor, fmt: str, hadamard_group: int = 0,
                  global_scale: Optional[torch.Tensor] = None, ste: bool = False) -> torch.Tensor:
    shape = x.shape
    x, rows, cols = _2d(x)
    y = torch.empty_like(x)
    if fmt == "nvfp4":
        if global_scale is None:
            raise ValueError("nvfp4 needs a global_scale tensor")
        global_scale = _cuda(global_scale, "global_scale").to(torch.float32)
    with _guard(x.device):
        C.call("fpq_fake_quantize", x.data_ptr(), _dt(x), rows, cols, hadamard_group, FORMATS[fmt],
               _ptr(global_scale) if fmt == "nvfp4" else None, y.data_ptr(), int(ste), _stream(x))
    return y.view(shape)


def apply_scales(x: torch.Tensor, scales: torch.Tensor, group: int, out_kind: int) -> torch.Tensor:
    x, rows, cols = _2d(x)
    s = _cuda(scales, "scales").to(torch.float32).contiguous()
    assert s.numel() == rows * (cols // group), "scales must be [rows, cols/group]"
    if out_kind == C.OUT_CODES:
        out = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    else:
        out = torch.empty_like(x)
    with _guard(x.device):
        C.call("fpq_apply_scales", x.data_ptr(), _dt(x), rows, cols, s.data_ptr(), group, out_kind,
               out.data_ptr(), _stream(x))
    return out


def pack_grid(q: torch.Tensor) -> torch.Tensor:
    q, rows, cols = _2d(q)
    out = torch.empty(rows, cols // 2, dtype=torch.uint8, device=q.device)
    with _guard(q.device):
        C.call("fpq_pack_grid", q.data_ptr(), _dt(q), rows, cols, out.data_ptr(), _stream(q))
    return out


def swizzle_scales(sb: torch.Tensor) -> torch.Tensor:
    sb = _cuda(sb, "scales")
    if sb.dtype != torch.uint8:
        sb = sb.view(torch.uint8)
    sb = sb.contiguous()
    rows, sf_cols = sb.shape
    pr, pc = padded_scale_shape(rows, sf_cols)
    out = torch.empty(pr, pc, dtype=torch.uint8, device=sb.device)
    with _guard(sb.device):
        C.call("fpq_swizzle_scales", sb.data_ptr(), rows, sf_cols, out.data_ptr(), _stream(sb))
    return out


_error_flags = {}


def device_error_flag(device: torch.device) -> torch.Tensor:
    """int32[1] on `device` that kernels with bounded waits set when a wait ran out."""
    key = torch.device(device).index or 0
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _error_flags[key]


def check_device_errors(device: torch.device) -> None:
    """Synchronising check: raises if any kernel on `device` reported a timed-out wait."""
    flag = device_error_flag(device)
    if int(flag.item()) != 0:
        flag.zero_()
        raise C.FpqError(C.ERR_DEVICE_TIMEOUT, "a bounded in-kernel wait ran out; results are invalid")


def gemm_fp4(a_codes: torch.Tensor, b_codes: torch.Tensor, a_scales_swizzled: torch.Tensor,
             b_scales_swizzled: torch.Tensor, alpha: torch.Tensor, fmt: str,
             bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 [M, N] = alpha * dq(A) dq(B)^T (+ bias); codes [rows, K/2] uint8, scales swizzled."""
    a = _cuda(a_codes, "a_codes").contiguous()
    b = _cuda(b_codes, "b_codes").contiguous()
    M, K = a.shape[0], a.shape[1] * 2
    N = b.shape[0]
    if b.shape[1] * 2 != K:
        raise ValueError(f"K mismatch: {a.shape} vs {b.shape}")
    sa = _cuda(a_scales_swizzled, "a_scales").contiguous()
    sb = _cuda(b_scales_swizzled, "b_scales").contiguous()
    g = GROUP_OF[fmt]
    for name, s, rows in (("a_scales", sa, M), ("b_scales", sb, N)):
        pr, pc = padded_scale_shape(rows, K // g)
        if s.numel() != pr * pc:
            raise ValueError(f"{name} must hold the swizzled layout of [{pr}, {pc}] bytes, got {tuple(s.shape)}")
    alpha = _cuda(alpha, "alpha").to(torch.float32).reshape(1)
    if bias is not None:
        bias = _cuda(bias, "bias").to(torch.bfloat16).contiguous()
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    with _guard(a.device):
        C.call("fpq_gemm_fp4", a.data_ptr(), b.data_ptr(), sa.data_ptr(), sb.data_ptr(), alpha.data_ptr(),
               _ptr(bias), out.data_ptr(), M, N, K, FORMATS[fmt], device_error_flag(a.device).data_ptr(), _stream(a))
    return out


def gemm_mxf8(a_e4m3: torch.Tensor, b_e4m3: torch.Tensor, a_scales_swizzled: torch.Tensor,
              b_scales_swizzled: torch.Tensor, alpha: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 [M, N] = alpha * dq(A) dq(B)^T for MXFP8 operands: E4M3 bytes [rows, K] (float8_e4m3fn or uint8),
    one E8M0 scale per 32 elements along K, scales swizzled."""
    a = _cuda(a_e4m3, "a").contiguous()
    b = _cuda(b_e4m3, "b").contiguous()
    for name, t in (("a", a), ("b", b)):
        if t.dtype not in (torch.float8_e4m3fn, torch.uint8) or t.dim() != 2:
            raise ValueError(f"{name} must be a 2-D float8_e4m3fn (or uint8) tensor, got {t.dtype} {tuple(t.shape)}")
    M, K = a.shape
    N = b.shape[0]
    if b.shape[1] != K:
        raise ValueError(f"K mismatch: {tuple(a.shape)} vs {tuple(b.shape)}")
    sa = _cuda(a_scales_swizzled, "a_scales").contiguous()
    sb = _cuda(b_scales_swizzled, "b_scales").contiguous()
    for name, s, rows in (("a_scales", sa, M), ("b_scales", sb, N)):
        pr, pc = padded_scale_shape(rows, K // 32)
        if s.numel() != pr * pc:
            raise ValueError(f"{name} must hold the swizzled layout of [{pr}, {pc}] bytes, got {tuple(s.shape)}")
    alpha = _cuda(alpha, "alpha").to(torch.float32).reshape(1)
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    with _guard(a.device):
        C.call("fpq_gemm_mxf8", a.data_ptr(), b.data_ptr(), sa.data_ptr(), sb.data_ptr(), alpha.data_ptr(),
               out.data_ptr(), M, N, K, device_error_flag(a.device).data_ptr(), _stream(a))
    return out


def _scale_buffer(rows: int, sf_cols: int, swizzled: bool, device) -> torch.Tensor:
    """Buffer for [rows, sf_cols] scale bytes: exact when row-major, the padded tile layout (padding zeroed) when swizzled."""
    if not swizzled:
        return torch.empty(rows, sf_cols, dtype=torch.uint8, device=device)
    pr, pc = padded_scale_shape(rows, sf_cols)
    alloc = torch.empty if (pr, pc) == (rows, sf_cols) else torch.zeros
    return alloc(pr, pc, dtype=torch.uint8, device=device)


def quantize_mxfp8_square(x: torch.Tensor, swizzled: bool = False, transposed: bool = False):
    """bf16 [rows, cols] -> (E4M3 [rows_pad, cols], row scales u8 [rows_pad, cols/32], column scales u8
    [cols, rows_pad/32]); one E8M0 byte per 32 x 32 square, rows_pad = rows rounded up to 128 (zero rows).
    swizzled: both scale tensors in the layout the GEMM reads.  transposed: additionally returns the bytes as
    [cols, rows_pad] (fourth value)."""
    x = _cuda(x, "x")
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise ValueError(f"x must be a 2-D bfloat16 tensor, got {x.dtype} {tuple(x.shape)}")
    x = x.contiguous()
    rows, cols = x.shape
    rp = (rows + 127) // 128 * 128
    out = torch.empty(rp, cols, dtype=torch.float8_e4m3fn, device=x.device)
    out_t = torch.empty(cols, rp, dtype=torch.float8_e4m3fn, device=x.device) if transposed else None
    rs = _scale_buffer(rp, cols // 32, swizzled, x.device)
    cs = _scale_buffer(cols, rp // 32, swizzled, x.device)
    with _guard(x.device):
        C.call("fpq_quantize_mxfp8_square", x.data_ptr(), rows, cols, out.data_ptr(), _ptr(out_t), rs.data_ptr(), cs.data_ptr(),
               C.SCALES_SWIZZLED if swizzled else C.SCALES_ROWMAJOR, _stream(x))
    return (out, rs, cs, out_t) if transposed else (out, rs, cs)


def mxfp4_transpose_mxfp8(codes: torch.Tensor, scales_rowmajor: torch.Tensor, swizzled: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """MXFP4 (codes u8 [rows, cols/2], E8M0 bytes [rows, cols/32], row-major, unpadded) -> the transpose as
    MXFP8: (E4M3 [cols, rows_pad], scales u8 [cols, rows_pad/32], swizzled for the GEMM on request)."""
    codes = _cuda(codes, "codes").contiguous()
    sc = _cuda(scales_rowmajor, "scales")
    sc = (sc if sc.dtype == torch.uint8 else sc.view(torch.uint8)).contiguous()
    rows, cols = codes.shape[0], codes.shape[1] * 2
    if tuple(sc.shape) != (rows, cols // 32):
        raise ValueError(f"scales must be [{rows}, {cols // 32}] row-major bytes, got {tuple(sc.shape)}")
    rp = (rows + 127) // 128 * 128
    out = torch.empty(cols, rp, dtype=torch.float8_e4m3fn, device=codes.device)
    os_ = _scale_buffer(cols, rp // 32, swizzled, codes.device)
    with _guard(codes.device):
        C.call("fpq_mxfp4_transpose_mxfp8", codes.data_ptr(), sc.data_ptr(), rows, cols, out.data_ptr(), os_.data_ptr(),
               C.SCALES_SWIZZLED if swizzled else C.SCALES_ROWMAJOR, _stream(codes))
    return out, os_


def mxfp4_transpose_dequant(codes: torch.Tensor, scales_rowmajor: torch.Tensor, alpha: torch.Tensor,
                            pad_to: int = 1) -> torch.Tensor:
    """MXFP4 (codes u8 [rows, cols/2], E8M0 bytes [rows, cols/32]) -> bf16 [cols, rows_pad] = dequantised^T / alpha,
    rows_pad = rows rounded up to a multiple of `pad_to` (the padding columns are zero)."""
    codes = _cuda(codes, "codes").contiguous()
    sc = _cuda(scales_rowmajor, "scales")
    sc = (sc if sc.dtype == torch.uint8 else sc.view(torch.uint8)).contiguous()
    rows, cols = codes.shape[0], codes.shape[1] * 2
    if tuple(sc.shape) != (rows, cols // 32):
        raise ValueError(f"scales must be [{rows}, {cols // 32}] row-major bytes, got {tuple(sc.shape)}")
    alpha = _cuda(alpha, "alpha").to(torch.float32).reshape(1)
    rp = -(-rows // pad_to) * pad_to
    out = (torch.empty if rp == rows else torch.zeros)(cols, rp, dtype=torch.bfloat16, device=codes.device)
    with _guard(codes.device):
        C.call("fpq_mxfp4_transpose_dequant", codes.data_ptr(), sc.data_ptr(), rows, cols, alpha.data_ptr(), out.data_ptr(), rp,
               _stream(codes))
    return out


def quantize_transposed(x: torch.Tensor, hadamard_group: int = 0, pad_to: int = 32, swizzled: bool = False):
    """MXFP4 of x^T for a bf16 matrix x [t, n] without materialising the transpose: (codes u8 [n, t_pad/2], E8M0 scale
    bytes [n, t_pad/32] row-major or swizzled); t_pad = t rounded up to a multiple of `pad_to` (a multiple of 32),
    the padding counts as zeros.  Rotation groups 0, 16 and 32."""
    x = _cuda(x, "x")
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise ValueError(f"x must be a 2-D bfloat16 tensor, got {x.dtype} {tuple(x.shape)}")
    if pad_to % 32 != 0:
        raise ValueError("pad_to must be a multiple of 32")
    x = x.contiguous()
    t, n = x.shape
    tp = -(-t // pad_to) * pad_to
    codes = torch.empty(n, tp // 2, dtype=torch.uint8, device=x.device)
    sb = _scale_buffer(n, tp // 32, swizzled, x.device)
    with _guard(x.device):
        C.call("fpq_quantize_transposed", x.data_ptr(), t, n, tp, hadamard_group, codes.data_ptr(), sb.data_ptr(),
               C.SCALES_SWIZZLED if swizzled else C.SCALES_ROWMAJOR, _stream(x))
    return codes, sb


# --------------------------------------------------------------------------- GPTQ core
def gemm_fp4_push(a_codes: torch.Tensor, b_codes: torch.Tensor, a_scales_swizzled: torch.Tensor,
                  b_scales_swizzled: torch.Tensor, alpha: torch.Tensor, fmt: str, out: torch.Tensor, peer_ptrs,
                  col_offset: int, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Column-parallel GEMM: writes this rank's [M, n_loc] product into columns [col_offset, col_offset + n_loc)
    of `out` [M, ldc] and of the other ranks' buffers (`peer_ptrs`: their device addresses as mapped on this
    GPU), from the same epilogue.  The caller synchronises the ranks afterwards."""
    import ctypes

    _cuda(a_codes, "a_codes"), _cuda(b_codes, "b_codes"), _cuda(out, "out")
    m, k = a_codes.shape[0], a_codes.shape[1] * 2
    n = b_codes.shape[0]
    if out.dtype != torch.bfloat16 or out.dim() != 2 or out.shape[0] != m or not out.is_contiguous():
        raise ValueError("out must be a contiguous bf16 [M, ldc] tensor")
    ptrs = (ctypes.c_void_p * max(1, len(peer_ptrs)))(*[int(p) for p in peer_ptrs])
    alpha = _cuda(alpha, "alpha").to(torch.float32).reshape(1)
    if bias is not None:
        bias = _cuda(bias, "bias").to(torch.bfloat16).contiguous()
    with _guard(out.device):
        C.call("fpq_gemm_fp4_push", a_codes.data_ptr(), b_codes.data_ptr(), a_scales_swizzled.data_ptr(),
               b_scales_swizzled.data_ptr(), alpha.data_ptr(), _ptr(bias), out.data_ptr(), ptrs, len(peer_ptrs),
               out.shape[1], col_offset, m, n, k, FORMATS[fmt],
               device_error_flag(out.device).data_ptr(), _stream(out))
    return out


def _f32(t: torch.Tensor, name: str, inplace: bool = False) -> torch.Tensor:
    t = _cuda(t, name)
    if t.dtype != torch.float32:
        raise ValueError(f"{name} must be a float32 tensor")
    if not t.is_contiguous():
        if inplace:
            raise ValueError(f"{name} is modified in place and must be contiguous")
        t = t.contiguous()
    return t


def sgemm(A: torch.Tensor, B: torch.Tensor, b_transposed: bool = False, C: Optional[torch.Tensor] = None,
          alpha: float = 1.0, beta: float = 0.0) -> torch.Tensor:
    """True-fp32 matrix product C = beta*C + alpha * A @ (B^T if b_transposed else B)."""
    A, B = _f32(A, "A"), _f32(B, "B")
    M, K = A.shape
    N = B.shape[0] if b_transposed else B.shape[1]
    if C is None:
        C = torch.zeros(M, N, dtype=torch.float32, device=A.device)
        beta = 0.0
    with _guard(A.device):
        _cabi_call("fpq_sgemm", A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), int(b_transposed), C.data_ptr(),
                   C.stride(0), M, N, K, alpha, beta, _stream(A))
    return C


def hessian_prepare(H: torch.Tensor, W: torch.Tensor, rel_damp: float) -> torch.Tensor:
    """In place: dead-column fix + damping of the Hessian (GPTQ._get_hessian_inverse, first half)."""
    H, W = _f32(H, "H", inplace=True), _f32(W, "W")
    d = H.shape[0]
    ws = torch.empty(d, dtype=torch.uint8, device=H.device)
    with _guard(H.device):
        C.call("fpq_hessian_prepare", H.data_ptr(), d, W.data_ptr(), W.shape[0], float(rel_damp), ws.data_ptr(),
               _stream(H))
    return H


def cholesky_inverse_upper(H: torch.Tensor):
    """(U, status): U upper with U^T U = H^-1; status is a device int32[1], 1 if H was not positive definite."""
    H = _f32(H, "H")
    d = H.shape[0]
    U = torch.empty_like(H)
    n = int(C.lib().fpq_cholesky_workspace_floats(d))
    ws = torch.empty(n, dtype=torch.float32, device=H.device)
    status = torch.zeros(1, dtype=torch.int32, device=H.device)
    with _guard(H.device):
        C.call("fpq_cholesky_inverse_upper", H.data_ptr(), U.data_ptr(), d, ws.data_ptr(), status.data_ptr(),
               device_error_flag(H.device).data_ptr(), _stream(H))
    return U, status


# --------------------------------------------------------------------------- CUDA-graph replays of the two long launch chains
# The Cholesky-inverse chain (786 dependent launches at d = 14336) and the column loop (two launches per 128
# columns) are bound by how fast the host issues small kernels: the same binary needed 0.08 s or 0.27 s per
# two transformer blocks for the chains depending on the host it ran on.  Both are static given their shapes,
# so each shape is captured once into a CUDA graph over buffers of its own and replayed afterwards.
_graphs: dict = {}


def _capture(key, build):
    """(graph, statics) for `key`; `build()` allocates the static buffers and returns (statics, run) where run()
    issues the launches on the current stream."""
    entry = _graphs.get(key)
    if entry is None:
        statics, run = build()
        run()                                   # first run outside the capture: one-time initialisation, warm caches
        torch.cuda.current_stream().synchronize()
        graph = torch.cuda.CUDAGraph()
        # thread-local: other threads of the process (NCCL's watchdog) may call into CUDA during the capture
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            run()
        entry = _graphs[key] = (graph, statics)
    return entry


def cholesky_inverse_upper_graphed(H: torch.Tensor):
    """`cholesky_inverse_upper` replayed from a CUDA graph captured per (device, d).  Same result; costs one
    copy of H in and one of U out, and holds H, U and the workspace of every d it has seen."""
    H = _f32(H, "H")
    d = H.shape[0]

    def build():
        st = {"H": torch.empty_like(H), "U": torch.empty_like(H),
              "ws": torch.empty(int(C.lib().fpq_cholesky_workspace_floats(d)), dtype=torch.float32, device=H.device),
              "status": torch.zeros(1, dtype=torch.int32, device=H.device)}
        flag = device_error_flag(H.device).data_ptr()

        def run():
            with _guard(H.device):
                C.call("fpq_cholesky_inverse_upper", st["H"].data_ptr(), st["U"].data_ptr(), d, st["ws"].data_ptr(),
                       st["status"].data_ptr(), flag, _stream(H))
        st["H"].copy_(H)
        return st, run

    graph, st = _capture(("chol", H.device.index, d), build)
    st["H"].copy_(H)
    graph.replay()
    return st["U"].clone(), st["status"].clone()


def gptq_quantize_graphed(W: torch.Tensor, scales: torch.Tensor, U: torch.Tensor, group: int,
                          group_index: Optional[torch.Tensor] = None):
    """`gptq_quantize` (codes wanted) replayed from a CUDA graph captured per shape; W is updated in place."""
    W, scales, U = _f32(W, "W", inplace=True), _f32(scales, "scales"), _f32(U, "U")
    rows, cols = W.shape
    ordered = group_index is not None

    def build():
        dev = W.device
        st = {"W": torch.empty_like(W), "scales": torch.empty_like(scales), "U": torch.empty_like(U),
              "codes": torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev),
              "ws": torch.empty(int(C.lib().fpq_gptq_workspace_bytes(rows, cols)), dtype=torch.uint8, device=dev),
              "gidx": torch.empty(cols, dtype=torch.int32, device=dev) if ordered else None}
        flag = device_error_flag(dev).data_ptr()

        def run():
            with _guard(dev):
                C.call("fpq_gptq_quantize_ordered", st["W"].data_ptr(), rows, cols, st["scales"].data_ptr(), group,
                       _ptr(st["gidx"]), st["U"].data_ptr(), st["codes"].data_ptr(), st["ws"].data_ptr(), flag, _stream(W))
        st["W"].copy_(W); st["scales"].copy_(scales); st["U"].copy_(U)
        if ordered:
            st["gidx"].copy_(group_index)
        return st, run

    graph, st = _capture(("gptq", W.device.index, rows, cols, group, ordered), build)
    st["W"].copy_(W); st["scales"].copy_(scales); st["U"].copy_(U)
    if ordered:
        st["gidx"].copy_(group_index)
    graph.replay()
    W.copy_(st["W"])
    return st["codes"].clone()


def gptq_quantize(W: torch.Tensor, scales: torch.Tensor, U: torch.Tensor, group: int, want_codes: bool = True,
                  group_index: Optional[torch.Tensor] = None):
    """Runs the GPTQ column loop on W in place (W becomes the dequantised weight).  Returns packed codes or None.
    `group_index` (int32 [cols]): activation order -- W's columns are already permuted and column c takes
    the static scale of group group_index[c]; W and the codes stay in the permuted order."""
    W, scales, U = _f32(W, "W", inplace=True), _f32(scales, "scales"), _f32(U, "U")
    rows, cols = W.shape
    if group_index is not None:
        if group_index.dtype != torch.int32 or not group_index.is_contiguous() or group_index.numel() != cols \
                or group_index.device != W.device:
            raise ValueError("group_index must be a contiguous int32 tensor of cols entries on W's device")
    codes = torch.empty(rows, cols // 2, dtype=torch.uint8, device=W.device) if want_codes else None
    ws = torch.empty(int(C.lib().fpq_gptq_workspace_bytes(rows, cols)), dtype=torch.uint8, device=W.device)
    with _guard(W.device):
        C.call("fpq_gptq_quantize_ordered", W.data_ptr(), rows, cols, scales.data_ptr(), group, _ptr(group_index),
               U.data_ptr(), _ptr(codes), ws.data_ptr(), device_error_flag(W.device).data_ptr(), _stream(W))
    return codes


def relative_mse(Wq: torch.Tensor, W: torch.Tensor, H: torch.Tensor, exact_fp32: bool = False) -> torch.Tensor:
    """Device fp32[1]: mean(((Wq-W) H) * (Wq-W)) / (mean((W H) * W) + 1e-6).
    Default: tensor-core form <H, A^T A> (~1e-5 relative); exact_fp32=True runs the two fp32 products."""
    Wq, W, H = _f32(Wq, "Wq"), _f32(W, "W"), _f32(H, "H")
    rows, d = W.shape
    if not exact_fp32 and d % 8 == 0:
        bf = torch.empty(2 * rows * d, dtype=torch.bfloat16, device=W.device)
        gram = torch.empty(d, d, dtype=torch.float32, device=W.device)
        acc = torch.empty(C.RELATIVE_MSE_ACC_DOUBLES, dtype=torch.float64, device=W.device)
        out = torch.empty(1, dtype=torch.float32, device=W.device)
        with _guard(W.device):
            C.call("fpq_relative_mse_tc", Wq.data_ptr(), W.data_ptr(), H.data_ptr(), rows, d, bf.data_ptr(),
                   gram.data_ptr(), acc.data_ptr(), out.data_ptr(), device_error_flag(W.device).data_ptr(), _stream(W))
        return out
    diff = torch.empty_like(W)
    acc = torch.empty(C.RELATIVE_MSE_ACC_DOUBLES, dtype=torch.float64, device=W.device)
    out = torch.empty(1, dtype=torch.float32, device=W.device)
    with _guard(W.device):
        C.call("fpq_relative_mse", Wq.data_ptr(), W.data_ptr(), H.data_ptr(), rows, d, diff.data_ptr(),
               acc.data_ptr(), out.data_ptr(), _stream(W))
    return out


def hessian_accumulate(H: torch.Tensor, x: torch.Tensor, alpha: float = 1.0, beta: float = 1.0) -> torch.Tensor:
    """H = beta * H + alpha * X^T X in place; X [..., d] bf16 (exact) or fp32 (split into three bf16
    terms whose six leading cross products are accumulated, ~2^-24 relative)."""
    H = _f32(H, "H", inplace=True)
    x = _cuda(x, "x")
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    flag = device_error_flag(H.device).data_ptr()

    def call(a, b, al, be):
        with _guard(H.device):
            C.call("fpq_hessian_accumulate", H.data_ptr(), d, a.data_ptr(), None if b is None else b.data_ptr(),
                   a.shape[0], float(al), float(be), flag, _stream(H))

    if x2.dtype == torch.bfloat16:
        call(x2.contiguous(), None, alpha, beta)
        return H
    if x2.dtype != torch.float32:
        x2 = x2.float()
    t0 = x2.to(torch.bfloat16)
    r1 = x2 - t0.float()
    t1 = r1.to(torch.bfloat16)
    t2 = (r1 - t1.float()).to(torch.bfloat16)
    call(t0, None, alpha, beta)
    call(t1, None, alpha, 1.0)
    for a, b in ((t0, t1), (t1, t0), (t0, t2), (t2, t0)):
        call(a, b, alpha, 1.0)
    return H
