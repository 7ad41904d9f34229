"""Forward functions of the quantised linear layer, mirroring
inference_lib/src/fp_quant/module/linear_fns.py (IST-DASLab/FP-Quant): `forward_quantize`,
`forward_gemm`, the two bf16-backward autograd functions and the MXFP8-backward pair
(`FPQuant4x8MasterFn`: both gradient GEMMs on MXFP8 operands).  Backward through pre-quantised
weights raises like the reference does.  `FPQuant4x4MasterFn` runs both gradient GEMMs on MXFP4 operands.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch.autograd import Function

from ..utils.config import FPQuantDtype
from ... import ops
from ...rotation import kind_of
from .qutlass_ops import (backward_bf16_square_double_mxfp8_op, backward_qt_bf16_op, backward_t_bf16_op,
                          fused_quantize_blocked_op, fused_quantize_mx_op,
                          fused_quantize_nv_op, matmul_fp4_bf16_tn_blocked_op, matmul_mxf4_bf16_tn_op,
                          matmul_mxf8_bf16_nn_op, matmul_mxf8_bf16_tn_op, matmul_nvf4_bf16_tn_op,
                          mxfp4_transpose_mxfp8_op)


def forward_quantize(x: torch.Tensor, hadamard_matrix: torch.Tensor, global_scale: torch.Tensor,
                     dtype: FPQuantDtype, forward_method: str) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """rotate + quantise -> (codes, row-major padded scales, mask) (linear_fns.py:27-50)."""
    if dtype == FPQuantDtype.MXFP4:
        return fused_quantize_mx_op(x.to(torch.bfloat16), hadamard_matrix.to(torch.bfloat16), forward_method,
                                    forward_method == "quest" and x.requires_grad)
    if dtype == FPQuantDtype.NVFP4:
        q, s = fused_quantize_nv_op(x.to(torch.bfloat16), hadamard_matrix.to(torch.bfloat16), global_scale.float())
        return q, s, None
    raise ValueError(f"Unsupported forward dtype: {dtype}")


def forward_gemm(x_q, w_q, x_scales, w_scales, alpha, dtype: FPQuantDtype):
    """bf16 = alpha * dq(x_q) dq(w_q)^T from row-major scales (linear_fns.py:53-64)."""
    if dtype == FPQuantDtype.MXFP4:
        return matmul_mxf4_bf16_tn_op(x_q, w_q, x_scales, w_scales, alpha.float())
    if dtype == FPQuantDtype.NVFP4:
        return matmul_nvf4_bf16_tn_op(x_q, w_q, x_scales, w_scales, alpha.float())
    raise ValueError(f"Unsupported dtype: {dtype}")


def forward_quantize_blocked(x, hadamard_matrix, global_scale, dtype: FPQuantDtype, forward_method: str,
                             rotation: int = 0):
    """Fast path of `forward_quantize`: scales come out in the layout the matmul reads."""
    if dtype not in (FPQuantDtype.MXFP4, FPQuantDtype.NVFP4):
        raise ValueError(f"Unsupported forward dtype: {dtype}")
    if forward_method not in ("abs_max", "quest"):
        raise ValueError(f"Unsupported forward method: {forward_method}")
    return fused_quantize_blocked_op(x.to(torch.bfloat16), hadamard_matrix.to(torch.bfloat16), global_scale.float(),
                                     dtype == FPQuantDtype.NVFP4, rotation, forward_method == "quest")


def forward_gemm_blocked(x_q, w_q, x_scales_blocked, w_scales_blocked, alpha, dtype: FPQuantDtype, bias=None):
    if dtype not in (FPQuantDtype.MXFP4, FPQuantDtype.NVFP4):
        raise ValueError(f"Unsupported dtype: {dtype}")
    return matmul_fp4_bf16_tn_blocked_op(x_q, w_q, x_scales_blocked, w_scales_blocked, alpha.float(),
                                         dtype == FPQuantDtype.NVFP4, bias)


def gemm_alpha(weight_global_scale: torch.Tensor, act_global_scale: torch.Tensor) -> torch.Tensor:
    """fp32 [1]: 1 / (weight_global_scale * act_global_scale) with the reference's rounding order -- product
    and reciprocal in the dtype of the buffers (bf16 once `pre_forward` made them), then the cast to fp32
    (linear_fns.py:433, :505 and `alpha.float()` at :57-62).  For the abs_max default 3 * 3 this is
    bf16(1/9) = 0.111328, not 0.111111."""
    return (1.0 / (weight_global_scale * act_global_scale)).float().reshape(1)


def _linear_forward(x, weight_q, weight_scales_blocked, weight_global_scale, act_global_scale, bias,
                    hadamard_matrix, dtype, forward_method, alpha=None):
    x_flat = x.contiguous().flatten(end_dim=-2)
    x_q, x_scales = forward_quantize_blocked(x_flat, hadamard_matrix, act_global_scale, dtype, forward_method)
    if alpha is None:
        alpha = gemm_alpha(weight_global_scale, act_global_scale)
    # the bias is added in the GEMM's epilogue (fp32 accumulator + bias, one rounding to bf16) instead of
    # the reference's separate bf16 add (linear_fns.py:514-515)
    fused_bias = bias if bias is not None and bias.dtype == torch.bfloat16 else None
    y = forward_gemm_blocked(x_q, weight_q, x_scales, weight_scales_blocked, alpha, dtype, fused_bias)
    y = y.unflatten(dim=0, sizes=x.shape[:-1])
    if bias is not None and fused_bias is None:
        y = y + bias
    return y


class FPQuant4x16NoMasterFn(Function):
    """Inference forward with pre-quantised weights (linear_fns.py:482-528).  `weight_scales` are
    the weight scale bytes already in the swizzled layout (cached by the module)."""

    @staticmethod
    def forward(ctx, x, weight_q, weight_scales, weight_global_scale, act_global_scale, bias,
                forward_hadamard_matrix, dtype, forward_method, alpha=None):
        """`alpha` (optional, fp32 [1]): the module's cached `gemm_alpha` of the two tensor scales."""
        return _linear_forward(x, weight_q, weight_scales, weight_global_scale, act_global_scale, bias,
                               forward_hadamard_matrix, dtype, forward_method, alpha)

    @staticmethod
    def backward(ctx, grad_output):
        raise NotImplementedError("Backward pass is not implemented for FPQuant4x16NoMasterFn yet")


class FPQuant4x16MasterFn(Function):
    """Forward quantises the bf16 master weight on the fly; backward is plain bf16
    (linear_fns.py:405-479)."""

    @staticmethod
    def forward(ctx, x, weight, weight_global_scale, act_global_scale, bias, forward_hadamard_matrix, dtype,
                forward_method):
        w_q, w_scales = forward_quantize_blocked(weight, forward_hadamard_matrix, weight_global_scale, dtype,
                                                 forward_method)
        y = _linear_forward(x, w_q, w_scales, weight_global_scale, act_global_scale, bias,
                            forward_hadamard_matrix, dtype, forward_method)
        ctx.x_shape, ctx.bias_present = x.shape, bias is not None
        ctx.save_for_backward(x.contiguous().flatten(end_dim=-2), weight)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        x_flat, weight = ctx.saved_tensors
        g = grad_output.flatten(end_dim=-2)
        grad_input = (g @ weight).view(ctx.x_shape)
        grad_weight = g.t() @ x_flat
        grad_bias = g.sum(dim=0) if ctx.bias_present else None
        return grad_input, grad_weight, None, None, grad_bias, None, None, None


def _unpack_mask(clip_mask: torch.Tensor) -> torch.Tensor:
    """[.., K/8] bytes -> [.., K] bool, bit i of byte b = element 8 b + i (linear_fns.py:67-77)."""
    bits = (clip_mask.unsqueeze(-1) >> torch.arange(8, device=clip_mask.device, dtype=torch.uint8)) & 1
    return bits.flatten(start_dim=-2).bool()


def _unrotate(g: torch.Tensor, hadamard_matrix: torch.Tensor) -> torch.Tensor:
    """`g.view(-1, h) @ hadamard_matrix.T` in bf16 (linear_fns.py:321-324): gradient with respect to the
    rotated operand -> gradient with respect to the operand.  The normalised Sylvester matrix is symmetric,
    so the butterfly kernel does it; any other matrix takes the dense product."""
    kind, group = kind_of(0, hadamard_matrix)
    if kind == "identity":
        return g
    if kind == "hadamard":
        return ops.rotate_hadamard(g.contiguous(), group, out_dtype=torch.bfloat16)
    return ops.rotate_dense(g.contiguous(), hadamard_matrix.t().contiguous(), out_dtype=torch.bfloat16)


def _row_major_scales(scales: torch.Tensor, rows: int, sf_cols: int) -> torch.Tensor:
    sb = scales.view(torch.uint8)
    return sb if tuple(sb.shape) == (rows, sf_cols) else sb[:rows, :sf_cols].contiguous()


def _mxfp8_backward(grad_output, x_q, w_q, x_scales, w_scales, act_global_scale, weight_global_scale, x_mask, w_mask,
                    hadamard_matrix, x_shape, want_weight_grad: bool):
    """The two gradient GEMMs of linear_fns.py:270-350 on MXFP8 operands.  The saved MXFP4 operands are
    transposed into MXFP8 (exactly, unless the scales of a 32-row band differ by more than 2^14), the bf16
    gradient is quantised once with a scale per 32 x 32 square and read along either axis.

    Same data flow as the reference's `mxfp4_transpose_mxfp8_op` / `backward_bf16_square_double_mxfp8_op` /
    `matmul_mxf8_bf16_tn_op` / `..._nn_op` sequence, with the re-layouts folded into the producers: the
    quantisers write their scales in the layout the GEMM reads, and the gradient's bytes come out in both
    orientations, so the `nn` product is a `tn` product of the transposed copy."""
    g = grad_output.flatten(end_dim=-2).to(torch.bfloat16).contiguous()
    tokens, out_features = g.shape
    in_features = w_q.size(-1) * 2
    g_fp8, g_row_scales, g_col_scales, g_t_fp8 = ops.quantize_mxfp8_square(g, swizzled=True, transposed=want_weight_grad) \
        if want_weight_grad else ops.quantize_mxfp8_square(g, swizzled=True) + (None,)
    if out_features % 128 == 0:
        w_t_fp8, w_t_scales = ops.mxfp4_transpose_mxfp8(w_q.view(torch.uint8), _row_major_scales(w_scales, out_features, in_features // 32),
                                                        swizzled=True)
    else:     # the transposed weight is padded along the contraction axis: cut it back to the gradient's width
        w_t_fp8, w_t_scales = ops.mxfp4_transpose_mxfp8(w_q.view(torch.uint8), _row_major_scales(w_scales, out_features, in_features // 32))
        w_t_fp8 = w_t_fp8[:, :out_features].contiguous()
        w_t_scales = ops.swizzle_scales(w_t_scales[:, : out_features // 32].contiguous())
    grad_input = ops.gemm_mxf8(g_fp8, w_t_fp8, g_row_scales, w_t_scales, (1.0 / weight_global_scale.float()).reshape(1))[:tokens]
    if x_mask is not None:
        grad_input = grad_input * _unpack_mask(x_mask).view_as(grad_input).to(grad_input.dtype)
    grad_input = _unrotate(grad_input, hadamard_matrix).view(x_shape)
    grad_weight = None
    if want_weight_grad:
        x_t_fp8, x_t_scales = ops.mxfp4_transpose_mxfp8(x_q.view(torch.uint8), _row_major_scales(x_scales, tokens, in_features // 32),
                                                        swizzled=True)                       # [in, tokens_up128]
        grad_weight = ops.gemm_mxf8(g_t_fp8, x_t_fp8, g_col_scales, x_t_scales, (1.0 / act_global_scale.float()).reshape(1))
        if w_mask is not None:
            grad_weight = grad_weight * _unpack_mask(w_mask).view_as(grad_weight).to(grad_weight.dtype)
        grad_weight = _unrotate(grad_weight, hadamard_matrix).view(out_features, in_features)
    return grad_input, grad_weight


class FPQuant4x8MasterFn(Function):
    """MXFP4 forward from a bf16 master weight, MXFP8 backward (linear_fns.py:232-350)."""

    @staticmethod
    def forward(ctx, x, weight, weight_global_scale, act_global_scale, bias, forward_hadamard_matrix, dtype,
                forward_method):
        x_flat = x.contiguous().flatten(end_dim=-2)
        x_q, x_scales, x_mask = forward_quantize(x_flat, forward_hadamard_matrix, act_global_scale, dtype, forward_method)
        w_q, w_scales, w_mask = forward_quantize(weight, forward_hadamard_matrix, weight_global_scale, dtype, forward_method)
        y = forward_gemm(x_q, w_q, x_scales, w_scales, 1.0 / (weight_global_scale * act_global_scale), dtype)
        y = y.unflatten(dim=0, sizes=x.shape[:-1])
        if bias is not None:
            y = y + bias
        ctx.x_shape, ctx.bias_present = x.shape, bias is not None
        ctx.masks = (x_mask, w_mask)
        ctx.save_for_backward(x_q, w_q, x_scales, w_scales, act_global_scale, weight_global_scale, forward_hadamard_matrix)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        x_q, w_q, x_scales, w_scales, act_global_scale, weight_global_scale, hadamard_matrix = ctx.saved_tensors
        x_mask, w_mask = ctx.masks
        grad_input, grad_weight = _mxfp8_backward(grad_output, x_q, w_q, x_scales, w_scales, act_global_scale,
                                                  weight_global_scale, x_mask, w_mask, hadamard_matrix, ctx.x_shape, True)
        grad_bias = grad_output.flatten(end_dim=-2).sum(dim=0) if ctx.bias_present else None
        return grad_input, grad_weight, None, None, grad_bias, None, None, None


class FPQuant4x8NoMasterFn(Function):
    """MXFP4 forward from pre-quantised weights (row-major scale bytes as stored in a checkpoint); the
    backward raises, as the reference's does (linear_fns.py:352-404)."""

    @staticmethod
    def forward(ctx, x, weight_q, weight_scales, weight_global_scale, act_global_scale, bias, forward_hadamard_matrix,
                dtype, forward_method):
        x_flat = x.contiguous().flatten(end_dim=-2)
        x_q, x_scales, _ = forward_quantize(x_flat, forward_hadamard_matrix, act_global_scale, dtype, forward_method)
        y = forward_gemm(x_q, weight_q, x_scales, weight_scales, 1.0 / (weight_global_scale * act_global_scale), dtype)
        y = y.unflatten(dim=0, sizes=x.shape[:-1])
        if bias is not None:
            y = y + bias
        return y

    @staticmethod
    def backward(ctx, grad_output):
        raise NotImplementedError("Backward pass is not implemented for FPQuant4x8NoMasterFn yet")


class FPQuant4x4MasterFn(Function):
    """MXFP4 forward from a bf16 master weight, MXFP4 backward (linear_fns.py:80-230): the gradient and the
    dequantised, transposed operands are rotated along the contraction axis with the Hadamard matrix,
    quantised to MXFP4 again (abs_max), and both gradient GEMMs run on the FP4 kernel."""

    @staticmethod
    def forward(ctx, x, weight, weight_global_scale, act_global_scale, bias, forward_hadamard_matrix, dtype,
                forward_method):
        x_flat = x.contiguous().flatten(end_dim=-2)
        x_q, x_scales, x_mask = forward_quantize(x_flat, forward_hadamard_matrix, act_global_scale, dtype, forward_method)
        w_q, w_scales, w_mask = forward_quantize(weight, forward_hadamard_matrix, weight_global_scale, dtype, forward_method)
        y = forward_gemm(x_q, w_q, x_scales, w_scales, 1.0 / (weight_global_scale * act_global_scale), dtype)
        y = y.unflatten(dim=0, sizes=x.shape[:-1])
        if bias is not None:
            y = y + bias
        ctx.x_shape, ctx.bias_present = x.shape, bias is not None
        ctx.masks = (x_mask, w_mask)
        ctx.save_for_backward(x_q, w_q, x_scales, w_scales, act_global_scale, weight_global_scale, forward_hadamard_matrix)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        x_q, w_q, x_scales, w_scales, act_global_scale, weight_global_scale, hadamard_matrix = ctx.saved_tensors
        x_mask, w_mask = ctx.masks
        # The reference multiplies the columns of the Hadamard matrix by fresh random signs here
        # (linear_fns.py:151-158).  With y = x @ (H D) that flips the sign of whole columns of both rotated
        # operands of a GEMM, which neither the sign-symmetric quantiser nor the product of the two notices:
        # both gradients are bit-identical with D = I.  The plain matrix is used, so the rotation stays on the
        # butterfly of the quantise kernel instead of a dense product.
        backward_hadamard_matrix = hadamard_matrix.to(torch.bfloat16)
        g = grad_output.flatten(end_dim=-2).to(torch.bfloat16).contiguous()
        tokens, out_features = g.shape
        in_features = w_q.size(-1) * 2
        # abs_max MXFP4 carries a factor 3 per operand (the scale is a third of the power of two that is stored)
        ninth = torch.full((1,), 1.0 / 9.0, dtype=torch.float32, device=g.device)
        kind, group = kind_of(0, backward_hadamard_matrix)
        if kind in ("hadamard", "identity") and group <= 32 and out_features % 8 == 0:
            # Same data flow as the op sequence below with the re-layouts folded into the producers: scales come
            # out in the layout the GEMM reads, the transposes happen inside the (de)quantise kernels, and the
            # token axis is padded to a whole number of K tiles by the kernels that write it.
            gh = group if kind == "hadamard" else 0
            w_rm = _row_major_scales(w_scales, out_features, in_features // 32)
            x_rm = _row_major_scales(x_scales, tokens, in_features // 32)
            g_q, g_s, _ = ops.quantize(g, "mxfp4", gh, None, swizzled=True)
            wt = ops.mxfp4_transpose_dequant(w_q.view(torch.uint8), w_rm, weight_global_scale.float())        # [in, out]
            wt_q, wt_s, _ = ops.quantize(wt, "mxfp4", gh, None, swizzled=True)
            grad_input = ops.gemm_fp4(g_q, wt_q, g_s, wt_s, ninth, "mxfp4")
            gt_q, gt_s = ops.quantize_transposed(g, gh, pad_to=128, swizzled=True)                             # [out, tokens_up128]
            xt = ops.mxfp4_transpose_dequant(x_q.view(torch.uint8), x_rm, act_global_scale.float(), pad_to=128)   # [in, tokens_up128]
            xt_q, xt_s, _ = ops.quantize(xt, "mxfp4", gh, None, swizzled=True)
            grad_weight = ops.gemm_fp4(gt_q, xt_q, gt_s, xt_s, ninth, "mxfp4")
        else:
            g_q, g_scales, _ = fused_quantize_mx_op(g, backward_hadamard_matrix, "abs_max", False)
            wt_q, wt_scales = backward_qt_bf16_op(w_q, w_scales, backward_hadamard_matrix, weight_global_scale.float())
            grad_input = matmul_mxf4_bf16_tn_op(g_q, wt_q, g_scales, wt_scales, ninth)
            # the weight gradient contracts over the tokens: pad them to a whole number of K tiles with zero rows
            pad = (-tokens) % 128
            g_pad = torch.nn.functional.pad(g, (0, 0, 0, pad)) if pad else g
            gt_q, gt_scales = backward_t_bf16_op(g_pad, backward_hadamard_matrix)
            if pad:
                zero_codes = torch.full((pad, x_q.shape[1]), 0x88, dtype=torch.uint8, device=x_q.device)
                x_q_pad = torch.cat([x_q.view(torch.uint8), zero_codes])
                xs = x_scales.view(torch.uint8)[:tokens, : x_q.shape[1] // 16]
                xs_pad = torch.cat([xs, torch.full((pad, xs.shape[1]), 127, dtype=torch.uint8, device=xs.device)])
            else:
                x_q_pad, xs_pad = x_q, x_scales
            xt_q, xt_scales = backward_qt_bf16_op(x_q_pad, xs_pad, backward_hadamard_matrix, act_global_scale.float())
            grad_weight = matmul_mxf4_bf16_tn_op(gt_q, xt_q, gt_scales, xt_scales, ninth)
        if x_mask is not None:
            grad_input = grad_input * _unpack_mask(x_mask).view_as(grad_input).to(grad_input.dtype)
        grad_input = _unrotate(grad_input, hadamard_matrix).view(ctx.x_shape)
        if w_mask is not None:
            grad_weight = grad_weight * _unpack_mask(w_mask).view_as(grad_weight).to(grad_weight.dtype)
        grad_weight = _unrotate(grad_weight, hadamard_matrix).view(out_features, in_features)
        grad_bias = g.sum(dim=0) if ctx.bias_present else None
        return grad_input, grad_weight, None, None, grad_bias, None, None, None
