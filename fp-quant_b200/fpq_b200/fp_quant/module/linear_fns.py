"""Forward functions of the quantised linear layer, mirroring
inference_lib/src/fp_quant/module/linear_fns.py (IST-DASLab/FP-Quant): `forward_quantize`,
`forward_gemm` and the two bf16-backward autograd functions.  Only the forward pass is on the
B200 path; backward through quantised weights raises like the reference does, and backward
through master weights is the plain bf16 einsum of the reference.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch.autograd import Function

from ..utils.config import FPQuantDtype
from .qutlass_ops import (fused_quantize_blocked_op, fused_quantize_mx_op, fused_quantize_nv_op,
                          matmul_fp4_bf16_tn_blocked_op, matmul_mxf4_bf16_tn_op, matmul_nvf4_bf16_tn_op)


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
