"""Pseudo-quantised forward (quantise-dequantise activations, bf16 matmul), mirroring
inference_lib/src/fp_quant/module/pseudoquant_linear_fns.py (IST-DASLab/FP-Quant).  The
Triton kernels of the reference are replaced by the fused fake-quantise CUDA kernel, which
uses the Quantizer's rounding (ties to even) rather than Triton's strict-greater thresholds."""
from __future__ import annotations

from typing import Tuple

import torch
from torch.autograd import Function

from ... import ops
from ...rotation import classify_rotation
from ..utils.config import FPQuantDtype


def forward_pseudoquantize(x: torch.Tensor, hadamard_matrix: torch.Tensor, global_scale: torch.Tensor,
                           dtype: FPQuantDtype, forward_method: str) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dequantised rotate+quantise of x and the clip mask (all ones for abs_max; for quest the elements
    with |x / divisor| < 6) (pseudoquant_linear_fns.py:12-48)."""
    if dtype not in (FPQuantDtype.MXFP4, FPQuantDtype.NVFP4):
        if dtype == FPQuantDtype.MXFP8:
            raise NotImplementedError("MXFP8 is not supported for forward quantization yet")
        raise ValueError(f"Unsupported forward dtype: {dtype}")
    if forward_method not in ("abs_max", "quest"):
        raise ValueError(f"Unsupported forward method: {forward_method}")
    if forward_method == "quest" and dtype == FPQuantDtype.NVFP4:
        raise AssertionError("NVFP4 only supports abs_max method")
    fmt = "nvfp4" if dtype == FPQuantDtype.NVFP4 else "mxfp4"
    kind, group = classify_rotation(hadamard_matrix)
    xin = x if x.dtype in (torch.bfloat16, torch.float32) else x.to(torch.bfloat16)
    if kind == "dense":
        xin, group = ops.rotate_dense(xin.reshape(-1, x.shape[-1]), hadamard_matrix).view(x.shape), 0
    elif kind == "identity":
        group = 0
    if forward_method == "quest":          # std-based scales; the mask marks the elements inside the grid's range
        y, mask = ops.fake_quantize_quest(xin, group, return_mask=True)
        return y.to(x.dtype), mask
    gs = global_scale.float() if fmt == "nvfp4" else None
    y = ops.fake_quantize(xin, fmt, group, gs).to(x.dtype)
    return y, torch.ones_like(y, dtype=torch.bool)


class PseudoQuant4x16NoMasterFn(Function):
    """F.linear on pseudo-quantised activations and a stored dequantised weight
    (pseudoquant_linear_fns.py:134-168; the reference adds the bias twice there, this does not)."""

    @staticmethod
    def forward(ctx, x, weight_dq, weight_global_scale, act_global_scale, bias, forward_hadamard_matrix, dtype,
                forward_method):
        x_flat = x.contiguous().flatten(end_dim=-2)
        x_dq, _ = forward_pseudoquantize(x_flat, forward_hadamard_matrix, act_global_scale, dtype, forward_method)
        y = torch.nn.functional.linear(x_dq, weight_dq, bias)
        return y.unflatten(dim=0, sizes=x.shape[:-1])

    @staticmethod
    def backward(ctx, grad_output):
        raise NotImplementedError("training through the pseudo-quantised path is outside the B200 hot path")


class PseudoQuant4x16MasterFn(Function):
    @staticmethod
    def forward(ctx, x, weight, weight_global_scale, act_global_scale, bias, forward_hadamard_matrix, dtype,
                forward_method):
        w_dq, _ = forward_pseudoquantize(weight, forward_hadamard_matrix, weight_global_scale, dtype, forward_method)
        return PseudoQuant4x16NoMasterFn.forward(ctx, x, w_dq, weight_global_scale, act_global_scale, bias,
                                                 forward_hadamard_matrix, dtype, forward_method)

    @staticmethod
    def backward(ctx, grad_output):
        raise NotImplementedError("training through the pseudo-quantised path is outside the B200 hot path")
