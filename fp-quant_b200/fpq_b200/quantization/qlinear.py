"""`QLinear` with the interface of src/quantization/qlinear.py (IST-DASLab/FP-Quant): a linear
layer whose weight (while `_train_mode`) and activations pass through rotate + fake-quantise.
The quantise-dequantise of each tensor is one fused kernel pass instead of the reference's chain
of elementwise torch ops; the matmul itself is the ordinary bf16 `F.linear`, as in the reference."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..transforms.transforms import BaseTransform, HadamardTransform
from .quantizer import Quantizer


def _fake_quantize(quantizer: Quantizer, x: torch.Tensor) -> torch.Tensor:
    return quantizer.fused_fake_quantize(x, hadamard_group=0, ste=False)


class QLinear(nn.Linear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, weight_quantizer: Quantizer = None,
                 act_quantizer: Quantizer = None, device: torch.device = None, dtype: torch.dtype = None):
        super().__init__(in_features, out_features, bias, device, dtype)
        self.weight_quantizer = weight_quantizer
        self.act_quantizer = act_quantizer
        self._train_mode = True

    def _prepared_weight(self, in_transform, out_transform, freeze: bool):
        weight, bias = self.weight, self.bias
        if out_transform is not None:
            raise NotImplementedError("output-side transforms are outside the MR-GPTQ path")
        if in_transform is not None:
            weight = in_transform(weight, inv_t=True, dim=-1)
        if self.weight_quantizer is not None:
            weight = _fake_quantize(self.weight_quantizer, weight)
            if freeze:
                self.weight_quantizer._track_global_scale = False
        return weight, bias

    def forward(self, x: torch.Tensor, in_transform: BaseTransform = None, out_transform: BaseTransform = None):
        weight, bias = self.weight, self.bias
        if self._train_mode:
            weight, bias = self._prepared_weight(in_transform, out_transform, freeze=False)
        if self.act_quantizer is not None:
            x = _fake_quantize(self.act_quantizer, x)
        return F.linear(x, weight, bias)

    @torch.no_grad()
    def fix_parametrization(self, in_transform: BaseTransform = None, out_transform: BaseTransform = None) -> None:
        weight, bias = self._prepared_weight(in_transform, out_transform, freeze=True)
        if self.act_quantizer is not None:
            self.act_quantizer._track_global_scale = False
        self.weight.data = weight
        if bias is not None:
            self.bias.data = bias
        self._train_mode = False
