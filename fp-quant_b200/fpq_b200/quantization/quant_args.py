"""String enums of the quantisation API (same names and values as
src/quantization/quant_args.py of IST-DASLab/FP-Quant)."""
from enum import Enum


class _StrEnum(str, Enum):
    def __str__(self) -> str:  # so f-strings print the value
        return self.value


QuantizationFormat = _StrEnum("QuantizationFormat", {"INT": "int", "FP": "fp", "NVFP": "nvfp", "MXFP": "mxfp"})
QuantizationGranularity = _StrEnum("QuantizationGranularity", {"TENSOR": "tensor", "CHANNEL": "channel", "GROUP": "group"})
QuantizationObserver = _StrEnum("QuantizationObserver", {"MINMAX": "minmax", "MSE": "mse"})
QuantizationOrder = _StrEnum("QuantizationOrder", {"DEFAULT": "default", "ACTIVATION": "activation"})
ScalePrecision = _StrEnum("ScalePrecision", {"FP16": "fp16", "E4M3": "e4m3", "E8M0": "e8m0"})
