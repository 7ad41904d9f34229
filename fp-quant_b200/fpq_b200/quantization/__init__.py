from .accumulate_hessian import accumulate_hessian
from .driver import gptq_quantization, rtn_quantization
from .gptq import GPTQ, get_relative_mse_error
from .qlinear import QLinear
from .quant_args import (QuantizationFormat, QuantizationGranularity, QuantizationObserver, QuantizationOrder,
                         ScalePrecision)
from .quantizer import Quantizer
