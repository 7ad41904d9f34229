from .accumulate_hessian import accumulate_hessian
from .driver import gptq_quantization, rtn_quantization
from .export import export_quantized_model, load_quantized_checkpoint
from .gptq import GPTQ, get_relative_mse_error
from .qconfig import prepare_quantization_config
from .qlinear import QLinear
from .quant_args import (QuantizationFormat, QuantizationGranularity, QuantizationObserver, QuantizationOrder,
                         ScalePrecision)
from .quantizer import Quantizer
