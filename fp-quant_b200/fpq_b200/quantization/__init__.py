from .quant_args import (QuantizationFormat, QuantizationGranularity, QuantizationObserver, QuantizationOrder,
                         ScalePrecision)
from .quantizer import Quantizer
