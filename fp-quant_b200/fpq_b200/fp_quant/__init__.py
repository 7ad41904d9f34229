"""Drop-in for the `fp_quant` inference package (inference_lib/src/fp_quant/__init__.py)."""
from .module import FPQuantLinear
from .utils import (FPQuantConfig, FPQuantDtype, finalize_master_weights, fuse_gated_mlp_activation,
                    replace_quantize_with_fp_quant_linear, replace_with_fp_quant_linear, validate_config)

__all__ = ["FPQuantLinear", "FPQuantConfig", "FPQuantDtype", "validate_config", "replace_with_fp_quant_linear",
           "replace_quantize_with_fp_quant_linear", "finalize_master_weights", "fuse_gated_mlp_activation"]
