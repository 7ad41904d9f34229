from .config import FPQuantConfig, FPQuantDtype, validate_config
from .replace import (finalize_master_weights, fuse_gated_mlp_activation, replace_quantize_with_fp_quant_linear,
                      replace_with_fp_quant_linear)
