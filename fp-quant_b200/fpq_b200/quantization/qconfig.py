"""`prepare_quantization_config` with the fields of src/quantization/qconfig.py:3-20 (IST-DASLab/FP-Quant):
the `quantization_config` block written into an exported model's config.json, which is what the
`fp_quant` loader of transformers / vLLM reads to rebuild the FPQuantLinear layers."""
from typing import Any, Dict


def prepare_quantization_config(hadamard_group_size: int, format: str, pseudoquantization: bool = False) -> Dict[str, Any]:
    fmt = getattr(format, "value", format)
    if fmt in ("mxfp", "nvfp"):
        return {
            "forward_dtype": f"{fmt}4",
            "backward_dtype": "bf16",
            "forward_method": "abs_max",
            "hadamard_group_size": hadamard_group_size,
            "modules_to_not_convert": ["lm_head"],
            "quant_method": "fp_quant",
            "store_master_weights": False,
            "pseudoquantization": pseudoquantization,
        }
    raise ValueError(f"Invalid format: {format}")
