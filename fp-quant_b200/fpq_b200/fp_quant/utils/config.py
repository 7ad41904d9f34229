"""`FPQuantConfig` / `FPQuantDtype` / `validate_config` with the fields and checks of
inference_lib/src/fp_quant/utils/config.py (IST-DASLab/FP-Quant)."""
from dataclasses import dataclass, field
from enum import Enum
from typing import List, Literal


class FPQuantDtype(Enum):
    MXFP4 = "mxfp4"
    NVFP4 = "nvfp4"
    MXFP8 = "mxfp8"
    BF16 = "bf16"


QuantMethod = Literal["quest", "abs_max"]
TransformInit = Literal["hadamard", "identity", "gsr"]


@dataclass
class FPQuantConfig:
    forward_dtype: FPQuantDtype = FPQuantDtype.MXFP4
    forward_method: QuantMethod = "quest"
    backward_dtype: FPQuantDtype = FPQuantDtype.MXFP4
    store_master_weights: bool = False
    hadamard_group_size: int = 32
    pseudoquantization: bool = False
    transform_init: TransformInit = "hadamard"
    modules_to_not_convert: List[str] = field(default_factory=lambda: ["lm_head"])


_GROUPS = {FPQuantDtype.NVFP4: (16, 32, 64, 128), FPQuantDtype.MXFP4: (32, 64, 128)}


def validate_config(config: FPQuantConfig) -> None:
    fwd, bwd = config.forward_dtype, config.backward_dtype
    if fwd == FPQuantDtype.NVFP4 and config.forward_method != "abs_max":
        raise ValueError("NVFP4 can only be used with abs_max method")
    for dt, groups in _GROUPS.items():
        if fwd == dt and config.hadamard_group_size not in groups:
            raise ValueError(f"{dt.name} can only be used with hadamard_group_size in {list(groups)}")
    if fwd == FPQuantDtype.MXFP8 or (bwd == FPQuantDtype.MXFP8 and fwd != FPQuantDtype.MXFP4):
        raise ValueError("MXFP8 can only be used on backward in combination with MXFP4 forward")
    if bwd == FPQuantDtype.MXFP4 and fwd != FPQuantDtype.MXFP4:
        raise ValueError("MXFP4 backward can only be used with MXFP4 forward")
