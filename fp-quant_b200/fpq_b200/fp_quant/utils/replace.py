"""Module-replacement helpers with the interface of inference_lib/src/fp_quant/utils/replace.py
(IST-DASLab/FP-Quant)."""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from .config import FPQuantConfig


def _skip(name: str, modules_to_not_convert: List[str]) -> bool:
    return any(name.endswith(key) for key in modules_to_not_convert)


def replace_with_fp_quant_linear(model: nn.Module, fp_quant_linear_config: FPQuantConfig,
                                 current_key_name: Optional[List[str]] = None, has_been_replaced: bool = False):
    """Swap every nn.Linear (outside `modules_to_not_convert`) for an FPQuantLinear allocated on the
    meta device; weights are filled in by the checkpoint loader, then `pre_forward()` is called
    (replace.py:7-71).  Returns (model, has_been_replaced)."""
    from ..module.linear import FPQuantLinear

    current_key_name = current_key_name or []
    for name, module in model.named_children():
        current_key_name.append(name)
        full = ".".join(current_key_name)
        if isinstance(module, nn.Linear) and not _skip(full, fp_quant_linear_config.modules_to_not_convert):
            with torch.device("meta"):
                new = FPQuantLinear(module.in_features, module.out_features, config=fp_quant_linear_config,
                                    bias=module.bias is not None, dtype=module.weight.dtype)
            new.source_cls = type(module)
            new.requires_grad_(False)
            model._modules[name] = new
            has_been_replaced = True
        if len(list(module.children())) > 0:
            _, has_been_replaced = replace_with_fp_quant_linear(module, fp_quant_linear_config, current_key_name,
                                                                has_been_replaced)
        current_key_name.pop(-1)
    return model, has_been_replaced


def replace_quantize_with_fp_quant_linear(model: nn.Module, fp_quant_linear_config: FPQuantConfig,
                                          current_key_name: Optional[List[str]] = None):
    """Same walk, but for a model whose weights are already materialised: hand them to the new
    module and quantise immediately (replace.py:74-117).  Returns the model."""
    from ..module.linear import FPQuantLinear

    current_key_name = current_key_name or []
    for name, module in model.named_children():
        current_key_name.append(name)
        full = ".".join(current_key_name)
        if isinstance(module, nn.Linear) and not _skip(full, fp_quant_linear_config.modules_to_not_convert):
            new = FPQuantLinear(module.in_features, module.out_features, config=fp_quant_linear_config,
                                bias=module.bias is not None, device=module.weight.device,
                                dtype=module.weight.dtype)
            new.weight.data = module.weight.data
            if module.bias is not None:
                new.bias.data = module.bias.data
            new.pre_forward()
            model._modules[name] = new
        if len(list(module.children())) > 0:
            replace_quantize_with_fp_quant_linear(module, fp_quant_linear_config, current_key_name)
        current_key_name.pop(-1)
    return model


def finalize_master_weights(model: nn.Module, current_key_name=None) -> None:
    """Turn layers trained with master weights into inference layers: clear the (shared) config
    flag and run `pre_forward()` on every FPQuantLinear, which quantises the weight once and
    drops the master copy (replace.py:120-144)."""
    from ..module.linear import FPQuantLinear

    for module in model.modules():
        if isinstance(module, FPQuantLinear):
            if module.config.store_master_weights:
                module.config.store_master_weights = False
            if module.weight is not None:
                module.pre_forward()


def fuse_gated_mlp_activation(model: nn.Module) -> int:
    """Route `down_proj(act_fn(gate_proj(x)) * up_proj(x))` of every gated-SiLU MLP whose down-projection is an
    FPQuantLinear through `FPQuantLinear.forward_silu_mul`, which evaluates SiLU(gate) * up inside the quantise
    kernel of the down-projection.  The reference leaves that product to a separate elementwise kernel followed
    by the rotation and the quantiser (src/utils/llama_utils.py:62-70); this helper is an addition of this
    package, not part of the reference's interface.  Modules are recognised by their attributes (`gate_proj`,
    `up_proj`, `down_proj`, `act_fn` = SiLU), as the Llama / Qwen / Mistral MLP classes of transformers have them.
    Returns the number of modules patched."""
    import types

    from ..module.linear import FPQuantLinear

    def forward(self, x):
        return self.down_proj.forward_silu_mul(self.gate_proj(x), self.up_proj(x))

    patched = 0
    for module in model.modules():
        act = getattr(module, "act_fn", None)
        is_silu = isinstance(act, nn.SiLU) or type(act).__name__ in ("SiLUActivation", "SiLU") or act is torch.nn.functional.silu
        if (is_silu and isinstance(getattr(module, "down_proj", None), FPQuantLinear)
                and hasattr(module, "gate_proj") and hasattr(module, "up_proj")):
            module.forward = types.MethodType(forward, module)
            patched += 1
    return patched
