"""Checkpoint export and its loader round trip.

`export_quantized_model` writes what model_quant.py:41-119 (IST-DASLab/FP-Quant) writes: the model's
state dict with every quantised linear's `weight` replaced by the per-layer entries the drivers return
(`qweight`, `scales`, `forward_hadamard_matrix`, `backward_hadamard_matrix`, `weight_global_scale`,
`act_global_scale`; `dqweight` instead of the first two for pseudo-quantisation; src/quantization/gptq.py:427-444),
split into safetensors shards with an index file, plus config.json carrying the `quantization_config`
block of `prepare_quantization_config`.

`load_quantized_checkpoint` is the other half: it rebuilds FPQuantLinear layers in a freshly constructed
model from such a directory, the way the `fp_quant` quantizer of transformers does for a pre-quantised
checkpoint (replace the linears on the meta device, hand each checkpoint tensor to the attribute of its
name, drop the attributes the checkpoint does not carry).  It is what the round-trip test runs; it reads
nothing but the files written above."""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List, Tuple

import torch
from torch import nn

from .qconfig import prepare_quantization_config

QUANTIZED_KEYS = ("qweight", "scales", "dqweight", "forward_hadamard_matrix", "backward_hadamard_matrix",
                  "weight_global_scale", "act_global_scale")


def build_model_state_dict(model: nn.Module, quantized_state_dict: Dict[str, Dict[str, torch.Tensor]],
                           non_quantized_state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Flat name -> CPU tensor map of the exported model (model_quant.py:49-73): block parameters first, in
    block order, a quantised layer's `weight` replaced by its entries; then everything outside the blocks
    except a tied `lm_head.weight`."""
    state: Dict[str, torch.Tensor] = {}
    for block_idx, block in enumerate(model.model.layers):
        prefix = f"model.layers.{block_idx}."
        for k, v in block.state_dict().items():
            layer_name, param_name = k.rsplit(".", 1)
            entry = quantized_state_dict.get(prefix + layer_name)
            if entry is not None and param_name == "weight":
                for kq, vq in entry.items():
                    state[f"{prefix}{layer_name}.{kq}"] = vq.cpu()
            elif prefix + k in non_quantized_state_dict:
                state[prefix + k] = non_quantized_state_dict[prefix + k].cpu()
            else:
                state[prefix + k] = v.cpu()
    state.update(non_quantized_state_dict)
    tied = bool(getattr(model.config, "tie_word_embeddings", False))
    for k, v in model.state_dict().items():
        if not (k.startswith("model.layers") or (k == "lm_head.weight" and tied)):
            state[k] = v.cpu()
    return state


def shard_state_dict(state: Dict[str, torch.Tensor], max_shard_size: int) -> List[Dict[str, torch.Tensor]]:
    """Greedy split in insertion order (model_quant.py:75-96): a shard is closed when the next tensor would
    overflow it; a tensor larger than the limit gets a shard of its own."""
    shards: List[Dict[str, torch.Tensor]] = []
    current: Dict[str, torch.Tensor] = {}
    size = 0
    for k, v in state.items():
        nbytes = v.numel() * v.element_size()
        if size + nbytes > max_shard_size:
            shards.append(current)
            current, size = {}, 0
        if nbytes > max_shard_size:
            shards.append({k: v})
            continue
        current[k] = v
        size += nbytes
    if current:
        shards.append(current)
    return [s for s in shards if s] or [{}]


def shard_file_names(num_shards: int) -> List[str]:
    digits = len(str(max(num_shards, 1)))
    return [f"model-{str(i + 1).zfill(digits)}-of-{str(num_shards).zfill(digits)}.safetensors" for i in range(num_shards)]


def export_quantized_model(model: nn.Module, quantized_state_dict, non_quantized_state_dict, args) -> None:
    """Write `args.save_path`: safetensors shards (at most `args.max_shard_size` bytes each),
    model.safetensors.index.json, config.json with the quantization block, and the generation config when
    the model has one.  `args` carries the fields of the reference's command line: save_path,
    max_shard_size, hadamard_group_size, format, export_quantized_model ("realquant" | "pseudoquant")."""
    from safetensors.torch import save_file

    os.makedirs(args.save_path, exist_ok=True)
    state = build_model_state_dict(model, quantized_state_dict, non_quantized_state_dict)
    shards = shard_state_dict(state, int(getattr(args, "max_shard_size", 5 * 2 ** 30)))
    names = shard_file_names(len(shards))
    weight_map = {}
    for name, shard in zip(names, shards):
        save_file({k: v.contiguous() for k, v in shard.items()}, os.path.join(args.save_path, name))
        for k in shard:
            weight_map[k] = name
    with open(os.path.join(args.save_path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    config = model.config
    config.quantization_config = prepare_quantization_config(
        args.hadamard_group_size, args.format, pseudoquantization=(args.export_quantized_model == "pseudoquant"))
    config.save_pretrained(args.save_path)
    generation_config = getattr(model, "generation_config", None)
    if generation_config is not None:
        generation_config.save_pretrained(args.save_path)


# ---------------------------------------------------------------------------------------------- loader
def read_checkpoint_tensors(path: str) -> Iterable[Tuple[str, torch.Tensor]]:
    """Yield (name, CPU tensor) for every entry of the index, shard by shard."""
    from safetensors import safe_open

    with open(os.path.join(path, "model.safetensors.index.json")) as f:
        weight_map = json.load(f)["weight_map"]
    by_file: Dict[str, List[str]] = {}
    for k, name in weight_map.items():
        by_file.setdefault(name, []).append(k)
    for name, keys in by_file.items():
        with safe_open(os.path.join(path, name), framework="pt", device="cpu") as f:
            for k in keys:
                yield k, f.get_tensor(k)


def fp_quant_config_from_dict(q: dict):
    """FPQuantConfig from a config.json `quantization_config` block."""
    from ..fp_quant.utils.config import FPQuantConfig, FPQuantDtype, validate_config

    if q.get("quant_method") != "fp_quant":
        raise ValueError(f"not an fp_quant checkpoint: quant_method = {q.get('quant_method')!r}")
    cfg = FPQuantConfig(
        forward_dtype=FPQuantDtype(q["forward_dtype"]), forward_method=q["forward_method"],
        backward_dtype=FPQuantDtype(q["backward_dtype"]), store_master_weights=bool(q["store_master_weights"]),
        hadamard_group_size=int(q["hadamard_group_size"]), pseudoquantization=bool(q["pseudoquantization"]),
        modules_to_not_convert=list(q.get("modules_to_not_convert", ["lm_head"])))
    validate_config(cfg)
    return cfg


def load_quantized_checkpoint(model: nn.Module, path: str, device) -> nn.Module:
    """Turn `model` (same architecture as the exported one, any weights) into the exported quantised model:
    linears outside `modules_to_not_convert` become FPQuantLinear holding the checkpoint's codes, scale
    bytes, rotation matrices and tensor scales; all other tensors are copied by name.  Unknown or missing
    names raise."""
    from ..fp_quant.module.linear import FPQuantLinear
    from ..fp_quant.utils.replace import replace_with_fp_quant_linear

    with open(os.path.join(path, "config.json")) as f:
        qdict = json.load(f).get("quantization_config")
    if qdict is None:
        raise ValueError(f"{path}/config.json has no quantization_config")
    cfg = fp_quant_config_from_dict(qdict)
    device = torch.device(device)
    model, replaced = replace_with_fp_quant_linear(model, cfg)
    if not replaced:
        raise ValueError("the model has no linear layer to replace")
    quantised = {name: m for name, m in model.named_modules() if isinstance(m, FPQuantLinear)}
    plain = dict(model.state_dict(keep_vars=True))
    seen = {name: set() for name in quantised}
    for key, tensor in read_checkpoint_tensors(path):
        owner, _, attr = key.rpartition(".")
        mod = quantised.get(owner)
        if mod is not None:
            if attr not in QUANTIZED_KEYS + ("bias",):
                raise KeyError(f"unexpected tensor {key} for a quantised layer")
            value = tensor.to(device)
            if attr in ("qweight", "scales", "dqweight", "bias"):
                setattr(mod, attr, nn.Parameter(value, requires_grad=False))
            else:
                setattr(mod, attr, nn.Buffer(value))
            seen[owner].add(attr)
        elif key in plain:
            plain[key].data = tensor.to(device=device, dtype=plain[key].dtype)
        else:
            raise KeyError(f"checkpoint tensor {key} has no place in the model")
    carried = ("dqweight",) if cfg.pseudoquantization else ("qweight", "scales")
    for name, mod in quantised.items():
        missing = [a for a in carried + QUANTIZED_KEYS[3:] if a not in seen[name]]
        if missing:
            raise KeyError(f"checkpoint lacks {missing} of {name}")
        mod.weight = None                      # the checkpoint carries no master weight
        if cfg.pseudoquantization:
            mod.qweight = mod.scales = None
        else:
            mod.dqweight = None
        if mod.bias is not None and mod.bias.device.type == "meta":
            raise KeyError(f"checkpoint lacks the bias of {name}")
        mod._scales_blocked = None
    tied = bool(getattr(model.config, "tie_word_embeddings", False))
    if tied and hasattr(model, "tie_weights"):
        model.tie_weights()
    return model
