"""Checkpoint export (src/quantization/qconfig.py:3-20, model_quant.py:41-119 of IST-DASLab/FP-Quant): the
files this package writes are compared, name by name, with the listing of what the unmodified reference
exporter wrote for the same tiny model and per-layer entries (tests/golden/export_listing.json, made by
tests/golden/make_export_listing.py), and read back through the loader."""
import json
import os

import pytest
import torch

from tests import export_case

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "export_listing.json")


def _listing(path):
    from safetensors import safe_open

    with open(os.path.join(path, "model.safetensors.index.json")) as f:
        index = json.load(f)
    tensors = {}
    for name in sorted(set(index["weight_map"].values())):
        with safe_open(os.path.join(path, name), framework="pt", device="cpu") as f:
            for k in f.keys():
                t = f.get_tensor(k)
                tensors[k] = [str(t.dtype), list(t.shape)]
    with open(os.path.join(path, "config.json")) as f:
        qc = json.load(f)["quantization_config"]
    return {"files": sorted(n for n in os.listdir(path) if n.endswith(".safetensors")),
            "index_metadata": index["metadata"], "weight_map": index["weight_map"], "tensors": tensors,
            "quantization_config": qc}


@pytest.mark.parametrize("case", export_case.CASES)
def test_export_matches_the_reference_listing(case, tmp_path):
    from fpq_b200.quantization.export import export_quantized_model

    with open(GOLDEN) as f:
        want = json.load(f)[case]
    model, quantized, non_quantized, args = export_case.build(case)
    args.save_path = str(tmp_path)
    export_quantized_model(model, quantized, non_quantized, args)
    got = _listing(str(tmp_path))
    assert got["files"] == want["files"]
    assert got["quantization_config"] == want["quantization_config"]
    assert got["tensors"] == want["tensors"]
    assert got["weight_map"] == want["weight_map"]           # same greedy sharding, shard by shard
    assert got["index_metadata"] == want["index_metadata"]
    tied = case.endswith("tied")
    assert ("lm_head.weight" in got["tensors"]) == (not tied)
    assert not any(k.endswith("q_proj.weight") for k in got["tensors"])
    assert os.path.exists(tmp_path / "generation_config.json")


def test_quantization_config_fields():
    from fpq_b200.quantization.qconfig import prepare_quantization_config
    from fpq_b200.quantization.quant_args import QuantizationFormat

    q = prepare_quantization_config(32, "mxfp")
    assert q == {"forward_dtype": "mxfp4", "backward_dtype": "bf16", "forward_method": "abs_max", "hadamard_group_size": 32,
                 "modules_to_not_convert": ["lm_head"], "quant_method": "fp_quant", "store_master_weights": False,
                 "pseudoquantization": False}
    assert prepare_quantization_config(128, QuantizationFormat.NVFP, True)["forward_dtype"] == "nvfp4"
    with pytest.raises(ValueError):
        prepare_quantization_config(32, "int")


def test_sharding_rule():
    from fpq_b200.quantization.export import shard_file_names, shard_state_dict

    t = lambda n: torch.zeros(n, dtype=torch.uint8)
    shards = shard_state_dict({"a": t(40), "b": t(40), "c": t(40), "big": t(500), "d": t(10)}, 100)
    assert [list(s) for s in shards] == [["a", "b"], ["c"], ["big"], ["d"]]
    assert shard_file_names(3) == ["model-1-of-3.safetensors", "model-2-of-3.safetensors", "model-3-of-3.safetensors"]
    assert shard_file_names(12)[0] == "model-01-of-12.safetensors"


@pytest.mark.parametrize("case", export_case.CASES)
def test_loader_reads_back_what_was_exported(case, tmp_path):
    from fpq_b200.fp_quant.module.linear import FPQuantLinear
    from fpq_b200.quantization.export import export_quantized_model, load_quantized_checkpoint

    model, quantized, non_quantized, args = export_case.build(case)
    args.save_path = str(tmp_path)
    export_quantized_model(model, quantized, non_quantized, args)
    fresh = export_case.tiny_llama(tie=case.endswith("tied"))
    with torch.no_grad():
        for p in fresh.parameters():
            p.zero_()
    loaded = load_quantized_checkpoint(fresh, str(tmp_path), "cpu")
    real = case.startswith("realquant")
    n = 0
    for key, entry in quantized.items():
        mod = loaded.get_submodule(key)
        assert isinstance(mod, FPQuantLinear) and mod.weight is None
        for k, v in entry.items():
            got = getattr(mod, k)
            assert got.dtype == v.dtype and torch.equal(got.view(torch.uint8) if v.dtype.itemsize == 1 else got,
                                                        v.view(torch.uint8) if v.dtype.itemsize == 1 else v), (key, k)
        assert (mod.dqweight is None) == real and (mod.qweight is None) == (not real)
        n += 1
    assert n == 14
    assert not isinstance(loaded.lm_head, FPQuantLinear)
    assert torch.equal(loaded.model.embed_tokens.weight, model.model.embed_tokens.weight)
    assert torch.equal(loaded.model.layers[1].input_layernorm.weight, non_quantized["model.layers.1.input_layernorm.weight"])
    assert torch.equal(loaded.model.layers[0].input_layernorm.weight, model.model.layers[0].input_layernorm.weight)
    if case.endswith("tied"):
        assert loaded.lm_head.weight.data_ptr() == loaded.model.embed_tokens.weight.data_ptr()
    assert not any(p.device.type == "meta" for p in loaded.parameters())
    assert not any(b.device.type == "meta" for b in loaded.buffers())


def test_loader_rejects_incomplete_checkpoints(tmp_path):
    from fpq_b200.quantization.export import export_quantized_model, load_quantized_checkpoint

    model, quantized, non_quantized, args = export_case.build("realquant_nvfp")
    del quantized["model.layers.0.mlp.up_proj"]["scales"]
    args.save_path = str(tmp_path)
    export_quantized_model(model, quantized, non_quantized, args)
    with pytest.raises(KeyError, match="scales"):
        load_quantized_checkpoint(export_case.tiny_llama(False), str(tmp_path), "cpu")
