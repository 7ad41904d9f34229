"""Generates tests/golden/export_listing.json by running the UNMODIFIED reference exporter
(`export_quantized_model`, model_quant.py:41-119 of IST-DASLab/FP-Quant, imported from its tree with
stubs for the absent `lm_eval` / `fast_hadamard_transform` packages) on the tiny model and the
synthetic per-layer entries of tests/export_case.py, and listing what it wrote: shard file names, the
index (tensor name -> shard), every tensor's dtype and shape, and config.json's quantization block.

    python tests/golden/make_export_listing.py        # needs the reference tree (FPQ_REFERENCE_ROOT)
"""
import json
import os
import sys
import tempfile
import types

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import ref_shim  # noqa: E402
from tests import export_case  # noqa: E402


def listing(path):
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


def main():
    ref_shim.load()
    for name in ("lm_eval", "lm_eval.utils", "lm_eval.models", "lm_eval.models.huggingface"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["lm_eval.utils"].make_table = None
    sys.modules["lm_eval.models.huggingface"].HFLM = None
    import model_quant  # the reference's command-line module

    out = {}
    for case in export_case.CASES:
        model, quantized, non_quantized, args = export_case.build(case)
        with tempfile.TemporaryDirectory() as tmp:
            args.save_path = tmp
            model_quant.export_quantized_model(model, quantized, non_quantized, args)
            out[case] = listing(tmp)
    with open(os.path.join(HERE, "export_listing.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote export_listing.json", {k: len(v["tensors"]) for k, v in out.items()})


if __name__ == "__main__":
    main()
