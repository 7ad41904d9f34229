"""An exported directory read by the real downstream caller: transformers' `FPQuantHfQuantizer`
(transformers/quantizers/quantizer_fp_quant.py) with this package standing where `fp_quant` stands.

The quantizer does `from fp_quant import FPQuantLinear, replace_with_fp_quant_linear, FPQuantConfig,
FPQuantDtype`, builds the modules on the meta device, loads `qweight` / `scales` / the two tensor scales
and the Hadamard matrices from the safetensors shards, and calls nothing else: if this package's
`fp_quant` mirror keeps the reference's names, parameters and buffers (inference_lib/src/fp_quant/
module/linear.py:40-140, utils/replace.py), the quantizer works unchanged.

Runs in a child process: the test has to tell transformers that `fp_quant` and `qutlass` are installed
(it looks for their package metadata) before its quantizer modules are imported.
"""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys, types
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/fp-quant_b200"); sys.path.insert(0, {root!r} + "/tests")
import torch
import transformers.utils as tu
import transformers.utils.import_utils as iu
for mod in (tu, iu):
    mod.is_fp_quant_available = lambda: True
    mod.is_qutlass_available = lambda: True
import fpq_b200.fp_quant as fp_quant
sys.modules["fp_quant"] = fp_quant

from transformers import AutoConfig, AutoModelForCausalLM
from transformers.quantizers.auto import AutoHfQuantizer
from test_driver_gpu import _args, _calibration, _tiny_llama
from fpq_b200.fp_quant.module.linear import FPQuantLinear
from fpq_b200.quantization.driver import gptq_quantization
from fpq_b200.quantization.export import export_quantized_model, load_quantized_checkpoint, read_checkpoint_tensors

fmt, path = sys.argv[1], sys.argv[2]
dev = torch.device("cuda:0")
data = _calibration(dev)
model = _tiny_llama(dev)
args = _args(fmt)
quantized, non_quantized = gptq_quantization(model, data, args, dev)
args.save_path, args.max_shard_size = path, 1 << 20
args.format = args.format.value
export_quantized_model(_tiny_llama(dev), quantized, non_quantized, args)

# `from_pretrained(..., device_map=...)` needs the `accelerate` package, which this image does not have: the
# quantizer's own steps are driven here in the order `from_pretrained` runs them.
config = AutoConfig.from_pretrained(path)
hfq = AutoHfQuantizer.from_config(config.quantization_config, pre_quantized=True)
assert type(hfq).__name__ == "FPQuantHfQuantizer"
hfq.validate_environment(device_map={{"": "cuda:0"}})
assert hfq.update_dtype(torch.bfloat16) == torch.bfloat16
hf = AutoModelForCausalLM.from_config(config, dtype=torch.bfloat16)
hfq.preprocess_model(model=hf, dtype=torch.bfloat16)          # replace_with_fp_quant_linear on the meta device
layers = [m for m in hf.modules() if isinstance(m, FPQuantLinear)]
assert len(layers) == 14, len(layers)
converters = hfq.get_weight_conversions()
assert [c.source_patterns for c in converters] == [[".qweight"]]
deserialize = converters[0].operations[0]
loaded = set()
def put(name, value):
    # what transformers' loader does with a converted tensor: replace the parameter or buffer of that name
    module, leaf = hf.get_submodule(name.rpartition(".")[0]), name.rpartition(".")[2]
    if leaf in module._buffers:
        module._buffers[leaf] = value.detach()
    else:
        module._parameters[leaf] = value if isinstance(value, torch.nn.Parameter) else torch.nn.Parameter(value, requires_grad=False)
    loaded.add(name)
for key, tensor in read_checkpoint_tensors(path):
    tensor = tensor.to(dev)
    if key.endswith(".qweight"):
        assert hfq.param_needs_quantization(hf, key)
        prefix = key[: -len(".qweight")]
        for suffix, value in deserialize.convert({{".qweight": [tensor]}}, model=hf, full_layer_name=key, missing_keys=set()).items():
            put(prefix + suffix, value)
    else:
        put(key, tensor)
missing = [k for k in hf.state_dict() if k not in loaded]
assert not missing, missing
hf.tie_weights()
hf = hfq.postprocess_model(hf).to(dev).eval()
for m in layers:
    assert m.qweight.dtype == torch.uint8 and m.qweight.is_cuda and m.scales.numel() > 0
# this package's own loader on a model built the same way (a model cast to bf16 after construction, like
# `_tiny_llama`, carries bf16 rotary frequencies; one constructed in bf16 keeps them in fp32)
own = load_quantized_checkpoint(AutoModelForCausalLM.from_config(config, dtype=torch.bfloat16).to(dev), path, dev).eval()
with torch.no_grad():
    got = torch.cat([hf(x.to(dev)).logits.float() for x in data])
    want = torch.cat([own(x.to(dev)).logits.float() for x in data])
    fake = torch.cat([model(x.to(dev)).logits.float() for x in data])
assert torch.equal(got, want), float((got - want).abs().max())
rel = float(((got - fake) ** 2).mean() / (fake ** 2).mean())
print("REL", rel)
assert rel < 0.1, rel      # real W4A4 against the fake-quantised model of the driver (whose rotary table is bf16)
print("CHILD-OK")
"""


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["nvfp", "mxfp"])
def test_transformers_quantizer_loads_the_exported_directory(fmt, tmp_path):
    """MR-GPTQ of a tiny Llama -> `export_quantized_model` -> the steps of `from_pretrained` through
    `FPQuantHfQuantizer` (environment check, module replacement on the meta device, its weight conversion
    for every `qweight`, post-processing): fourteen real-quantised `FPQuantLinear` modules, logits
    bit-identical to this package's own loader and close to the driver's fake-quantised model."""
    script = tmp_path / "child.py"
    script.write_text(textwrap.dedent(CHILD.format(root=ROOT)))
    out = tmp_path / "export"
    out.mkdir()
    run = subprocess.run([sys.executable, str(script), fmt, str(out)], capture_output=True, text=True, timeout=900)
    assert run.returncode == 0 and "CHILD-OK" in run.stdout, run.stdout[-3000:] + run.stderr[-3000:]
