"""Golden outputs of the reference's model-level drivers on a tiny random Llama, for the driver parity tests.

    python tests/golden/make_driver_golden.py        # needs the reference tree (FPQ_REFERENCE_ROOT)

Runs the UNMODIFIED `gptq_quantization` (src/quantization/gptq.py:225-470) and `rtn_quantization`
(src/quantization/rtn.py:17-237) of IST-DASLab/FP-Quant on the CPU, on the model, calibration ids and
arguments of tests/test_driver_gpu.py, and writes per layer what they export (packed codes, scale bytes,
weight and activation tensor scales) plus the logits of the model they leave behind:
    driver_gptq_<fmt>.npz, driver_rtn_<fmt>.npz      fmt in nvfp, mxfp
and, as the strict target of the GPTQ driver test,
    driver_gptq_fp32act_<fmt>.npz
from the same run with ONE change to the reference: `QLinear.forward` (src/quantization/qlinear.py:46-48)
hands its activation quantiser `x.float()` instead of the bf16 tensor.  The reference's Quantizer
computes in the dtype it is given; parity with this package is defined on its fp32 arithmetic, and the
choice matters here: GPTQ codes of every layer behind a quantised activation agree only to 66-81 %
between the reference's own bf16-fed and fp32-fed runs (the codes of the first block's q/k/v, whose
input is not quantised data, agree to 100 %).

Three things outside the reference's Python are stood in for, because they need a CUDA device or an absent
package; none of them is reference code:
  * `fast_hadamard_transform` (external CUDA package): the oracle's fp32 butterfly, so that the rotation
    is the one this repository defines parity on (oracle/fp4.py::fwht_butterfly);
  * the Triton `accumulate_hessian` kernel: `H.addmm_(X^T, X)` in fp32, the restatement the oracle uses
    (oracle/gptq.py::hessian_update);
  * `torch.accelerator.current_accelerator()`, which is None on a CPU-only host: an object whose `.type`
    is "cpu" (the drivers only read it to open a disabled autocast context).
"""
import contextlib
import io
import os
import re
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import fp4, ref_shim  # noqa: E402

LINEARS = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
           "mlp.up_proj", "mlp.down_proj"]


def install_stand_ins():
    stub = types.ModuleType("fast_hadamard_transform")

    def butterfly(x, scale=1.0):
        # the oracle's butterfly with the caller's scale as the one final fp32 multiply
        g = x.shape[-1]
        y = x.detach().to(torch.float32).reshape(-1, g).clone()
        d = 1
        while d < g:
            v = y.view(-1, g // (2 * d), 2, d)
            a, b = v[:, :, 0, :].clone(), v[:, :, 1, :].clone()
            v[:, :, 0, :], v[:, :, 1, :] = a + b, a - b
            d *= 2
        return (y * torch.tensor(scale, dtype=torch.float32)).reshape(x.shape).to(x.dtype)

    stub.hadamard_transform = butterfly
    sys.modules["fast_hadamard_transform"] = stub
    ref_shim.load()
    import src.quantization.gptq as ref_gptq

    ref_gptq.accumulate_hessian = lambda H, x: H.addmm_(x.t(), x)

    class _Cpu:
        type = "cpu"

    torch.accelerator.current_accelerator = lambda *a, **k: _Cpu()
    # the stand-in rotation is the oracle's
    probe = torch.randn(5, 256, generator=torch.Generator().manual_seed(0))
    assert torch.equal(butterfly(probe.reshape(-1, 128), 128 ** -0.5).reshape(5, 256), fp4.fwht_butterfly(probe, 128))


def tiny_llama():
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=160, max_position_embeddings=128)
    model = LlamaForCausalLM(cfg).to(dtype=torch.bfloat16).eval()
    model.config.use_cache = False
    return model


def calibration(n=6, t=96):
    g = torch.Generator().manual_seed(1)
    return [torch.randint(0, 160, (1, t), generator=g) for _ in range(n)]


def reference_args(fmt):
    from src.quantization.quant_args import (QuantizationFormat, QuantizationGranularity, QuantizationObserver,
                                             QuantizationOrder, ScalePrecision)
    nv = fmt == "nvfp"
    return types.SimpleNamespace(
        format=QuantizationFormat.NVFP if nv else QuantizationFormat.MXFP,
        w_bits=4, a_bits=4, w_granularity=QuantizationGranularity.GROUP, a_granularity=QuantizationGranularity.GROUP,
        w_observer=QuantizationObserver.MINMAX, a_observer=QuantizationObserver.MINMAX,
        w_group_size=16 if nv else 32, a_group_size=16 if nv else 32,
        scale_precision=ScalePrecision.E4M3 if nv else ScalePrecision.E8M0,
        transform_class="hadamard", hadamard_group_size=128, cpu_offload_activations=False, cpu_offload_modules=False,
        quantization_order=QuantizationOrder.DEFAULT, rel_damp=0.01, export_quantized_model="realquant",
        dtype=torch.bfloat16, fuse_global_scale=False, amp=False, log_wandb=False)


def feed_activation_quantiser_fp32():
    """QLinear.forward with the activation quantiser computing in fp32 (everything else as qlinear.py:26-51)."""
    import torch.nn.functional as F

    import src.quantization.qlinear as ref_qlinear

    def forward(self, x, in_transform=None, out_transform=None):
        weight, bias = self.weight, self.bias
        if self._train_mode:
            if in_transform:
                weight = in_transform(weight, inv_t=True, dim=-1)
            assert out_transform is None
            if self.weight_quantizer is not None:
                w_scales, w_zeros = self.weight_quantizer.get_quantization_params(weight)
                weight = self.weight_quantizer(weight, w_scales, w_zeros)
        if self.act_quantizer is not None:
            xf = x.float()
            a_scales, a_zeros = self.act_quantizer.get_quantization_params(xf)
            x = self.act_quantizer(xf, a_scales, a_zeros).to(x.dtype)
        return F.linear(x, weight, bias)

    ref_qlinear.QLinear.forward = forward


def main():
    install_stand_ins()
    from src.quantization.gptq import gptq_quantization
    from src.quantization.rtn import rtn_quantization

    data = calibration()
    for tag, driver in (("gptq", gptq_quantization), ("rtn", rtn_quantization), ("gptq_fp32act", gptq_quantization)):
        if tag == "gptq_fp32act":
            feed_activation_quantiser_fp32()
        for fmt in ("nvfp", "mxfp"):
            model = tiny_llama()
            printed = io.StringIO()
            with contextlib.redirect_stdout(printed):
                quantized, _ = driver(model, data, reference_args(fmt), torch.device("cpu"))
            with torch.no_grad():
                logits = torch.cat([model(x).logits.float() for x in data])
            out = {"logits": logits.numpy().astype(np.float16)}
            # the GPTQ driver prints every layer's relative MSE (gptq.py:414-415), in layer order, three digits
            mse = [float(v) for v in re.findall(r"Relative MSE error: ([0-9.e+-]+)", printed.getvalue())]
            if mse:
                assert len(mse) == 14
                order = [n for _, n in re.findall(r"(\[)(\S+)\s*\]: Relative MSE", printed.getvalue())]
                for i, (name, v) in enumerate(zip(order, mse)):
                    out[f"{i // 7}.{name}.relative_mse"] = np.float32(v)
            for b in range(2):
                for name in LINEARS:
                    e = quantized[f"model.layers.{b}.{name}"]
                    k = f"{b}.{name}"
                    out[k + ".qweight"] = e["qweight"].numpy()
                    out[k + ".scales"] = e["scales"].view(torch.uint8).numpy()
                    out[k + ".weight_global_scale"] = e["weight_global_scale"].float().numpy()
                    out[k + ".act_global_scale"] = e["act_global_scale"].float().numpy()
            path = os.path.join(HERE, f"driver_{tag}_{fmt}.npz")
            np.savez_compressed(path, **out)
            print("wrote", os.path.basename(path), os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
