"""Model-level drivers (gptq_quantization / rtn_quantization) on a tiny randomly initialised Llama:
the same call a user of the reference's model_quant.py makes (src/quantization/gptq.py:225-470,
src/quantization/rtn.py:17-237), checked for the export format, for consistency between the exported
codes / scales and the weights left in the model, and for GPTQ beating RTN on the calibration data."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import fp4  # noqa: E402  (checker only)


def _tiny_llama(device):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=160, max_position_embeddings=128)
    model = LlamaForCausalLM(cfg).to(device=device, dtype=torch.bfloat16).eval()
    model.config.use_cache = False
    return model


def _args(fmt):
    from fpq_b200.quantization.quant_args import (QuantizationFormat, QuantizationGranularity, QuantizationObserver,
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
        dtype=torch.bfloat16, fuse_global_scale=False, amp=False)


def _calibration(device, n=6, t=96):
    g = torch.Generator().manual_seed(1)
    return [torch.randint(0, 160, (1, t), generator=g) for _ in range(n)]


LINEARS = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
           "mlp.up_proj", "mlp.down_proj"]


@pytest.mark.parametrize("fmt", ["nvfp", "mxfp"])
def test_gptq_quantization_tiny_llama(fmt):
    from fpq_b200.quantization.driver import gptq_quantization, rtn_quantization

    dev = torch.device("cuda:0")
    data = _calibration(dev)
    ref_model = _tiny_llama(dev)
    with torch.no_grad():
        ref_logits = torch.cat([ref_model(x.to(dev)).logits.float() for x in data])

    def run(driver):
        model = _tiny_llama(dev)
        quantized, non_quantized = driver(model, data, _args(fmt), dev)
        with torch.no_grad():
            logits = torch.cat([model(x.to(dev)).logits.float() for x in data])
        return model, quantized, logits

    model, quantized, logits = run(gptq_quantization)
    assert torch.isfinite(logits).all()
    group = 16 if fmt == "nvfp" else 32
    for b in range(2):
        for name in LINEARS:
            key = f"model.layers.{b}.{name}"
            assert key in quantized, key
            e = quantized[key]
            mod = model.model.layers[b].get_submodule(name)
            n, k = mod.out_features, mod.in_features
            assert e["qweight"].dtype == torch.uint8 and tuple(e["qweight"].shape) == (n, k // 2)
            assert tuple(e["scales"].shape) == (n, k // group)
            assert tuple(e["forward_hadamard_matrix"].shape) == (128, 128)
            # exported codes x exported scales reproduce the weight the model now computes with
            sc = fp4.decode_scale_bytes(e["scales"].view(torch.uint8), "nvfp4" if fmt == "nvfp" else "mxfp4")
            sc = sc / e["weight_global_scale"].float().cpu()     # exported scales carry the tensor scale
            deq = fp4.dequantize(fp4.unpack_codes(e["qweight"]), sc, group)
            w = mod.weight.detach().float().cpu()
            assert torch.allclose(deq, w, rtol=2 ** -7, atol=1e-6), (key, (deq - w).abs().max())

    _, _, logits_rtn = run(rtn_quantization)
    err_gptq = ((logits - ref_logits) ** 2).mean() / (ref_logits ** 2).mean()
    err_rtn = ((logits_rtn - ref_logits) ** 2).mean() / (ref_logits ** 2).mean()
    assert err_gptq < 0.5 and err_rtn < 0.5, (err_gptq, err_rtn)
    # error compensation must not be worse than plain rounding on the data it was calibrated on
    assert err_gptq < 1.1 * err_rtn, (err_gptq, err_rtn)


def test_calibration_batching_gives_an_equivalent_model():
    """Several calibration sequences per block call: same Hessians (a sum over sequences) up to summation
    order; the activation tensor scale advances per batch instead of per sequence."""
    from fpq_b200.quantization.driver import gptq_quantization

    dev = torch.device("cuda:0")
    data = _calibration(dev)

    def run(batch):
        model = _tiny_llama(dev)
        args = _args("nvfp")
        args.calibration_batch = batch
        quantized, _ = gptq_quantization(model, data, args, dev)
        with torch.no_grad():
            return quantized, torch.cat([model(x.to(dev)).logits.float() for x in data])

    q1, l1 = run(1)
    q3, l3 = run(3)
    assert sorted(q1) == sorted(q3)
    first = "model.layers.0.self_attn.q_proj"       # identical inputs: only the order of the Hessian sum differs
    a, b = q1[first]["qweight"], q3[first]["qweight"]
    agree = float((((a & 0xF) == (b & 0xF)).sum() + ((a >> 4) == (b >> 4)).sum()) / (2 * a.numel()))
    assert agree > 0.99, agree
    assert float(((l1 - l3) ** 2).mean() / (l1 ** 2).mean()) < 0.05


@pytest.mark.parametrize("fmt", ["nvfp", "mxfp"])
def test_export_round_trip_runs_as_real_w4a4(fmt, tmp_path):
    """gptq_quantization -> export_quantized_model -> load_quantized_checkpoint: every reloaded layer (real
    FP4 codes through the fused quantise + FP4 GEMM) computes, on the input its counterpart in the driver's
    model saw, what that counterpart (dequantised weight, fake-quantised activation, bf16 matmul) computed.
    The two differ where the driver, like the reference's QLinear, rounds the rotated activation to bf16
    before quantising it while the fused kernel quantises the fp32 rotation: a fraction of a percent of the
    activation codes land on the neighbouring grid point (3e-4 .. 1.3e-3 relative MSE per layer on this model)."""
    from fpq_b200.fp_quant.module.linear import FPQuantLinear
    from fpq_b200.quantization.driver import gptq_quantization
    from fpq_b200.quantization.export import export_quantized_model, load_quantized_checkpoint

    dev = torch.device("cuda:0")
    data = _calibration(dev)
    model = _tiny_llama(dev)
    args = _args(fmt)
    quantized, non_quantized = gptq_quantization(model, data, args, dev)
    args.save_path, args.max_shard_size = str(tmp_path), 1 << 20
    args.format = args.format.value
    export_quantized_model(_tiny_llama(dev), quantized, non_quantized, args)   # block weights come from the entries
    loaded = load_quantized_checkpoint(_tiny_llama(dev), str(tmp_path), dev)
    layers = [m for m in loaded.modules() if isinstance(m, FPQuantLinear)]
    assert len(layers) == 14 and all(m.qweight.is_cuda and m.weight is None for m in layers)

    seen = {}
    hooks = [model.model.layers[b].get_submodule(n).register_forward_hook(
        lambda mod, inp, out, key=(b, n): seen.__setitem__(key, (inp[0].detach().clone(), out.detach().clone())))
        for b in range(2) for n in LINEARS]
    with torch.no_grad():
        want = torch.cat([model(x.to(dev)).logits.float() for x in data])
        got = torch.cat([loaded(x.to(dev)).logits.float() for x in data])
    for h in hooks:
        h.remove()
    worst = 0.0
    for (b, n), (x, y) in seen.items():
        with torch.no_grad():
            y2 = loaded.model.layers[b].get_submodule(n)(x)
        worst = max(worst, float(((y2.float() - y.float()) ** 2).mean() / (y.float() ** 2).mean()))
    rel = float(((got - want) ** 2).mean() / (want ** 2).mean())
    print(f"{fmt}: reloaded W4A4 model vs the driver's model: worst layer {worst:.3e}, logits {rel:.3e} (relative MSE)")
    assert worst < 3e-3, worst
    assert rel < 0.08, rel


def test_gptq_quantization_in_activation_order():
    """The driver with quantization_order="activation": every layer permutes and factors its own Hessian;
    the exported codes x scales still reproduce the weights left in the model, and the result is as good
    as the default order on the calibration data."""
    from fpq_b200.quantization.driver import gptq_quantization
    from fpq_b200.quantization.quant_args import QuantizationOrder

    dev = torch.device("cuda:0")
    data = _calibration(dev)
    with torch.no_grad():
        ref_logits = torch.cat([_tiny_llama(dev)(x.to(dev)).logits.float() for x in data])

    def run(order):
        model = _tiny_llama(dev)
        args = _args("nvfp")
        args.quantization_order = order
        quantized, _ = gptq_quantization(model, data, args, dev)
        with torch.no_grad():
            logits = torch.cat([model(x.to(dev)).logits.float() for x in data])
        return model, quantized, float(((logits - ref_logits) ** 2).mean() / (ref_logits ** 2).mean())

    model, quantized, err_act = run(QuantizationOrder.ACTIVATION)
    _, quantized_default, err_default = run(QuantizationOrder.DEFAULT)
    key = "model.layers.0.mlp.down_proj"
    e = quantized[key]
    sc = fp4.decode_scale_bytes(e["scales"].view(torch.uint8), "nvfp4") / e["weight_global_scale"].float().cpu()
    deq = fp4.dequantize(fp4.unpack_codes(e["qweight"]), sc, 16)
    w = model.model.layers[0].mlp.down_proj.weight.detach().float().cpu()
    assert torch.allclose(deq, w, rtol=2 ** -7, atol=1e-6)
    assert not torch.equal(e["qweight"], quantized_default[key]["qweight"])
    print(f"relative logit error: activation order {err_act:.3e}, default order {err_default:.3e}")
    assert err_act < 1.5 * err_default + 1e-3


def test_gptq_quantization_with_the_mse_observer():
    """w_observer = a_observer = "mse": the scale search replaces the min-max scales for weights (static
    GPTQ scales) and activations; the model stays usable and the exported scales differ from min-max's."""
    from fpq_b200.quantization.driver import gptq_quantization
    from fpq_b200.quantization.quant_args import QuantizationObserver

    dev = torch.device("cuda:0")
    data = _calibration(dev)
    with torch.no_grad():
        ref_logits = torch.cat([_tiny_llama(dev)(x.to(dev)).logits.float() for x in data])

    def run(observer):
        model = _tiny_llama(dev)
        args = _args("mxfp")
        args.w_observer = args.a_observer = observer
        quantized, _ = gptq_quantization(model, data, args, dev)
        with torch.no_grad():
            logits = torch.cat([model(x.to(dev)).logits.float() for x in data])
        return quantized, float(((logits - ref_logits) ** 2).mean() / (ref_logits ** 2).mean())

    q_mse, err_mse = run(QuantizationObserver.MSE)
    q_mm, err_mm = run(QuantizationObserver.MINMAX)
    key = "model.layers.0.self_attn.q_proj"
    a, b = q_mse[key]["scales"].view(torch.uint8), q_mm[key]["scales"].view(torch.uint8)
    changed = float((a != b).float().mean())
    print(f"relative logit error: MSE observer {err_mse:.3e}, min-max {err_mm:.3e}; {changed:.3f} of the q_proj scale bytes differ")
    assert changed > 0.01
    assert err_mse < 1.5 * err_mm + 1e-3


# --------------------------------------------------------------------------- against the reference's drivers
GOLDEN = __import__("os").path.join(__import__("os").path.dirname(__import__("os").path.abspath(__file__)), "golden")


def _code_agreement(a, b):
    return float((((a & 0xF) == (b & 0xF)).sum() + ((a >> 4) == (b >> 4)).sum()) / (2 * a.numel()))


@pytest.mark.parametrize("fmt", ["nvfp", "mxfp"])
def test_gptq_driver_matches_the_reference_driver(fmt):
    """`gptq_quantization` against what the reference driver exported for the same tiny model, calibration ids
    and arguments (tests/golden/make_driver_golden.py ran it on the CPU).

    Strict target, driver_gptq_fp32act_<fmt>.npz: the reference with its activation quantiser fed fp32 (the
    arithmetic parity is defined on; the generator's docstring says what was changed and why).  Every weight
    tensor scale and stored scale byte must be identical, every activation tensor scale within 15 % (the
    first block's q/k/v, whose input passed through no quantised layer: identical), every layer's relative MSE
    (the metric GPTQ parity is defined on) within 5 % of the value the reference printed, and the codes must
    agree to >= 99 % for the first block's q/k/v.  Behind the first attention the two runs differ by the
    rounding of bf16 matmuls and softmax on a GPU against a CPU, and on this 256-wide model with 576
    calibration tokens a perturbation of that size moves 2 % (o_proj) to 30 % (down_proj) of the codes while
    leaving the error unchanged to three digits: the fractions are printed and only bounded below by 60 %.
    Informative, driver_gptq_<fmt>.npz: the unmodified reference, whose bf16-fed activation quantiser
    rounds scales and quotients to 8 bits (src/quantization/qlinear.py:46-48 on bf16 tensors).  Scales and
    weight tensor scales are still identical (they depend on the rotated weights only and are computed in
    fp32, src/quantization/gptq.py:119, :142); the codes of layers behind a quantised activation agree to
    66-81 %, which is also what the reference's own two arithmetic modes give against each other."""
    import numpy as np

    from fpq_b200.quantization import driver
    from fpq_b200.quantization.driver import gptq_quantization

    dev = torch.device("cuda:0")
    data = _calibration(dev)
    model = _tiny_llama(dev)
    quantized, _ = gptq_quantization(model, data, _args(fmt), dev)
    with torch.no_grad():
        logits = torch.cat([model(x.to(dev)).logits.float() for x in data]).cpu()
    strict = np.load(f"{GOLDEN}/driver_gptq_fp32act_{fmt}.npz")
    plain = np.load(f"{GOLDEN}/driver_gptq_{fmt}.npz")
    for b in range(2):
        for name in LINEARS:
            e, k = quantized[f"model.layers.{b}.{name}"], f"{b}.{name}"
            first = b == 0 and name in LINEARS[:3]
            for ref in (strict, plain):
                assert torch.equal(e["weight_global_scale"].float().cpu(), torch.from_numpy(ref[k + ".weight_global_scale"])), k
                assert torch.equal(e["scales"].view(torch.uint8).cpu(), torch.from_numpy(ref[k + ".scales"])), k
            ags, ags_ref = float(e["act_global_scale"]), float(strict[k + ".act_global_scale"][0])
            if first:
                assert ags == ags_ref == float(plain[k + ".act_global_scale"][0]), (k, ags, ags_ref)
            else:       # 2688 / max |activation|: an extreme-value statistic of data that already differs in the last bits
                assert ags == pytest.approx(ags_ref, rel=0.15), (k, ags, ags_ref)
            agree = _code_agreement(e["qweight"].cpu(), torch.from_numpy(strict[k + ".qweight"]))
            loose = _code_agreement(e["qweight"].cpu(), torch.from_numpy(plain[k + ".qweight"]))
            print(f"{fmt} {k:22} codes equal to the reference driver's: fp32-fed activation quantiser {agree:.4f}, "
                  f"unmodified (bf16-fed) {loose:.4f}")
            assert agree >= (0.99 if first else 0.60), (k, agree)
            assert loose >= (0.99 if first else 0.60), (k, loose)
            # GPTQ's own parity metric (gptq.py:28-30) per layer, as the reference driver printed it
            mse, mse_ref = driver.last_relative_mse[f"model.layers.{b}.{name}"], float(strict[k + ".relative_mse"])
            print(f"{'':26} relative MSE {mse:.3e}, reference driver {mse_ref:.3e}")
            assert mse == pytest.approx(mse_ref, rel=0.01 if first else 0.05), (k, mse, mse_ref)
    for tag, ref, bound in (("fp32-fed", strict, 0.05), ("unmodified", plain, 0.1)):
        want = torch.from_numpy(ref["logits"].astype(np.float32))
        rel = float(((logits - want) ** 2).mean() / (want ** 2).mean())
        print(f"{fmt}: logits of the quantised model vs the reference driver's ({tag}): {rel:.3e}")
        assert rel < bound


@pytest.mark.parametrize("fmt", ["nvfp", "mxfp"])
def test_rtn_driver_matches_the_reference_driver(fmt):
    """`rtn_quantization` against the reference driver's export (tests/golden/driver_rtn_<fmt>.npz).  The
    weight tensor scales are exact.  The reference's RTN driver feeds bf16 weights to its Quantizer, whose
    scale arithmetic then runs in bf16 (rtn.py:175 on a bf16 tensor: `2 * max / 12` and, for MXFP, `log2`
    rounded to 8 bits, which moves the exponent of about one group in six); this package computes the
    scales in fp32, the mode parity is defined on.  So scale bytes and codes agree on most, not all, groups:
    the fractions are printed and bounded below, and the settled activation tensor scales must agree."""
    import numpy as np

    from fpq_b200.quantization.driver import rtn_quantization

    dev = torch.device("cuda:0")
    data = _calibration(dev)
    model = _tiny_llama(dev)
    quantized, _ = rtn_quantization(model, data, _args(fmt), dev)
    with torch.no_grad():
        logits = torch.cat([model(x.to(dev)).logits.float() for x in data]).cpu()
    ref = np.load(f"{GOLDEN}/driver_rtn_{fmt}.npz")
    for b in range(2):
        for name in LINEARS:
            e, k = quantized[f"model.layers.{b}.{name}"], f"{b}.{name}"
            assert torch.equal(e["weight_global_scale"].float().cpu(), torch.from_numpy(ref[k + ".weight_global_scale"])), k
            ags, ags_ref = float(e["act_global_scale"]), float(ref[k + ".act_global_scale"][0])
            assert ags > 0 and ags != float("inf")
            if b == 0 and name in LINEARS[:3]:
                assert ags == ags_ref, (k, ags, ags_ref)
            else:
                assert ags == pytest.approx(ags_ref, rel=0.15), (k, ags, ags_ref)
            sb, sb_ref = e["scales"].view(torch.uint8).cpu(), torch.from_numpy(ref[k + ".scales"])
            same_scale = float((sb == sb_ref).float().mean())
            agree = _code_agreement(e["qweight"].cpu(), torch.from_numpy(ref[k + ".qweight"]))
            print(f"{fmt} {k:22} scale bytes equal {same_scale:.4f}, codes equal {agree:.4f}")
            assert same_scale >= 0.95, (k, same_scale)
            assert agree >= 0.97, (k, agree)
    want = torch.from_numpy(ref["logits"].astype(np.float32))
    rel = float(((logits - want) ** 2).mean() / (want ** 2).mean())
    print(f"{fmt}: logits of the RTN model vs the reference's {rel:.3e}")
    assert rel < 0.1


def test_rtn_export_settles_the_activation_scales_and_reloads(tmp_path):
    """NVFP4 RTN: the calibration pass (rtn.py:58-75, 152-156) leaves a finite activation tensor scale in
    every exported entry -- for the first block's q/k/v exactly 2688 / max |rotate(input)| over the
    calibration sequences -- `fuse_global_scale` gives q/k/v (and gate/up) one weight tensor scale
    (rtn.py:134-150), and the exported directory reloads and runs as real W4A4."""
    from fpq_b200.fp_quant.module.linear import FPQuantLinear
    from fpq_b200.quantization.driver import rtn_quantization
    from fpq_b200.quantization.export import export_quantized_model, load_quantized_checkpoint

    dev = torch.device("cuda:0")
    data = _calibration(dev)
    model = _tiny_llama(dev)
    fp_model = _tiny_llama(dev)
    amax = 0.0
    with torch.no_grad():
        for x in data:       # input of block 0's q/k/v: the first RMSNorm of the unquantised model
            h = fp_model.model.layers[0].input_layernorm(fp_model.model.embed_tokens(x.to(dev)))
            amax = max(amax, float(fp4.fwht_butterfly(h.cpu(), 128).bfloat16().abs().max()))
    want_ags = fp4.nvfp4_global_scale(torch.tensor(amax))
    args = _args("nvfp")
    args.fuse_global_scale = True
    quantized, non_quantized = rtn_quantization(model, data, args, dev)
    for key, e in quantized.items():
        assert bool(torch.isfinite(e["act_global_scale"]).all()) and float(e["act_global_scale"]) > 0, key
    for name in LINEARS[:3]:
        assert torch.equal(quantized[f"model.layers.0.{name}"]["act_global_scale"].float().cpu(), want_ags)
    for b in range(2):
        for names in (LINEARS[:3], LINEARS[4:6]):
            scales = {float(quantized[f"model.layers.{b}.{n}"]["weight_global_scale"]) for n in names}
            assert len(scales) == 1, (b, names, scales)

    args.save_path, args.max_shard_size = str(tmp_path), 1 << 20
    args.format = args.format.value
    export_quantized_model(_tiny_llama(dev), quantized, non_quantized, args)
    loaded = load_quantized_checkpoint(_tiny_llama(dev), str(tmp_path), dev)
    assert sum(isinstance(m, FPQuantLinear) for m in loaded.modules()) == 14
    with torch.no_grad():
        want = torch.cat([model(x.to(dev)).logits.float() for x in data])
        got = torch.cat([loaded(x.to(dev)).logits.float() for x in data])
    rel = float(((got - want) ** 2).mean() / (want ** 2).mean())
    print(f"reloaded RTN checkpoint as real W4A4 vs the driver's fake-quantised model: {rel:.3e} (relative MSE of the logits)")
    assert torch.isfinite(got).all() and rel < 0.08
