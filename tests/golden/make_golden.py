"""Generates the golden vectors under tests/golden/ by running the UNMODIFIED reference
(IST-DASLab/FP-Quant, imported from its tree with a stub for the absent
`fast_hadamard_transform` package) on small seeded inputs, and pins the oracle against them.

    python tests/golden/make_golden.py            # needs the reference tree (FPQ_REFERENCE_ROOT)

Outputs (a few hundred KB in total):
  rtn_<fmt>.npz      rotate(128) -> Quantizer.get_quantization_params -> quantize ->
                     pack_fp4_to_uint8 / cast_scales_to_eXmY on a 64 x 512 weight, fp32 mode
  edge_<fmt>.npz     the same chain without rotation on rows of ties / zeros / extremes
  log2_probes.npz    cast_to_eBm0 on maxima a few ulps around powers of two
  gptq_<fmt>.npz     GPTQ.quantize (export path) on a 64 x 256 layer with a correlated Hessian
  mse_<fmt>.npz      Quantizer(observer="mse").get_quantization_params on a rotated 64 x 512 weight
  gptq_actorder_<fmt>.npz   the same layer with quantization_order="activation"
The rotation fed to the reference is the oracle's butterfly (the reference's own FWHT is an
external CUDA kernel whose summation order is unknown), everything downstream is reference code.
"""
import os
import sys

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import fp4, gptq as ogptq, ref_shim  # noqa: E402
from tests import inputs  # noqa: E402


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu()
            v = v.view(torch.int16).numpy() if v.dtype == torch.bfloat16 else v.numpy()
        out[k] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name), **out)
    print("wrote", name, {k: v.shape for k, v in out.items()})


def main():
    ref_shim.load()
    from src.quantization.gptq import GPTQ, get_relative_mse_error
    from src.quantization.quant_ops import cast_scales_to_eXmY, cast_to_eBm0, pack_fp4_to_uint8
    from src.quantization.quantizer import Quantizer

    specs = {"nvfp4": ("nvfp", 16, "e4m3"), "mxfp4": ("mxfp", 32, "e8m0")}

    def ref_chain(y, fmt):
        name, g, prec = specs[fmt]
        q = Quantizer(bits=4, format=name, granularity="group", group_size=g, scale_precision=prec)
        s, z = q.get_quantization_params(y)
        grid = q.quantize(y, s, z)
        return (pack_fp4_to_uint8(grid), cast_scales_to_eXmY(s * q.global_scale, prec), s, q.global_scale.clone(),
                q.dequantize(grid, s, z))

    # ---- RTN round trip
    w = inputs.normal_weight(64, 512, seed=0)
    y = fp4.fwht_butterfly(w, 128)
    for fmt in specs:
        codes, sbytes, s, gs, dq = ref_chain(y, fmt)
        o_codes, o_sb, o_s = fp4.quantize(y, fmt, fp4.nvfp4_global_scale(y.abs().max()) if fmt == "nvfp4" else None)
        assert torch.equal(codes, o_codes) and torch.equal(sbytes, o_sb) and torch.equal(s, o_s), fmt
        save(f"rtn_{fmt}.npz", weight_bf16=w, rotated=y, codes=codes, scale_bytes=sbytes, scales=s,
             global_scale=gs, mse=((dq - y) ** 2).mean())

    # ---- edge rows (no rotation).  NVFP4 uses a fixed tensor scale of 3 so that extremes stay finite.
    x = inputs.edge_case_rows(128)
    for fmt in specs:
        name, g, prec = specs[fmt]
        q = Quantizer(bits=4, format=name, granularity="group", group_size=g, scale_precision=prec)
        if fmt == "nvfp4":
            q.global_scale = torch.tensor([3.0])
            q._track_global_scale = False
        s, z = q.get_quantization_params(x)
        grid = q.quantize(x, s, z)
        codes = pack_fp4_to_uint8(grid)
        sbytes = cast_scales_to_eXmY(s * q.global_scale, prec)
        o_codes, o_sb, o_s = fp4.quantize(x, fmt, torch.tensor([3.0]) if fmt == "nvfp4" else None)
        # NVFP4 groups whose E4M3 scale underflows to zero: the reference then divides by 1 (all
        # codes are zero) and stores e4m3(global_scale) -- not a usable scale, NaN once the
        # global scale exceeds 448 -- where the oracle and the kernels store byte 0.
        underflow = (o_sb == 0) if fmt == "nvfp4" else torch.zeros_like(o_sb, dtype=torch.bool)
        assert torch.equal(codes, o_codes) and torch.equal(s, o_s), fmt
        assert torch.equal(sbytes[~underflow], o_sb[~underflow]), fmt
        assert bool((fp4.unpack_codes(codes).view(x.shape[0], -1, g)[underflow] & 7).eq(0).all())
        save(f"edge_{fmt}.npz", x=x, codes=codes, scale_bytes=sbytes, scales=s, scale_underflow=underflow)

    # ---- log2 rounding artefact of the E8M0 exponent
    probes = []
    for k in range(-126, 127, 3):
        p = torch.tensor(2.0 ** k, dtype=torch.float32)
        v = p.clone()
        for _ in range(70):
            probes.append(v.clone())
            v = torch.nextafter(v, torch.tensor(0.0))
        v = p.clone()
        for _ in range(4):
            v = torch.nextafter(v, torch.tensor(float("inf")))
            probes.append(v.clone())
    m = torch.stack(probes)
    ref_pow = cast_to_eBm0(m, ebits=8, emax=2)            # 2^(floor(log2 m) - 2)
    ref_e = torch.log2(ref_pow).round() + 2
    assert torch.equal(ref_e, fp4.mx_exponent(m.clamp(min=2.0 ** -126)))
    bumped = ref_e != torch.floor(torch.log2(m.double())).float()
    print("log2 probes:", m.numel(), "exponent raised by the fp32 rounding on", int(bumped.sum()))
    save("log2_probes.npz", m=m, exponent=ref_e)

    # ---- GPTQ column loop (export path) with the reference class
    R, C, T = 64, 256, 1024
    wl = inputs.normal_weight(R, C, seed=0, dtype=torch.float32)
    xr = fp4.fwht_butterfly(inputs.correlated_activations(T, C, seed=6), 128)
    wr = fp4.fwht_butterfly(wl, 128)
    H, n = None, 0
    for i in range(4):
        H, n = ogptq.hessian_update(H, n, xr[i * 256:(i + 1) * 256].unsqueeze(0))
    for fmt in specs:
        name, g, prec = specs[fmt]
        layer = nn.Linear(C, R, bias=False)
        layer.weight.data = wr.clone()
        q = Quantizer(bits=4, format=name, granularity="group", group_size=g, scale_precision=prec)
        if fmt == "nvfp4":
            q.get_quantization_params(wr)
            q._track_global_scale = False
        h = GPTQ(layer, q, block_size=128, rel_damp=0.01, export_quantized_model="realquant")
        h.H, h.num_samples = H.clone(), n
        wq, qweight, scales = h.quantize()
        rel = get_relative_mse_error(wq.float(), wr, h.H)
        Hd = ogptq.prepare_hessian(H, wr, 0.01)
        U, ok = ogptq.cholesky_inverse_upper(Hd)
        o_wq, o_codes = ogptq.gptq_column_loop(wr, scales, U, g, 128)
        assert ok and torch.equal(fp4.pack_codes(o_codes), pack_fp4_to_uint8(qweight)) and torch.equal(o_wq, wq), fmt
        assert torch.allclose(Hd, h.H)
        save(f"gptq_{fmt}.npz", weight=wr, hessian=H, damped_hessian=h.H, u=U, scales=scales,
             codes=pack_fp4_to_uint8(qweight), dequantized=wq, relative_mse=rel,
             global_scale=q.global_scale.clone())
    # ---- MSE observer (quantizer.py:117-134) on the rotated weight, one all-zero group included
    ym = fp4.fwht_butterfly(inputs.normal_weight(64, 512, seed=0, dtype=torch.float32), 128)
    ym[3, 32:64] = 0
    for fmt in specs:
        name, g, prec = specs[fmt]
        q = Quantizer(bits=4, format=name, granularity="group", observer="mse", group_size=g, scale_precision=prec)
        sm, _ = q.get_quantization_params(ym)
        raw = fp4.mse_observer_raw_scales(ym, g)
        if fmt == "nvfp4":
            _, so = fp4.nvfp4_scales_from_raw(raw, fp4.nvfp4_global_scale(ym.abs().max()))
        else:
            _, so = fp4.mxfp4_scales_from_raw(raw)
        assert torch.equal(sm, so), fmt
        save(f"mse_{fmt}.npz", rotated=ym, scales=sm, global_scale=q.global_scale.clone())

    # ---- the same layer in activation order (gptq.py:146-155, 190-193)
    for fmt in specs:
        name, g, prec = specs[fmt]
        layer = nn.Linear(C, R, bias=False)
        layer.weight.data = wr.clone()
        q = Quantizer(bits=4, format=name, granularity="group", group_size=g, scale_precision=prec)
        if fmt == "nvfp4":
            q.get_quantization_params(wr)
            q._track_global_scale = False
        h = GPTQ(layer, q, quantization_order="activation", block_size=128, rel_damp=0.01,
                 export_quantized_model="realquant")
        h.H, h.num_samples = H.clone(), n
        wq, qweight, scales = h.quantize()
        rel = get_relative_mse_error(wq.float(), wr, h.H)
        perm, perm_inv, gidx = ogptq.activation_order(H, g)
        Hd = ogptq.prepare_hessian(H[perm][:, perm], wr, 0.01)
        U, ok = ogptq.cholesky_inverse_upper(Hd)
        o_wq, o_codes = ogptq.gptq_column_loop(wr[:, perm], scales, U, g, 128, group_index=gidx)
        o_wq, o_codes = o_wq[:, perm_inv].contiguous(), o_codes[:, perm_inv].contiguous()
        assert ok and torch.equal(fp4.pack_codes(o_codes), pack_fp4_to_uint8(qweight)) and torch.equal(o_wq, wq), fmt
        assert torch.allclose(Hd[perm_inv][:, perm_inv], h.H)
        assert not torch.equal(perm, torch.arange(C))
        save(f"gptq_actorder_{fmt}.npz", weight=wr, hessian=H, damped_hessian=h.H, u_permuted=U, scales=scales,
             perm=perm, codes=pack_fp4_to_uint8(qweight), dequantized=wq, relative_mse=rel,
             global_scale=q.global_scale.clone())
    print("oracle pinned against the reference on every case")


if __name__ == "__main__":
    main()
