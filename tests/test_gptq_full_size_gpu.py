"""MR-GPTQ of one linear at the sizes of a Llama-3.1-8B block, against the oracle.

Two layers: the MLP up-projection (14336 x 4096: the single-layer benchmark shape) and the down-projection
(4096 x 14336: the widest Hessian, 28 outer blocks of the two-level Cholesky and 112 column blocks).  NVFP4,
Hadamard 128, rel_damp 0.01, block 128, default order (src/quantization/gptq.py:126-218 of
IST-DASLab/FP-Quant).  The calibration input is the rank-64-mixed one of tests/inputs.py, so the Hessian
is far from diagonal and a wrong error-propagation step cannot hide behind "GPTQ ~ RTN".

What is compared with what:
  * Hessian: the tensor-core accumulation against fp64 on a column slab (1e-5 relative).
  * U = chol(H^-1, upper): the defining property max |U^T U H - I| on a column slab, evaluated in fp64, must
    be no worse than 5x that of the reference's own chain (torch.linalg.cholesky -> cholesky_inverse ->
    cholesky(upper), gptq.py:212-215, run here in fp32 by torch on the same device).
  * column loop: the rows of a weight are independent given U and the static scales, so the CPU oracle
    re-runs a fixed sample of rows with the device's U and scales: >= 99 % of the codes must agree, the
    relative MSE (gptq.py:28-30) of those rows must be within 1 % of the oracle's and below round-to-nearest.
  * the device's relative-MSE metric against an fp64 evaluation of the same formula on the full layer.
"""
import pytest
import torch

from oracle import fp4, gptq as ogptq
from tests import inputs

pytestmark = pytest.mark.gpu


def _relative_mse_fp64(wq, w, H):
    """gptq.py:28-30 in fp64 (the formula of oracle/gptq.py::relative_mse, on either device)."""
    d = (wq - w).double()
    Hd, wd = H.double(), w.double()
    return float(((d @ Hd) * d).mean() / (((wd @ Hd) * wd).mean() + 1e-6))


@pytest.mark.parametrize("rows,cols,tokens,sample", [(14336, 4096, 8192, 1024), (4096, 14336, 16384, 256)])
def test_mr_gptq_layer_at_llama8b_size(cuda_device, rows, cols, tokens, sample):
    from fpq_b200 import ops

    dev = cuda_device
    group, hg = 16, 128
    w_bf16 = inputs.normal_weight(rows, cols, seed=0)
    x = inputs.correlated_activations(tokens, cols, seed=6)

    # rotated weight and calibration input (rotation parity has its own bit-exact tests)
    w = ops.rotate_hadamard(w_bf16.to(dev), hg, out_dtype=torch.float32)
    xr = ops.rotate_hadamard(x.to(dev), hg)                                   # bf16, as the drivers feed it
    n_seq = tokens // 2048
    H = torch.zeros(cols, cols, device=dev)
    ops.hessian_accumulate(H, xr, alpha=2.0 / n_seq, beta=0.0)
    slab = torch.arange(cols - 256, cols, device=dev)
    want_H = (xr.double().t() @ xr[:, slab].double()) * (2.0 / n_seq)
    assert ((H[:, slab].double() - want_H).norm() / want_H.norm()).item() < 1e-5
    del want_H

    # static scales of the unmodified rotated weight (gptq.py:142), NVFP4 with its tensor scale
    gs = torch.full((1,), float("inf"), device=dev)
    ops.global_scale_update(ops.absmax_bits(w, 0), gs)
    _, _, scales = ops.quantize(w, "nvfp4", 0, gs, codes=False, scale_bytes=False, scales_f32=True)
    rows_s = torch.randperm(rows, generator=torch.Generator().manual_seed(5))[:sample].sort().values
    w_s = w[rows_s.to(dev)].cpu()
    want_codes, _, want_scales = fp4.quantize(w_s, "nvfp4", gs.cpu())
    assert torch.equal(scales[rows_s.to(dev)].cpu(), want_scales)

    # damped Hessian and its inverse factor
    ops.hessian_prepare(H, w, 0.01)
    U, status = ops.cholesky_inverse_upper(H)
    ops.check_device_errors(dev)
    assert int(status.item()) == 0
    assert torch.equal(U, torch.triu(U))

    def residual(factor):
        f = factor.double()
        r = f.t() @ (f @ H[:, slab].double())
        r[slab, torch.arange(slab.numel(), device=dev)] -= 1.0
        return r.abs().max().item()

    U_ref = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True)
    res, res_ref = residual(U), residual(U_ref)
    rel_u = ((U - U_ref).norm() / U_ref.norm()).item()
    print(f"d={cols}: max|U^T U H - I| {res:.3e} (reference chain {res_ref:.3e}); |U - U_ref|/|U_ref| {rel_u:.3e}")
    assert res <= max(5 * res_ref, 1e-3), (res, res_ref)
    assert rel_u < 5e-3
    del U_ref

    # column loop on the whole layer, checked on the sampled rows with the device's U and scales
    Wq = w.clone()
    codes = ops.gptq_quantize(Wq, scales, U, group)
    ops.check_device_errors(dev)
    U_cpu, H_cpu = U.cpu(), H.cpu().double()
    wq_ref, codes_ref = ogptq.gptq_column_loop(w_s, want_scales, U_cpu, group, 128)
    got_codes = fp4.unpack_codes(codes[rows_s.to(dev)].cpu())
    agree = (got_codes == codes_ref).float().mean().item()
    wq_s = Wq[rows_s.to(dev)].cpu()
    assert torch.equal(wq_s, fp4.dequantize(got_codes, want_scales, group))       # output = grid(code) * scale
    rel, rel_ref = _relative_mse_fp64(wq_s, w_s, H_cpu), _relative_mse_fp64(wq_ref, w_s, H_cpu)
    rtn = fp4.dequantize(fp4.unpack_codes(want_codes), want_scales, group)
    rel_rtn = _relative_mse_fp64(rtn, w_s, H_cpu)
    print(f"{rows}x{cols}: code agreement {agree:.5f} on {sample} rows; relative MSE device {rel:.4e} "
          f"oracle {rel_ref:.4e} round-to-nearest {rel_rtn:.4e}")
    assert agree >= 0.99
    assert abs(rel - rel_ref) <= 0.01 * rel_ref
    assert rel < rel_rtn

    # the metric kernel on the full layer against fp64
    # (tensor-core form <H, D^T D> from a two-term bf16 split of D = Wq - W: ~1e-5 on the Gram matrix, but GPTQ
    # shapes D so that D H D^T is some thirty times smaller than |D|^2 |H| would allow, and the cancellation
    # magnifies that error; measured 1.5e-3 on this layer)
    got_metric = ops.relative_mse(Wq, w, H).item()
    want_metric = _relative_mse_fp64(Wq, w, H)
    print(f"relative-MSE kernel {got_metric:.5e}, fp64 {want_metric:.5e}")
    assert got_metric == pytest.approx(want_metric, rel=5e-3)
    assert want_metric == pytest.approx(rel, rel=0.1)          # the row sample is representative
