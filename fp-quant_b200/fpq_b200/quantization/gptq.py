"""`GPTQ` with the interface of the class in src/quantization/gptq.py:33-222 (IST-DASLab/FP-Quant);
every numeric step runs in the CUDA library: Hessian accumulation on tensor cores, damped
Cholesky-inverse factor, the column-block quantise / error-propagation loop, relative MSE.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from .quant_args import QuantizationOrder
from .quant_ops import FP4_CODE_VALUES
from .quantizer import Quantizer


def get_relative_mse_error(q: torch.Tensor, w: torch.Tensor, H: torch.Tensor) -> torch.Tensor:
    """mean(((q - w) H) * (q - w)) / (mean((w H) * w) + 1e-6)  (gptq.py:28-30), a device scalar."""
    return ops.relative_mse(q.float().contiguous(), w.float().contiguous(), H).reshape(())


class GPTQ:
    def __init__(self, layer: nn.Module, quantizer: Quantizer, quantization_order: str = "default",
                 block_size: int = 128, rel_damp: float = 1e-2, export_quantized_model: str = ""):
        w = getattr(layer, "weight", None)
        assert isinstance(w, torch.Tensor) and w.dim() == 2, "the B200 path quantises layers with a 2-D weight"
        if block_size != 128:
            raise NotImplementedError("the column-block kernel is built for block_size = 128")
        self.layer = layer
        self.W = layer.weight
        self.d_row, self.d_col = layer.weight.shape
        self.quantizer = quantizer
        self.quantization_order = QuantizationOrder(quantization_order)
        self.block_size, self.rel_damp = block_size, rel_damp
        self.W_device, self.W_dtype, self.W_shape = self.W.device, self.W.dtype, self.W.shape
        self.H: Optional[torch.Tensor] = None
        self.num_samples = 0
        self.export_quantized_model = export_quantized_model
        self.packed_codes: Optional[torch.Tensor] = None     # uint8 [rows, cols/2] of the last `step`
        self.used_identity_fallback = False
        self.defer_host_syncs = False     # True: nothing in quantize() waits for the device (multi-GPU driver's critical path)
        self.use_cuda_graphs = False      # True: the Cholesky chain and the column loop are replayed from CUDA graphs (drivers)
        self.fallback_status: Optional[torch.Tensor] = None

    @torch.no_grad()
    def update(self, input: torch.Tensor) -> None:
        """Fold a batch of layer inputs into the running mean H = (2/N) sum X^T X, N counted in
        `input.shape[0]` units exactly as the reference does (gptq.py:69-102).  The mean's factors
        go onto H (alpha, beta of the kernel) instead of rescaling the input."""
        batch_size = input.shape[0]
        if self.H is None:
            self.H = torch.zeros((self.d_col, self.d_col), device=input.device, dtype=torch.float32)
        x = input.reshape(-1, input.shape[-1])
        beta = self.num_samples / (self.num_samples + batch_size)
        alpha = 2.0 / (self.num_samples + batch_size)
        ops.hessian_accumulate(self.H, x, alpha=alpha, beta=beta)
        self.num_samples += batch_size

    def reset(self) -> None:
        self.W = self.layer.weight
        self.H = None
        self.num_samples = 0
        self.packed_codes = None

    @torch.no_grad()
    def quantization_pre_step(self) -> None:
        assert self.H is not None, "One has to process at least one sample of calibration data to run pruning"
        self.W = self.W.clone().float()
        self.pre_step_completed = True

    @torch.no_grad()
    def step(self, U: Optional[torch.Tensor] = None, shard_rows: bool = False, process_group=None,
             want_grid_values: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor]:
        """Returns (dequantised weight in the layer dtype, E2M1 grid values or None, fp32 group scales).
        `self.H` is left damped, as in the reference, where the caller reuses it for the relative MSE.

        Two additions for multi-GPU drivers (the reference is single-GPU): `U` hands in a factor that was
        computed elsewhere (then `self.H` must already be damped); with `shard_rows` (a collective call:
        every rank of `process_group` must make it) the rows of the weight -- independent given U -- are
        split over the ranks and the results gathered, so every rank returns the full tensors."""
        from .. import dist as fdist

        group = self.quantizer.group_size
        scales, _ = self.quantizer.get_quantization_params(self.W)        # static scales, gptq.py:142
        act_order = self.quantization_order == QuantizationOrder.ACTIVATION
        group_index = perm_inv = None
        W = self.W
        if act_order:
            # gptq.py:146-155: columns by falling diag(H); the Hessian is permuted before it is damped and
            # inverted (the dead-column test still reads the unpermuted weight, as in the reference), and a
            # permuted column keeps the static scale of the group it came from
            if U is not None:
                raise ValueError("activation order derives the factor from the permuted Hessian: do not pass U")
            perm = torch.argsort(self.H.diag(), descending=True)
            perm_inv = torch.argsort(perm)
            group_index = (perm // group).to(torch.int32).contiguous()
            self.H = self.H[perm][:, perm].contiguous()
            W = self.W[:, perm].contiguous()
        if U is None:
            U = self._get_hessian_inverse()
        rank, ws = fdist.world(process_group)
        sc = scales.float().contiguous()
        if shard_rows and ws > 1 and self.d_row >= 128 * ws:
            lo, hi = fdist.shard_bounds(self.d_row, ws, rank, multiple=128)
            w_loc = W[lo:hi].clone()
            codes_loc = ops.gptq_quantize(w_loc, sc[lo:hi].contiguous(), U, group, want_codes=True, group_index=group_index)
            w = fdist.allgather_rows(w_loc, self.d_row, 128, process_group)
            self.packed_codes = fdist.allgather_rows(codes_loc, self.d_row, 128, process_group)
        else:
            w = W.clone()
            if self.use_cuda_graphs:
                self.packed_codes = ops.gptq_quantize_graphed(w, sc, U, group, group_index=group_index)
            else:
                self.packed_codes = ops.gptq_quantize(w, sc, U, group, want_codes=True, group_index=group_index)
        if act_order:
            # gptq.py:190-193: back to the original column order (weights, codes, Hessian)
            w = w[:, perm_inv].contiguous()
            nib = torch.stack((self.packed_codes & 0xF, self.packed_codes >> 4), dim=-1).reshape(self.d_row, self.d_col)
            nib = nib[:, perm_inv]
            self.packed_codes = (nib[:, 0::2] | (nib[:, 1::2] << 4)).contiguous()
            self.H = self.H[perm_inv][:, perm_inv].contiguous()
        qweight = None
        if self.export_quantized_model and want_grid_values:
            # grid values of both nibbles of a byte from one 256-entry table
            lut = torch.tensor(FP4_CODE_VALUES, dtype=self.W_dtype, device=w.device)
            byte = torch.arange(256, device=w.device)
            lut2 = torch.stack((lut[byte & 0xF], lut[byte >> 4]), dim=-1)
            qweight = lut2[self.packed_codes.int()].reshape(self.W.shape)
        return w.to(self.W_dtype), qweight, scales

    @torch.no_grad()
    def prepare_hessian(self) -> None:
        """Dead-column fix and damping of `self.H` in place (first half of gptq.py:200-211)."""
        ops.hessian_prepare(self.H, self.W, self.rel_damp)

    @torch.no_grad()
    def _get_hessian_inverse(self, prepared: bool = False) -> torch.Tensor:
        if not prepared:
            self.prepare_hessian()
        U, status = (ops.cholesky_inverse_upper_graphed if self.use_cuda_graphs else ops.cholesky_inverse_upper)(self.H)
        if self.defer_host_syncs:
            # the reference's `except:` branch (gptq.py:216-217) without reading the status on the host:
            # U becomes the identity on the device when the factorisation failed
            failed = (status != 0).to(torch.float32)
            U.mul_(1.0 - failed)
            U.diagonal().add_(failed)
            self.fallback_status = status
            return U
        self.used_identity_fallback = bool(status.item())
        if self.used_identity_fallback:      # the reference's `except:` branch (gptq.py:216-217)
            U = torch.eye(self.d_col, device=self.H.device, dtype=torch.float32)
        return U

    def quantize(self, U: Optional[torch.Tensor] = None, shard_rows: bool = False, process_group=None,
                 want_grid_values: bool = True):
        self.quantization_pre_step()
        return self.step(U, shard_rows, process_group, want_grid_values)
