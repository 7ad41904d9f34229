"""`Quantizer` with the interface of src/quantization/quantizer.py (IST-DASLab/FP-Quant),
computing on the GPU through the fused CUDA kernels.

Supported: 4-bit NVFP (group 16, E4M3 scales + fp32 tensor scale) and MXFP (group 32, E8M0
scales), symmetric, group granularity along the last dim, min-max or MSE observer -- the
configurations of the MR-GPTQ path.  Everything else raises NotImplementedError.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _cabi as C
from .. import ops
from .quant_args import QuantizationFormat, QuantizationGranularity, QuantizationObserver, ScalePrecision
from .quant_ops import get_quantization_range


class Quantizer:
    def __init__(self, bits: int, symmetric: bool = True, format: str = "int", granularity: str = "channel",
                 observer: str = "minmax", dim: int = -1, group_size: Optional[int] = None,
                 scale_precision: str = "fp16", scale_min_clip: Optional[float] = None):
        self.format = QuantizationFormat(format)
        self.granularity = QuantizationGranularity(granularity)
        self.observer = QuantizationObserver(observer)
        self.scale_precision = ScalePrecision(scale_precision)
        if self.format in (QuantizationFormat.FP, QuantizationFormat.NVFP, QuantizationFormat.MXFP):
            assert symmetric, "Only symmetric quantization is supported for floating point formats."
        if self.granularity == QuantizationGranularity.GROUP:
            assert group_size is not None, "Group size must be specified when granularity is 'group'."
        else:
            assert group_size is None, "Group size must be None when granularity is not 'group'."
        self.bits, self.symmetric, self.dim = bits, symmetric, dim
        self.group_size, self.scale_min_clip = group_size, scale_min_clip
        self.q_min, self.q_max = get_quantization_range(self.format, bits, symmetric)
        # MXFP quantisation has the fixed implicit tensor scale 3 (quantizer.py:64-65);
        # NVFP starts at +inf and keeps the running minimum while tracking (:145-150).
        first = 3.0 if self.format == QuantizationFormat.MXFP else float("inf")
        self.global_scale = torch.tensor([first], dtype=torch.float32)
        self._track_global_scale = self.scale_precision == ScalePrecision.E4M3
        self._kernel_format = self._resolve_kernel_format()
        # None: the finiteness checks of `get_quantization_params` synchronise and raise at once, like the
        # reference's.  A list: the checks are appended as device booleans ("something is wrong") and the
        # caller raises later with `raise_deferred_checks` -- for drivers that must not stall the host.
        self.deferred_checks = None

    # ------------------------------------------------------------------ helpers
    def _resolve_kernel_format(self) -> str:
        ok = (self.bits == 4 and self.symmetric and self.granularity == QuantizationGranularity.GROUP
              and self.observer in (QuantizationObserver.MINMAX, QuantizationObserver.MSE) and self.dim == -1)
        if ok and self.format == QuantizationFormat.NVFP and self.scale_precision == ScalePrecision.E4M3 \
                and self.group_size == 16:
            return "nvfp4"
        if ok and self.format == QuantizationFormat.MXFP and self.scale_precision == ScalePrecision.E8M0 \
                and self.group_size == 32:
            return "mxfp4"
        raise NotImplementedError(
            "the B200 path implements 4-bit nvfp (group 16, e4m3 scales) and mxfp (group 32, e8m0 scales) "
            f"with the min-max or MSE observer; got format={self.format} group={self.group_size} "
            f"scales={self.scale_precision} observer={self.observer}")

    def _device_global_scale(self, device: torch.device) -> torch.Tensor:
        if self.global_scale.device != device:
            self.global_scale = self.global_scale.to(device)
        return self.global_scale

    # ------------------------------------------------------------------ API
    @torch.no_grad()
    def get_quantization_params(self, x: torch.Tensor, scale_search_iters: int = 100,
                                max_scale_shrink_factor: float = 0.80,
                                error_norm: float = 2.4) -> Tuple[torch.Tensor, torch.Tensor]:
        """Per-group scales (the divisor of the FP4 cast) and zero points (all zero).
        NVFP also folds max|x| into `global_scale` while `_track_global_scale` is set.  The three search
        parameters only matter for the MSE observer (quantizer.py:117-134)."""
        fmt = self._kernel_format
        gs = None
        if fmt == "nvfp4":
            gs = self._device_global_scale(x.device)
            if self._track_global_scale:
                bits = ops.absmax_bits(x, 0)
                status = torch.zeros(1, dtype=torch.int32, device=x.device)
                ops.global_scale_update(bits, gs, status)
                bad = (status != 0) | ~torch.isfinite(gs)
                if self.deferred_checks is not None:
                    self.deferred_checks.append(bad.reshape(()))
                elif bool(bad.item()):
                    raise ValueError(f"Global scale is not finite: {gs}")
        if self.observer == QuantizationObserver.MSE:
            scales = ops.mse_scales(x, fmt, gs, scale_search_iters, max_scale_shrink_factor, error_norm)
        else:
            _, _, scales = ops.quantize(x, fmt, 0, gs, codes=False, scale_bytes=False, scales_f32=True)
        scales = scales.view(*x.shape[:-1], x.shape[-1] // self.group_size).to(x.dtype)
        bad = scales.isnan().any()
        if self.deferred_checks is not None:
            self.deferred_checks.append(bad)
        elif bool(bad.item()):
            raise ValueError("Scales are not finite.")
        return scales, torch.zeros_like(scales)

    def raise_deferred_checks(self) -> None:
        """One synchronisation for all checks collected since `deferred_checks` was set to a list."""
        if self.deferred_checks:
            bad = bool(torch.stack(self.deferred_checks).any().item())
            self.deferred_checks.clear()
            if bad:
                raise ValueError("Scales or global scale are not finite.")

    def _apply(self, x: torch.Tensor, scales: torch.Tensor, kind: int) -> torch.Tensor:
        group = self.group_size
        if group is None:  # one scale per leading index (the column-at-a-time use inside GPTQ)
            if scales.numel() == x.numel():
                return ops.apply_scales(x.reshape(1, -1), scales.reshape(1, -1), 1, kind).view(x.shape)
            group = x.shape[-1]
        return ops.apply_scales(x, scales, group, kind).view(x.shape)

    @torch.no_grad()
    def quantize(self, x: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor] = None) -> torch.Tensor:
        """E2M1 grid values of x / scales, in the dtype of x."""
        return self._apply(x, scales, C.OUT_GRID)

    @torch.no_grad()
    def dequantize(self, q: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor] = None) -> torch.Tensor:
        s = scales.to(q.dtype)
        if self.group_size:
            return (q.reshape(*q.shape[:-1], -1, self.group_size) * s.unsqueeze(-1)).reshape(q.shape)
        return q * s

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Quantise-dequantise in the straight-through form x + (xq - x)."""
        return self._apply(x, scales, C.OUT_DEQUANT_STE)

    # fused paths the drivers use instead of the three calls above ------------------------
    @torch.no_grad()
    def fused_fake_quantize(self, x: torch.Tensor, hadamard_group: int = 0, ste: bool = True) -> torch.Tensor:
        """rotate + get_quantization_params + __call__ in one kernel pass (min-max observer; the MSE observer
        takes the three steps one after the other)."""
        fmt = self._kernel_format
        if self.observer == QuantizationObserver.MSE:
            xr = ops.rotate_hadamard(x, hadamard_group) if hadamard_group else x
            scales, _ = self.get_quantization_params(xr)
            return self._apply(xr, scales.float(), C.OUT_DEQUANT_STE if ste else C.OUT_DEQUANT)
        gs = None
        if fmt == "nvfp4":
            gs = self._device_global_scale(x.device)
            if self._track_global_scale:
                ops.global_scale_update(ops.absmax_bits(x, hadamard_group), gs)
        return ops.fake_quantize(x, fmt, hadamard_group, gs, ste=ste)
