"""`FPQuantLinear` with the constructor, buffers, `pre_forward` and `forward` dispatch of
inference_lib/src/fp_quant/module/linear.py (IST-DASLab/FP-Quant), on the fpq_b200 kernels.

Differences a caller can observe: the weight scales are additionally cached in the swizzled
layout the matmul reads (`_scales_blocked`, rebuilt when `scales` changes).
"""
from __future__ import annotations

import torch
from torch import nn

from ... import ops
from ...rotation import sylvester
from ..utils.config import FPQuantConfig, FPQuantDtype, validate_config
from .linear_fns import (FPQuant4x4MasterFn, FPQuant4x8MasterFn, FPQuant4x8NoMasterFn, FPQuant4x16MasterFn, FPQuant4x16NoMasterFn,
                         _linear_forward, forward_gemm_blocked, forward_quantize, gemm_alpha)
from .pseudoquant_linear_fns import PseudoQuant4x16MasterFn, PseudoQuant4x16NoMasterFn, forward_pseudoquantize
from .qutlass_ops import (HAS_QUTLASS, fused_silu_mul_quantize_blocked_op,  # noqa: F401  (HAS_QUTLASS: API compatibility)
                          swizzle_scales_op)


def get_hadamard_matrix(group_size: int, dtype: torch.dtype, device: torch.device):
    return (sylvester(group_size) * group_size ** -0.5).to(dtype=dtype, device=device)


def get_identity_matrix(group_size: int, dtype: torch.dtype, device: torch.device):
    return torch.eye(group_size, dtype=dtype, device=device)


def get_gsr_matrix(group_size: int, dtype: torch.dtype, device: torch.device):
    """Hadamard with columns ordered by their number of sign changes (linear.py:37-41)."""
    h = get_hadamard_matrix(group_size, dtype, device)
    order = torch.argsort(torch.diff(h, dim=0).ne(0).sum(dim=0))
    return h[:, order].contiguous()


_TRANSFORM_INIT = {"hadamard": get_hadamard_matrix, "identity": get_identity_matrix, "gsr": get_gsr_matrix}
_SCALE_GROUP = {FPQuantDtype.MXFP4: 32, FPQuantDtype.NVFP4: 16}


class FPQuantLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, config: FPQuantConfig, bias: bool = True,
                 device: torch.device = None, dtype: torch.dtype = None):
        super().__init__()
        validate_config(config)
        if config.forward_dtype not in _SCALE_GROUP:
            raise ValueError(f"Unsupported forward dtype: {config.forward_dtype}")
        kw = {"device": device, "dtype": dtype}
        self.in_features, self.out_features, self.config = in_features, out_features, config
        self.weight = nn.Parameter(torch.empty((out_features, in_features), **kw))
        self.dqweight = nn.Parameter(torch.empty((out_features, in_features), **kw))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, **kw))
        else:
            self.register_parameter("bias", None)
        g = _SCALE_GROUP[config.forward_dtype]
        self.register_buffer("qweight", torch.empty(out_features, in_features // 2, dtype=torch.uint8, device=device))
        self.register_buffer("scales", torch.empty(out_features, in_features // g, dtype=torch.uint8, device=device))
        self.register_buffer("weight_global_scale", torch.empty(1, **kw))
        self.register_buffer("act_global_scale", torch.empty(1, **kw))
        hg = config.hadamard_group_size
        self.register_buffer("forward_hadamard_matrix", torch.empty(hg, hg, **kw))
        self.register_buffer("backward_hadamard_matrix", torch.empty(hg, hg, **kw))
        self._scales_blocked = None
        self._scales_blocked_key = None
        self._alpha = None
        self._alpha_key = None

    # ------------------------------------------------------------------ load-time step
    @torch.no_grad()
    def pre_forward(self):
        cfg = self.config
        ref = self.weight if self.weight is not None else self.qweight
        assert self.in_features % cfg.hadamard_group_size == 0, (
            f"Weight shape must be divisible by hadamard group size: {self.in_features} % "
            f"{cfg.hadamard_group_size} = {self.in_features % cfg.hadamard_group_size}")
        if not cfg.pseudoquantization:
            assert ref.device.type == "cuda", f"Weight must be on CUDA, but is on {ref.device}"
        if cfg.transform_init not in _TRANSFORM_INIT:
            raise ValueError(f"Invalid transform init: {cfg.transform_init}")
        make = _TRANSFORM_INIT[cfg.transform_init]
        wdtype = self.weight.dtype if self.weight is not None else torch.bfloat16
        self.forward_hadamard_matrix = nn.Buffer(make(cfg.hadamard_group_size, wdtype, ref.device))
        self.backward_hadamard_matrix = nn.Buffer(make(cfg.hadamard_group_size, wdtype, ref.device))
        # Same branch order as the reference (linear.py:190-200): abs_max gives 3.0 for both
        # formats, the 10.0 branch is only reachable for NVFP4 with another method.
        if cfg.forward_dtype == FPQuantDtype.MXFP4 and cfg.forward_method == "quest":
            gsv = 1.0
        elif cfg.forward_method == "abs_max":
            gsv = 3.0
        else:
            gsv = 10.0
        self.weight_global_scale = nn.Buffer(torch.tensor([gsv], dtype=wdtype, device=ref.device))
        self.act_global_scale = nn.Buffer(torch.tensor([gsv], dtype=wdtype, device=ref.device))

        if cfg.store_master_weights:
            self.qweight = self.scales = self.dqweight = None
        elif cfg.pseudoquantization:
            w_dq, _ = forward_pseudoquantize(self.weight.data, self.forward_hadamard_matrix,
                                             self.weight_global_scale, cfg.forward_dtype, cfg.forward_method)
            self.dqweight = nn.Parameter(w_dq, requires_grad=False)
            self.weight = self.qweight = self.scales = None
        else:
            w_q, scales, _ = forward_quantize(self.weight, self.forward_hadamard_matrix, self.weight_global_scale,
                                              cfg.forward_dtype, cfg.forward_method)
            self.qweight = nn.Parameter(w_q, requires_grad=False)
            self.scales = nn.Parameter(scales.view(dtype=torch.uint8), requires_grad=False)
            self.weight = self.dqweight = None
        self._scales_blocked = None

    def _blocked_weight_scales(self) -> torch.Tensor:
        """Weight scale bytes in the swizzled layout, built once per `scales` tensor.  While torch.compile
        traces the module the cache check (addresses and version counters, which a tracer cannot see) is left
        out: a cache filled by an earlier eager call is used as it is, otherwise the re-layout becomes an op of
        the graph."""
        g = _SCALE_GROUP[self.config.forward_dtype]
        if torch.compiler.is_compiling():
            if self._scales_blocked is not None:
                return self._scales_blocked
            return swizzle_scales_op(self.scales.view(torch.uint8)[: self.out_features, : self.in_features // g].contiguous())
        key = (self.scales.data_ptr(), self.scales._version, tuple(self.scales.shape))
        if self._scales_blocked is None or self._scales_blocked_key != key:
            rowmajor = self.scales.view(torch.uint8)[: self.out_features, : self.in_features // g]
            self._scales_blocked = ops.swizzle_scales(rowmajor.contiguous())
            self._scales_blocked_key = key
        return self._scales_blocked

    def _gemm_alpha(self) -> torch.Tensor:
        """1 / (weight_global_scale * act_global_scale) as fp32 [1], recomputed only when a tensor scale changed
        (three small kernels per forward otherwise: the decode path is bound by launches)."""
        w, a = self.weight_global_scale, self.act_global_scale
        if torch.compiler.is_compiling():
            return gemm_alpha(w, a)
        key = (w.data_ptr(), w._version, a.data_ptr(), a._version)
        if self._alpha is None or self._alpha_key != key:
            self._alpha, self._alpha_key = gemm_alpha(w, a), key
        return self._alpha

    def forward_silu_mul(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        """`self(silu(gate) * up)` for the down-projection of a gated MLP, with the activation computed inside
        the quantise kernel (one pass over gate and up instead of three passes over memory; same rounding
        points as the unfused computation).  Falls back to the plain forward for configurations the fused
        kernel does not cover (pseudo-quantisation, master weights, QuEST scales, dense rotations, non-bf16)."""
        cfg = self.config
        fused = (cfg.forward_dtype in _SCALE_GROUP and cfg.backward_dtype == FPQuantDtype.BF16
                 and not cfg.pseudoquantization and not cfg.store_master_weights and cfg.forward_method == "abs_max"
                 and cfg.transform_init in ("hadamard", "identity")
                 and gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and gate.is_cuda)
        if not fused:
            return self.forward(torch.nn.functional.silu(gate) * up)
        lead = gate.shape[:-1]
        g2, u2 = gate.contiguous().flatten(end_dim=-2), up.contiguous().flatten(end_dim=-2)
        nv = cfg.forward_dtype == FPQuantDtype.NVFP4
        rotation = 1 if cfg.transform_init == "hadamard" else 2
        x_q, x_scales = fused_silu_mul_quantize_blocked_op(g2, u2, self.forward_hadamard_matrix,
                                                           self.act_global_scale.float(), nv, rotation)
        bias = self.bias if self.bias is not None and self.bias.dtype == torch.bfloat16 else None
        y = forward_gemm_blocked(x_q, self.qweight, x_scales, self._blocked_weight_scales(), self._gemm_alpha(),
                                 cfg.forward_dtype, bias)
        if self.bias is not None and bias is None:
            y = y + self.bias
        return y.unflatten(dim=0, sizes=lead)

    # ------------------------------------------------------------------ forward
    def forward(self, x) -> torch.Tensor:
        cfg = self.config
        fp4 = cfg.forward_dtype in (FPQuantDtype.MXFP4, FPQuantDtype.NVFP4)
        if fp4 and cfg.backward_dtype == FPQuantDtype.BF16:
            common = (self.weight_global_scale, self.act_global_scale, self.bias, self.forward_hadamard_matrix,
                      cfg.forward_dtype, cfg.forward_method)
            if cfg.pseudoquantization:
                if cfg.store_master_weights:
                    return PseudoQuant4x16MasterFn.apply(x, self.weight, *common)
                return PseudoQuant4x16NoMasterFn.apply(x, self.dqweight, *common)
            if cfg.store_master_weights:
                return FPQuant4x16MasterFn.apply(x, self.weight, *common)
            if not (torch.is_grad_enabled() and x.requires_grad):
                # inference: the function body without the autograd.Function wrapper (its backward only raises)
                return _linear_forward(x, self.qweight, self._blocked_weight_scales(), *common, self._gemm_alpha())
            return FPQuant4x16NoMasterFn.apply(x, self.qweight, self._blocked_weight_scales(), *common,
                                               self._gemm_alpha())
        if cfg.forward_dtype == FPQuantDtype.MXFP4 and cfg.backward_dtype == FPQuantDtype.MXFP8 and not cfg.pseudoquantization:
            common = (self.weight_global_scale, self.act_global_scale, self.bias, self.forward_hadamard_matrix,
                      cfg.forward_dtype, cfg.forward_method)
            if cfg.store_master_weights:
                return FPQuant4x8MasterFn.apply(x, self.weight, *common)
            return FPQuant4x8NoMasterFn.apply(x, self.qweight, self.scales, *common)
        if cfg.forward_dtype == FPQuantDtype.MXFP4 and cfg.backward_dtype == FPQuantDtype.MXFP4 and not cfg.pseudoquantization \
                and cfg.store_master_weights:
            return FPQuant4x4MasterFn.apply(x, self.weight, self.weight_global_scale, self.act_global_scale, self.bias,
                                            self.forward_hadamard_matrix, cfg.forward_dtype, cfg.forward_method)
        raise ValueError(
            f"Forward dtype: {cfg.forward_dtype}, backward dtype: {cfg.backward_dtype}, store_master_weights: "
            f"{cfg.store_master_weights}, pseudoquantization: {cfg.pseudoquantization} isn't supported yet.")
