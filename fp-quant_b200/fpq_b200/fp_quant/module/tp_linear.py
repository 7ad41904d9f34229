"""Column-split (output-feature) tensor parallelism for `FPQuantLinear` -- new in this package: the reference
is single-GPU (README.md:92 of IST-DASLab/FP-Quant) and leaves tensor parallelism to the serving stack.

The split is along N only.  K is never split, so Hadamard groups, scale groups and the activation
quantisation are untouched: every rank quantises the (replicated) activations itself, multiplies by its own
rows of `qweight` / `scales`, and the [M, N/p] slices are gathered along N.  The weight's tensor scale was
fixed on the full weight before the split, so the slices decode exactly as the full layer does and the
gathered output equals the unsplit layer's output bit for bit.

Two ways to gather: NCCL (`all_gather_into_tensor` + a transposing copy), or `fused=True`: the GEMM's
epilogue stores every finished tile into its place of every rank's [M, N] buffer through peer pointers of a
torch symmetric-memory allocation (ordinary stores over NVLink, overlapping the remaining tiles), followed
by one device-side barrier among the ranks.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ... import dist as fdist
from ... import ops
from ..utils.config import FPQuantDtype
from .linear import FPQuantLinear
from .linear_fns import forward_gemm_blocked, forward_quantize_blocked, gemm_alpha

_SCALE_GROUP = {FPQuantDtype.MXFP4: 32, FPQuantDtype.NVFP4: 16}
BARRIER_TIMEOUT_MS = 10_000


def fused_path_allowed(out_features: int, world_size: int) -> bool:
    """True when every rank's slice of `out_features` is at least 256 rows (what the epilogue-push kernel
    needs).  Depends on nothing rank-local, so all ranks agree."""
    return min(hi - lo for lo, hi in fdist.all_bounds(out_features, world_size, 128)) >= 256


class ColumnParallelFPQuantLinear(nn.Module):
    """Rows [lo, hi) of a real-quantised `FPQuantLinear` (after `pre_forward`) on this rank.

    forward(x) returns the full [.., N] output on every rank (`gather_output=True`) or this rank's
    [.., hi - lo] slice.  Slices are multiples of 128 rows (the scale-tile height) except the last."""

    def __init__(self, full: FPQuantLinear, process_group=None, gather_output: bool = True, fused: bool = False):
        super().__init__()
        self.fused = fused and gather_output
        self._symm = {}                  # M -> (buffer, handle)
        cfg = full.config
        if full.qweight is None or cfg.forward_dtype not in _SCALE_GROUP:
            raise ValueError("ColumnParallelFPQuantLinear needs a real-quantised FP4 layer (call pre_forward first)")
        self.config, self.group, self.gather_output = cfg, process_group, gather_output
        self.rank, self.world_size = fdist.world(process_group)
        self.in_features, self.out_features = full.in_features, full.out_features
        self.lo, self.hi = fdist.shard_bounds(self.out_features, self.world_size, self.rank, multiple=128)
        # Shares differ by one 128-row unit, so "my slice is wide enough for the large-M kernel" is not the same
        # on every rank.  The fused path is a collective (symmetric-memory barriers on all ranks): it is taken
        # only when EVERY rank's slice qualifies, a decision all ranks reach identically.
        self.fused_ok = fused_path_allowed(self.out_features, self.world_size)
        g = _SCALE_GROUP[cfg.forward_dtype]
        self.register_buffer("qweight", full.qweight[self.lo:self.hi].contiguous())
        rowmajor = full.scales.view(torch.uint8)[self.lo:self.hi, : self.in_features // g].contiguous()
        self.register_buffer("scales", rowmajor)
        self.register_buffer("scales_blocked", ops.swizzle_scales(rowmajor) if self.hi > self.lo else rowmajor)
        self.register_buffer("weight_global_scale", full.weight_global_scale.detach().clone())
        self.register_buffer("act_global_scale", full.act_global_scale.detach().clone())
        self.register_buffer("forward_hadamard_matrix", full.forward_hadamard_matrix.detach().clone())
        self.bias = None if full.bias is None else nn.Parameter(full.bias.detach()[self.lo:self.hi].clone(), requires_grad=False)
        # the fused path adds the bias to the gathered output, as the unsplit module does (after the bf16 rounding)
        self.bias_full = None if full.bias is None else nn.Parameter(full.bias.detach().clone(), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        x_flat = x.contiguous().flatten(end_dim=-2)
        m = x_flat.shape[0]
        n_loc = self.hi - self.lo
        if self.fused and self.world_size > 1 and m > 128 and self.fused_ok:
            return self._forward_fused(x_flat, m).unflatten(dim=0, sizes=x.shape[:-1])
        if n_loc > 0:
            x_q, x_scales = forward_quantize_blocked(x_flat, self.forward_hadamard_matrix, self.act_global_scale,
                                                     cfg.forward_dtype, cfg.forward_method)
            alpha = gemm_alpha(self.weight_global_scale, self.act_global_scale)
            y = forward_gemm_blocked(x_q, self.qweight, x_scales, self.scales_blocked, alpha, cfg.forward_dtype)
            if self.bias is not None:
                y = y + self.bias
        else:
            y = torch.empty(m, 0, dtype=torch.bfloat16, device=x.device)
        if self.gather_output and self.world_size > 1:
            y = self._gather_columns(y, m)
        return y.unflatten(dim=0, sizes=x.shape[:-1])

    def _symmetric_buffer(self, m: int, device):
        import torch.distributed._symmetric_memory as symm_mem

        if m not in self._symm:
            group = self.group if self.group is not None else dist.group.WORLD
            buf = symm_mem.empty(m, self.out_features, dtype=torch.bfloat16, device=device)
            self._symm[m] = (buf, symm_mem.rendezvous(buf, group))
        return self._symm[m]

    def _forward_fused(self, x_flat: torch.Tensor, m: int) -> torch.Tensor:
        cfg = self.config
        fmt = "nvfp4" if cfg.forward_dtype == FPQuantDtype.NVFP4 else "mxfp4"
        buf, hdl = self._symmetric_buffer(m, x_flat.device)
        x_q, x_scales = forward_quantize_blocked(x_flat, self.forward_hadamard_matrix, self.act_global_scale,
                                                 cfg.forward_dtype, cfg.forward_method)
        alpha = gemm_alpha(self.weight_global_scale, self.act_global_scale)
        # bounded: a rank that never arrives ends the wait with an error instead of a stuck kernel
        hdl.barrier(channel=0, timeout_ms=BARRIER_TIMEOUT_MS)    # every rank is done with the previous contents
        # the tensor may sit at an offset inside the symmetric allocation; the offset is the same on every rank
        off = buf.data_ptr() - int(hdl.buffer_ptrs[self.rank])
        if off < 0 or off + buf.numel() * 2 > int(hdl.buffer_size):
            raise RuntimeError("symmetric buffer does not contain the output tensor")
        peers = [int(hdl.buffer_ptrs[r]) + off for r in range(self.world_size) if r != self.rank]
        ops.gemm_fp4_push(x_q, self.qweight, x_scales, self.scales_blocked, alpha, fmt, buf, peers, self.lo, None)
        hdl.barrier(channel=1, timeout_ms=BARRIER_TIMEOUT_MS)    # every rank's slice has landed everywhere
        return buf.clone() if self.bias_full is None else buf + self.bias_full

    def _gather_columns(self, y: torch.Tensor, m: int) -> torch.Tensor:
        bounds = fdist.all_bounds(self.out_features, self.world_size, 128)
        widest = max(hi - lo for lo, hi in bounds)
        if y.shape[1] != widest:
            pad = torch.zeros(m, widest, dtype=y.dtype, device=y.device)
            pad[:, : y.shape[1]] = y
            y = pad
        stacked = torch.empty(self.world_size, m, widest, dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(stacked, y.contiguous(), group=self.group)
        if all(hi - lo == widest for lo, hi in bounds):
            return stacked.permute(1, 0, 2).reshape(m, self.out_features)
        return torch.cat([stacked[r, :, : hi - lo] for r, (lo, hi) in enumerate(bounds)], dim=1)


def column_parallel(full: FPQuantLinear, process_group=None, gather_output: bool = True, fused: bool = False) -> nn.Module:
    """The layer itself when there is a single rank, else its column-parallel slice."""
    if fdist.world(process_group)[1] == 1:
        return full
    return ColumnParallelFPQuantLinear(full, process_group, gather_output, fused)
