"""Tensor parallelism for `FPQuantLinear` -- new in this package: the reference is single-GPU (README.md:92 of
IST-DASLab/FP-Quant) and leaves tensor parallelism to the serving stack.  Two layers: column-parallel (output
features split; described first) and row-parallel (input features split, outputs summed with one NCCL
all-reduce), and `tensor_parallelize`, which pairs them inside the decoder blocks of a model.

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
        # (only for a bias that is not bf16: the kernels' epilogue takes a bf16 bias, anything else is added afterwards)
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
            # the bias slice goes into the GEMM's epilogue, as in the unsplit layer (same single rounding)
            fused_bias = self.bias if self.bias is not None and self.bias.dtype == torch.bfloat16 else None
            y = forward_gemm_blocked(x_q, self.qweight, x_scales, self.scales_blocked, alpha, cfg.forward_dtype, fused_bias)
            if self.bias is not None and fused_bias is None:
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
        fused_bias = self.bias if self.bias is not None and self.bias.dtype == torch.bfloat16 else None
        ops.gemm_fp4_push(x_q, self.qweight, x_scales, self.scales_blocked, alpha, fmt, buf, peers, self.lo, fused_bias)
        hdl.barrier(channel=1, timeout_ms=BARRIER_TIMEOUT_MS)    # every rank's slice has landed everywhere
        return buf.clone() if (self.bias_full is None or fused_bias is not None) else buf + self.bias_full

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


class RowParallelFPQuantLinear(nn.Module):
    """Input features [lo, hi) of a real-quantised `FPQuantLinear` on this rank: forward(x_local) takes this
    rank's slice of the input (what a column-parallel layer with `gather_output=False` produces), multiplies
    it by the matching columns of the weight and sums the partial products of all ranks with one NCCL
    all-reduce of the bf16 output.  Slices are multiples of 128 input features, so Hadamard groups (<= 128)
    and scale groups stay whole and every rank quantises its slice exactly as the unsplit layer quantises
    those columns; the tensor scales are the unsplit layer's.  The sum over ranks is a bf16 all-reduce of
    bf16-rounded partial products: the result differs from the unsplit layer's single fp32 accumulation by
    rounding (~2^-8 relative), which is why this layer is tested to a tolerance and the column-parallel one
    bit for bit.  The bias is added once, by rank 0's GEMM epilogue, before the sum."""

    def __init__(self, full: FPQuantLinear, process_group=None, reduce_output: bool = True):
        super().__init__()
        cfg = full.config
        if full.qweight is None or cfg.forward_dtype not in _SCALE_GROUP:
            raise ValueError("RowParallelFPQuantLinear needs a real-quantised FP4 layer (call pre_forward first)")
        self.config, self.group, self.reduce_output = cfg, process_group, reduce_output
        self.rank, self.world_size = fdist.world(process_group)
        self.in_features, self.out_features = full.in_features, full.out_features
        self.lo, self.hi = fdist.shard_bounds(self.in_features, self.world_size, self.rank, multiple=128)
        if self.hi <= self.lo:
            raise ValueError(f"in_features = {self.in_features} leaves rank {self.rank} of {self.world_size} without a 128-wide slice")
        g = _SCALE_GROUP[cfg.forward_dtype]
        self.register_buffer("qweight", full.qweight[:, self.lo // 2:self.hi // 2].contiguous())
        rowmajor = full.scales.view(torch.uint8)[: self.out_features, self.lo // g:self.hi // g].contiguous()
        self.register_buffer("scales", rowmajor)
        self.register_buffer("scales_blocked", ops.swizzle_scales(rowmajor))
        self.register_buffer("weight_global_scale", full.weight_global_scale.detach().clone())
        self.register_buffer("act_global_scale", full.act_global_scale.detach().clone())
        self.register_buffer("forward_hadamard_matrix", full.forward_hadamard_matrix.detach().clone())
        self.bias = None
        if full.bias is not None and self.rank == 0:
            self.bias = nn.Parameter(full.bias.detach().clone(), requires_grad=False)
        self._alpha = gemm_alpha(self.weight_global_scale, self.act_global_scale)

    def _finish(self, x_q, x_scales, lead):
        cfg = self.config
        fused_bias = self.bias if self.bias is not None and self.bias.dtype == torch.bfloat16 else None
        y = forward_gemm_blocked(x_q, self.qweight, x_scales, self.scales_blocked, self._alpha, cfg.forward_dtype, fused_bias)
        if self.bias is not None and fused_bias is None:
            y = y + self.bias
        if self.reduce_output and self.world_size > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y.unflatten(dim=0, sizes=lead)

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        x_flat = x_local.contiguous().flatten(end_dim=-2)
        if x_flat.shape[1] != self.hi - self.lo:
            raise ValueError(f"expected this rank's {self.hi - self.lo} input features, got {x_flat.shape[1]}")
        x_q, x_scales = forward_quantize_blocked(x_flat, self.forward_hadamard_matrix, self.act_global_scale,
                                                 cfg.forward_dtype, cfg.forward_method)
        return self._finish(x_q, x_scales, x_local.shape[:-1])

    def forward_silu_mul(self, gate_local: torch.Tensor, up_local: torch.Tensor) -> torch.Tensor:
        """forward(silu(gate) * up) on this rank's slices, the activation computed inside the quantise kernel."""
        cfg = self.config
        if not (cfg.forward_method == "abs_max" and cfg.transform_init in ("hadamard", "identity")
                and gate_local.dtype == torch.bfloat16 and up_local.dtype == torch.bfloat16):
            return self.forward(torch.nn.functional.silu(gate_local) * up_local)
        from .qutlass_ops import fused_silu_mul_quantize_blocked_op

        g2 = gate_local.contiguous().flatten(end_dim=-2)
        u2 = up_local.contiguous().flatten(end_dim=-2)
        x_q, x_scales = fused_silu_mul_quantize_blocked_op(g2, u2, self.forward_hadamard_matrix, self.act_global_scale.float(),
                                                           cfg.forward_dtype == FPQuantDtype.NVFP4,
                                                           1 if cfg.transform_init == "hadamard" else 2)
        return self._finish(x_q, x_scales, gate_local.shape[:-1])


def tensor_parallelize(model: nn.Module, process_group=None) -> int:
    """Splits the real-quantised FPQuantLinear layers of every decoder block over the ranks of `process_group`
    the Megatron way: q/k/v and gate/up column-parallel without gathering (each rank keeps its heads and its
    slice of the MLP width), o_proj and down_proj row-parallel with one all-reduce each, the gated activation
    fused into down_proj's quantise kernel.  Everything else (norms, rotary embedding, residuals, attention
    over the local heads: transformers' attention modules derive the head count from the projection's
    width) runs unchanged on every rank.
    Blocks are recognised by the attribute names of transformers' Llama / Qwen / Mistral decoder layers.
    Returns the number of blocks converted (0 on a single rank: nothing to do)."""
    import types

    rank, world = fdist.world(process_group)
    if world == 1:
        return 0

    def mlp_forward(self, x):
        return self.down_proj.forward_silu_mul(self.gate_proj(x), self.up_proj(x))

    converted = 0
    for module in model.modules():
        attn, mlp = getattr(module, "self_attn", None), getattr(module, "mlp", None)
        if attn is None or mlp is None:
            continue
        names = ("q_proj", "k_proj", "v_proj", "o_proj")
        if not all(isinstance(getattr(attn, n, None), FPQuantLinear) for n in names) or \
                not all(isinstance(getattr(mlp, n, None), FPQuantLinear) for n in ("gate_proj", "up_proj", "down_proj")):
            continue
        head_dim = attn.head_dim
        n_q, n_kv = attn.q_proj.out_features // head_dim, attn.k_proj.out_features // head_dim
        if n_q % world or n_kv % world or (n_q // world * head_dim) % 128 or (n_kv // world * head_dim) % 128:
            raise ValueError(f"{n_q} query / {n_kv} key-value heads of {head_dim} do not split over {world} ranks in 128-wide slices")
        for n in ("q_proj", "k_proj", "v_proj"):
            setattr(attn, n, ColumnParallelFPQuantLinear(getattr(attn, n), process_group, gather_output=False))
        attn.o_proj = RowParallelFPQuantLinear(attn.o_proj, process_group)
        for n in ("gate_proj", "up_proj"):
            setattr(mlp, n, ColumnParallelFPQuantLinear(getattr(mlp, n), process_group, gather_output=False))
        mlp.down_proj = RowParallelFPQuantLinear(mlp.down_proj, process_group)
        mlp.forward = types.MethodType(mlp_forward, mlp)
        converted += 1
    return converted


def column_parallel(full: FPQuantLinear, process_group=None, gather_output: bool = True, fused: bool = False) -> nn.Module:
    """The layer itself when there is a single rank, else its column-parallel slice."""
    if fdist.world(process_group)[1] == 1:
        return full
    return ColumnParallelFPQuantLinear(full, process_group, gather_output, fused)
