"""Multi-GPU partitioning of the GPTQ path (the reference is single-GPU, README.md:92 of
IST-DASLab/FP-Quant; this layer is new).

One process per GPU, `torch.distributed` for the plumbing (NCCL over NVLink on GPUs; the same code
runs on gloo/CPU tensors for the host-logic tests).  The path shards naturally:

* Hessian: H = (2/N) sum_seq X_s^T X_s is a sum over calibration sequences.  Every rank accumulates
  the sequences it owns with the GLOBAL factor 2/N, then one all-reduce(sum) of the fp32 d x d
  matrix gives every rank the full H.
* Column loop: rows of W are independent given U (gptq.py:159-187 works on all rows at once only
  for convenience), so each rank quantises a contiguous slab of rows and the slabs are gathered.
* The Cholesky-inverse factor U is computed redundantly on every rank (no communication; the ranks
  would otherwise idle).
No collective touches a kernel's inner loop; each is one NCCL call on a whole tensor.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def world(group=None) -> Tuple[int, int]:
    """(rank, world_size); (0, 1) when torch.distributed is not initialised."""
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def shard_bounds(n: int, world_size: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """[lo, hi) of rank's contiguous share of n items, shares being multiples of `multiple`
    (except possibly the last non-empty one) and differing by at most one unit."""
    units = (n + multiple - 1) // multiple
    base, extra = divmod(units, world_size)
    lo_u = rank * base + min(rank, extra)
    hi_u = lo_u + base + (1 if rank < extra else 0)
    return min(lo_u * multiple, n), min(hi_u * multiple, n)


def weighted_bounds(n: int, weights: List[float]) -> List[Tuple[int, int]]:
    """Contiguous shares of n items proportional to `weights` (largest-remainder rounding; every rank with a
    positive weight gets at least one item when n allows)."""
    total = float(sum(weights))
    raw = [n * w / total for w in weights]
    counts = [int(r) for r in raw]
    for i in sorted(range(len(weights)), key=lambda i: raw[i] - counts[i], reverse=True)[: n - sum(counts)]:
        counts[i] += 1
    for i, w in enumerate(weights):          # nobody with work to do is left empty-handed
        if w > 0 and counts[i] == 0 and max(counts) > 1:
            counts[counts.index(max(counts))] -= 1
            counts[i] = 1
    out, lo = [], 0
    for c in counts:
        out.append((lo, lo + c))
        lo += c
    return out


def all_bounds(n: int, world_size: int, multiple: int = 1) -> List[Tuple[int, int]]:
    return [shard_bounds(n, world_size, r, multiple) for r in range(world_size)]


def allreduce_sum_(t: torch.Tensor, group=None) -> torch.Tensor:
    if world(group)[1] > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


def reduce_sum_(t: torch.Tensor, dst: int, group=None) -> torch.Tensor:
    """Sum over the ranks, delivered to rank `dst` of the group only; the other ranks' `t` is left undefined."""
    if world(group)[1] > 1:
        dist.reduce(t, dst=dst if group is None else dist.get_global_rank(group, dst), op=dist.ReduceOp.SUM, group=group)
    return t


def allreduce_min_(t: torch.Tensor, group=None) -> torch.Tensor:
    """Running-minimum quantities (NVFP4 global scales) across ranks."""
    if world(group)[1] > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    return t


def allgather_rows(local: torch.Tensor, total_rows: int, multiple: int = 1, group=None) -> torch.Tensor:
    """Concatenate row slabs (split by `shard_bounds(total_rows, ...)`) from all ranks, in rank order."""
    rank, ws = world(group)
    if ws == 1:
        return local
    bounds = all_bounds(total_rows, ws, multiple)
    assert local.shape[0] == bounds[rank][1] - bounds[rank][0], "local slab does not match this rank's bounds"
    biggest = max(hi - lo for lo, hi in bounds)
    padded = local
    if local.shape[0] != biggest:
        padded = torch.zeros((biggest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        padded[: local.shape[0]] = local
    out = torch.empty((ws * biggest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded.contiguous(), group=group)
    if all(hi - lo == biggest for lo, hi in bounds):
        return out
    return torch.cat([out[r * biggest: r * biggest + (hi - lo)] for r, (lo, hi) in enumerate(bounds)], dim=0)


class ShardedLayerGPTQ:
    """MR-GPTQ of one linear layer over the ranks of a process group.

    update(x)            x: this rank's calibration sequences [n_local, tokens, d] (already rotated)
    finish_hessian(N)    all-reduce; N = total number of sequences over all ranks
    quantize(W, ...)     every rank passes the same rotated fp32 weight; returns the full results
    """

    def __init__(self, d_col: int, device, group=None):
        self.group = group
        self.rank, self.world_size = world(group)
        self.H = torch.zeros(d_col, d_col, dtype=torch.float32, device=device)
        self.local_sequences = 0

    def update(self, x: torch.Tensor, total_sequences: int, accumulate) -> None:
        """`accumulate(H, x2d, alpha, beta)` adds alpha * x^T x to H (the CUDA op on GPUs)."""
        accumulate(self.H, x.reshape(-1, x.shape[-1]), 2.0 / total_sequences, 1.0)
        self.local_sequences += x.shape[0]

    def finish_hessian(self) -> torch.Tensor:
        return allreduce_sum_(self.H, self.group)

    def quantize(self, W: torch.Tensor, scales: torch.Tensor, U: torch.Tensor, group_size: int, column_loop):
        """`column_loop(W_slab, scales_slab, U, group_size) -> (dequantised slab, packed codes slab)`.
        Returns the gathered dequantised weight and packed codes."""
        rows = W.shape[0]
        lo, hi = shard_bounds(rows, self.world_size, self.rank, multiple=128)
        wq, codes = column_loop(W[lo:hi].contiguous(), scales[lo:hi].contiguous(), U, group_size)
        return (allgather_rows(wq, rows, 128, self.group), allgather_rows(codes, rows, 128, self.group))
