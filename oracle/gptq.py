"""Oracle: Hessian accumulation, damped Cholesky inverse and the GPTQ column loop.

TEST INFRASTRUCTURE ONLY (see the package docstring).  torch-CPU fp32 arithmetic
following src/quantization/gptq.py of IST-DASLab/FP-Quant.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import fp4


def hessian_update(H: Optional[torch.Tensor], num_samples: int, inp: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """One `GPTQ.update` call (gptq.py:69-102): running mean
    H <- H * n/(n+b) + (2/(n+b)) * X^T X with b = inp.shape[0] (sequences, not tokens)
    and X = inp flattened to [tokens, d] in fp32.  The Triton kernel it calls
    (accumulate_hessian.py:112-148) is restated as an fp32 matmul accumulate.
    """
    b = inp.shape[0]
    x = inp.reshape(-1, inp.shape[-1]).to(torch.float32)
    d = x.shape[1]
    if H is None:
        H = torch.zeros(d, d, dtype=torch.float32)
    beta = num_samples / (num_samples + b)
    alpha = 2.0 / (num_samples + b)
    H = H * beta
    xs = x * math.sqrt(alpha)
    H = H + xs.t() @ xs
    return H, num_samples + b


def hessian_exact(inputs, num_sequences: int) -> torch.Tensor:
    """(2/N_seq) * sum X^T X in fp64: what the running mean converges to."""
    acc = None
    for inp in inputs:
        x = inp.reshape(-1, inp.shape[-1]).to(torch.float64)
        acc = x.t() @ x if acc is None else acc + x.t() @ x
    return acc * (2.0 / num_sequences)


def prepare_hessian(H: torch.Tensor, W: torch.Tensor, rel_damp: float) -> torch.Tensor:
    """Dead-column fix and damping (gptq.py:201-211), returns a new tensor:
    columns of W that are entirely zero get H row/col zeroed and diagonal 1;
    then H += rel_damp * mean(diag H) * I.
    """
    H = H.clone()
    dead = W.eq(0).all(dim=0)
    H[dead, :] = 0
    H[:, dead] = 0
    idx = torch.nonzero(dead).flatten()
    H[idx, idx] = 1
    damp = rel_damp * torch.diag(H).mean()
    H.diagonal().add_(damp)
    return H


def cholesky_inverse_upper(Hd: torch.Tensor) -> Tuple[torch.Tensor, bool]:
    """U upper-triangular with U^T U = Hd^-1 (gptq.py:212-217,
    src/utils/linalg_utils.py:8-12): cholesky -> cholesky_inverse -> cholesky(upper).
    On any failure the reference silently substitutes the identity; the flag
    reports that.
    """
    try:
        L = torch.linalg.cholesky(Hd)
        Hinv = torch.cholesky_inverse(L)
        U = torch.linalg.cholesky(Hinv, upper=True)
        return U, True
    except Exception:
        return torch.eye(Hd.shape[0], dtype=torch.float32), False


def gptq_column_loop(W: torch.Tensor, scales: torch.Tensor, U: torch.Tensor, group: int,
                     block_size: int = 128, group_index: torch.Tensor = None):
    """The hot loop of `GPTQ.step` (gptq.py:159-187), export path.  Default order: column i uses the
    scale of group i // group; with `group_index` (activation order, gptq.py:146-148, 170-171) W's columns
    are already permuted and column i uses the scale of group group_index[i].

    W [R, C] fp32 (rotated), scales fp32 [R, C/group] fixed beforehand from the
    unmodified W (gptq.py:142), U from `cholesky_inverse_upper`.
    Per column i: q = e2m1(w_i / s), w_q = grid(q) * s, err = (w_i - w_q) / U[i, i],
    W_blk[:, i:] -= err (x) U[i, i:]; after each block W[:, c2:] -= Err @ U[c1:c2, c2:].
    Returns (dequantised W fp32, codes uint8 [R, C]).
    """
    w = W.clone().to(torch.float32)
    R, C = w.shape
    codes = torch.empty(R, C, dtype=torch.uint8)
    for c1 in range(0, C, block_size):
        c2 = min(c1 + block_size, C)
        blk = w[:, c1:c2].clone()
        errs = torch.zeros_like(blk)
        Ub = U[c1:c2, c1:c2]
        for i in range(c2 - c1):
            col = blk[:, i]
            s = scales[:, (c1 + i) // group] if group_index is None else scales[:, int(group_index[c1 + i])]
            c = fp4.e2m1_codes(col.unsqueeze(-1), s.unsqueeze(-1), 1).squeeze(-1)
            wq = fp4.code_values(c) * s
            codes[:, c1 + i] = c
            w[:, c1 + i] = wq
            err = (col - wq) / Ub[i, i]
            blk[:, i:].addr_(err, Ub[i, i:], alpha=-1)
            errs[:, i] = err
        w[:, c2:].addmm_(errs, U[c1:c2, c2:], alpha=-1)
    return w, codes


def relative_mse(Wq: torch.Tensor, W: torch.Tensor, H: torch.Tensor) -> float:
    """gptq.py:28-30: mean((dW H) * dW) / (mean((W H) * W) + 1e-6)."""
    d = (Wq - W).to(torch.float64)
    Hd = H.to(torch.float64)
    Wd = W.to(torch.float64)
    return float((d @ Hd).mul(d).mean() / ((Wd @ Hd).mul(Wd).mean() + 1e-6))


def activation_order(H: torch.Tensor, group: int):
    """gptq.py:146-152: columns sorted by falling diag(H); returns (perm, perm_inv, group_index) where
    group_index[i] is the scale group of the column that lands at position i."""
    perm = torch.argsort(torch.diag(H), descending=True)
    d = H.shape[0]
    group_index = torch.arange(d // group).repeat_interleave(group)[perm]
    return perm, torch.argsort(perm), group_index
