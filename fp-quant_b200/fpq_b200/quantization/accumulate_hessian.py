"""`accumulate_hessian` with the signature of src/quantization/accumulate_hessian.py:112-148
(IST-DASLab/FP-Quant): H += X^T X, on the tcgen05 kernel of the CUDA library."""
from __future__ import annotations

import torch

from .. import ops


def accumulate_hessian(mat_hessian: torch.Tensor, mat_input: torch.Tensor, save_lower_only: bool = False,
                       compute_lower_only: bool = True) -> torch.Tensor:
    """mat_hessian ([meta,] d, d) fp32 is updated in place with the outer products of mat_input
    ([meta,] tokens, d; bf16 is exact, fp32 is split into bf16 terms).  The kernel always computes
    the lower triangle and mirrors it, so the result is the full symmetric matrix whatever the two
    flags say (they are kept for call compatibility)."""
    assert compute_lower_only or not save_lower_only, "compute_lower_only must be True when save_lower_only is True"
    assert mat_hessian.is_contiguous() and mat_input.is_contiguous()
    d = mat_input.shape[-1]
    H = mat_hessian.view(-1, d, d)
    X = mat_input.view(H.shape[0], -1, d)
    for m in range(H.shape[0]):
        ops.hessian_accumulate(H[m], X[m], alpha=1.0, beta=1.0)
    return mat_hessian
