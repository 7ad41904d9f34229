"""Recognise the g x g rotation matrices the inference API passes around (hadamard / identity /
anything else) so that the fused kernel can use its in-register butterfly instead of a dense
product.  The classification reads the matrix once (one device sync) and is cached."""
from __future__ import annotations

from typing import Tuple

import torch

ROT_DETECT, ROT_HADAMARD, ROT_IDENTITY, ROT_DENSE = 0, 1, 2, 3
_KIND_CODE = {"hadamard": ROT_HADAMARD, "identity": ROT_IDENTITY, "dense": ROT_DENSE}
_CODE_KIND = {v: k for k, v in _KIND_CODE.items()}


def sylvester(group: int) -> torch.Tensor:
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < group:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h


def classify_rotation(matrix: torch.Tensor) -> Tuple[str, int]:
    """('hadamard' | 'identity' | 'dense', group).  The verdict is remembered on the tensor
    object (and dropped when the tensor is modified in place)."""
    g = matrix.shape[-1]
    memo = getattr(matrix, "_fpq_rotation", None)
    if memo is not None and memo[0] == matrix._version:
        return memo[1], g
    kind = "dense"
    if matrix.ndim == 2 and matrix.shape[0] == g and g in (16, 32, 64, 128):
        m = matrix.detach().to(torch.float64).cpu()
        had = sylvester(g) * g ** -0.5
        # the caller's matrix was rounded to its dtype (bf16 in the inference path)
        if torch.equal(m, had.to(matrix.dtype).to(torch.float64)):
            kind = "hadamard"
        elif torch.equal(m, torch.eye(g, dtype=torch.float64)):
            kind = "identity"
    try:
        matrix._fpq_rotation = (matrix._version, kind)
    except Exception:
        pass
    return kind, g


def rotation_code(matrix: torch.Tensor) -> int:
    return _KIND_CODE[classify_rotation(matrix)[0]]


def kind_of(code: int, matrix: torch.Tensor) -> Tuple[str, int]:
    if code == ROT_DETECT:
        return classify_rotation(matrix)
    return _CODE_KIND[code], matrix.shape[-1]
