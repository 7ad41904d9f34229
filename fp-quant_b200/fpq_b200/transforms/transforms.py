"""Rotations of the MR-GPTQ path with the interface of src/transforms/transforms.py
(IST-DASLab/FP-Quant): identity and block-Hadamard.  The Hadamard runs as the fp32 butterfly
kernel of the CUDA library (the reference calls the external `fast_hadamard_transform`)."""
from __future__ import annotations

import inspect
import math

import torch
import torch.nn as nn

from .. import ops


class BaseTransform(nn.Module):
    def forward(self, x: torch.Tensor, inv_t: bool = False, dim: int = -1):
        raise NotImplementedError

    def remove_parametrizations(self) -> None:
        pass


class IdentityTransform(BaseTransform):
    def __init__(self, *args, **kwargs):
        super().__init__()

    def forward(self, x: torch.Tensor, inv_t: bool = False, dim: int = -1):
        return x


class HadamardTransform(BaseTransform):
    """Block-diagonal Sylvester-Hadamard / sqrt(g) over contiguous groups of the last dim.
    Symmetric and orthogonal, hence its own inverse transpose: `inv_t` changes nothing
    (transforms.py:81-84)."""

    def __init__(self, group_size: int = 128):
        super().__init__()
        self.group_size = group_size
        self.scale = 1 / math.sqrt(group_size)

    def forward(self, x: torch.Tensor, inv_t: bool = False, dim: int = -1):
        if dim not in (-1, x.ndim - 1):
            raise NotImplementedError("the Hadamard rotation acts on the last dim")
        if x.dtype not in (torch.bfloat16, torch.float32):
            return ops.rotate_hadamard(x.float(), self.group_size).to(x.dtype).view(x.shape)
        return ops.rotate_hadamard(x, self.group_size).view(x.shape)


TRANSFORMS = {"identity": IdentityTransform, "hadamard": HadamardTransform}


def build_transform(transform_class: str, **transform_kwargs) -> BaseTransform:
    if transform_class not in TRANSFORMS:
        raise NotImplementedError(f"transform '{transform_class}' is outside the MR-GPTQ path (have {list(TRANSFORMS)})")
    cls = TRANSFORMS[transform_class]
    accepted = inspect.signature(cls.__init__).parameters
    return cls(**{k: v for k, v in transform_kwargs.items() if k in accepted})


def get_transform_matrix(transform_class: str, size: int, device=None, dtype=None) -> torch.Tensor:
    """The g x g matrix a checkpoint stores as forward/backward_hadamard_matrix (transforms.py:312-323)."""
    if transform_class == "hadamard":
        eye = torch.eye(size, device=device, dtype=torch.float32)
        return ops.rotate_hadamard(eye, size).to(dtype or torch.float32)
    if transform_class == "identity":
        return torch.eye(size, device=device, dtype=dtype)
    raise NotImplementedError("get_transform_matrix is implemented only for Hadamard and Identity transforms")
