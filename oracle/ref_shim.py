"""Import the unmodified reference (when its tree is present) for pinning the oracle.

TEST INFRASTRUCTURE ONLY.  The reference's `fast_hadamard_transform` dependency
is an external CUDA package that is not vendored; a stub computing the same
product with an explicit Sylvester matrix in fp32 stands in for it
(src/transforms/transforms.py:7, :84).  Nothing here is reachable from the
shipped package, the GPU tests or the benchmark.
"""
from __future__ import annotations

import os
import sys
import types

import torch

# FPQ_REFERENCE_ROOT, or a checkout named "reference" beside this repository
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE_ROOT = os.environ.get("FPQ_REFERENCE_ROOT") or os.path.join(os.path.dirname(_REPO), "reference")


def available() -> bool:
    return os.path.isdir(os.path.join(REFERENCE_ROOT, "src", "quantization"))


def load():
    """Returns the reference's `src` package (quantization, transforms, utils)."""
    if not available():
        raise RuntimeError("reference tree not present")
    if "fast_hadamard_transform" not in sys.modules:
        import scipy.linalg

        stub = types.ModuleType("fast_hadamard_transform")

        def hadamard_transform(x, scale=1.0):
            n = x.shape[-1]
            h = torch.tensor(scipy.linalg.hadamard(n), dtype=torch.float32, device=x.device)
            return ((x.float() @ h) * scale).to(x.dtype)

        stub.hadamard_transform = hadamard_transform
        sys.modules["fast_hadamard_transform"] = stub
    if REFERENCE_ROOT not in sys.path:
        sys.path.insert(0, REFERENCE_ROOT)
    import src.quantization.gptq  # noqa: F401
    import src.quantization.quantizer  # noqa: F401
    import src.quantization.quant_ops  # noqa: F401
    import src  # type: ignore

    return src
