"""CPU oracle for the MR-GPTQ hot path.  TEST INFRASTRUCTURE ONLY.

This package restates, with plain torch-CPU / numpy arithmetic, the algorithms
that the CUDA library implements: block-Hadamard rotation, NVFP4 / MXFP4
micro-scaled quantisation, E2M1 packing, the block-scaled FP4 matmul, Hessian
accumulation, the damped Cholesky inverse and the GPTQ column loop.  Every
function cites the file and lines of IST-DASLab/FP-Quant that it follows.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import it.  The shipped package never does: it has no CPU code path and
raises when the CUDA library is missing.

Parity status: PINNED.  The restatement is checked against the unmodified
reference (imported with a stub for its absent `fast_hadamard_transform`
dependency) by `tests/golden/make_golden.py`, which also writes the golden
vectors under `tests/golden/` that the CPU test-suite replays.  Two parts of
the path have no reference code to pin against because they live in the
un-vendored, un-pinned `qutlass` package: the swizzled scale layout (pinned
instead against torch's own `to_blocked` helper) and the FP4 matmul (restated
from the block-scaled format definition; parity unpinned for that kernel).
"""
