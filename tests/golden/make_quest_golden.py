"""Golden vectors for the "quest" forward method from the reference's own Triton kernel.

    python tests/golden/make_quest_golden.py        # needs the reference tree (FPQ_REFERENCE_ROOT) and triton

`mxfp4_forward_kernel` (inference_lib/src/fp_quant/module/triton/mxfp4.py:19-119 of IST-DASLab/FP-Quant) is
the only statement of the QuEST scale rule in the reference tree (the real-quantisation twin lives in the
absent `qutlass` package).  Triton's interpreter (TRITON_INTERPRET=1) runs the UNMODIFIED kernel body on the
CPU.  Two things about the call differ from the reference's wrapper, neither touching the kernel: the
autotuner (which needs a GPU to time configurations) is bypassed with BLOCK_SIZE = 1024, one of its own
choices, and the tensors are fp32 holding bf16-exact values, because the interpreter has no bf16 (the kernel
computes in fp32 either way).  The rotation matrix handed in is the identity, so the kernel's `tl.dot`
returns the input bit for bit and what is recorded is the scale / rounding / clip-mask rule alone.
Output: quest_triton.npz (input, dequantised output, clip mask), also for quest=False (abs_max).
"""
import importlib.util
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import ref_shim  # noqa: E402
from tests import inputs  # noqa: E402


def main():
    path = os.path.join(ref_shim.REFERENCE_ROOT, "inference_lib", "src", "fp_quant", "module", "triton", "mxfp4.py")
    spec = importlib.util.spec_from_file_location("reference_triton_mxfp4", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    kernel = mod.mxfp4_forward_kernel.fn                      # the jitted function under the autotuner
    x = inputs.outlier_activations(64, 512, seed=41).float()  # bf16-exact values in fp32
    x[3, 32:64] = 0.0                                          # an all-zero group
    x[5, :32] = 1.0                                            # a constant group: zero variance
    eye = torch.eye(32, dtype=torch.float32)
    out = {"x": x.numpy()}
    for tag, quest, c in (("quest", True, 2.92247856 / 6.0), ("absmax", False, 3.0 / 4.0)):
        y = torch.empty_like(x)
        mask = torch.empty_like(x, dtype=torch.bool)
        n = x.numel()
        kernel[(n // 1024,)](x_ptr=x, hadamard_matrix_ptr=eye, output_ptr=y, clip_mask_ptr=mask, n_elements=n,
                             hadamard_dim=32, group_size=32, gaussian_scale=c, quest=quest, BLOCK_SIZE=1024)
        out[tag + "_dequantized"] = y.numpy()
        out[tag + "_mask"] = mask.numpy()
    np.savez_compressed(os.path.join(HERE, "quest_triton.npz"), **out)
    print("wrote quest_triton.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
