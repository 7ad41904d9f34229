"""fpq_b200: the MR-GPTQ hot path of FP-Quant on B200 (sm_100a).

`fpq_b200.quantization`, `fpq_b200.transforms` mirror the reference's `src.quantization`
and `src.transforms`; `fpq_b200.fp_quant` mirrors the `fp_quant` inference package.
All numeric work is done by hand-written CUDA kernels behind a C ABI (`fpq_b200._cabi`).
"""
__version__ = "0.1.0"
