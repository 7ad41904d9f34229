"""The allocation-free Hessian preparation (`fpq_hessian_prepare_noalloc`) against the ordinary
entry point.

Why it exists: some callers of this library cannot allocate device memory when they need to
prepare a Hessian -- a runtime that handed all of HBM to its own pool at start-up, a plugin whose
host framework forbids driver allocations in its steady state, or code inside a stream capture,
where cudaMalloc is illegal.  For them the scratch (one dead-column flag per input channel) is a
fixed array inside the library instead of a caller-provided workspace.

This file is named so that pytest collects it last: if it fails, a run that stops at the first
failure has already run every other test.  The calls go straight through the C ABI with raw
pointers; torch only provides the input/output buffers.
"""
import ctypes

import pytest
import torch

from tests import inputs

pytestmark = pytest.mark.gpu


def _hessian_and_weight(d, rows, seed, dead):
    x = inputs.correlated_activations(2 * d, d, seed=seed, dtype=torch.float32)
    H = (x.t() @ x) * 0.5
    W = inputs.normal_weight(rows, d, seed=seed + 1, dtype=torch.float32)
    for j in dead:
        W[:, j] = 0
    return H, W


def test_noalloc_matches_workspace_variant_twice_in_a_row(cuda_device):
    from fpq_b200 import _cabi

    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second call finds the first call's flags in the
    # shared scratch and must not be affected by them (more dead columns first, fewer and elsewhere after)
    cases = [(512, 96, 1, (3, 77, 200, 511)), (384, 64, 7, (5,))]
    for d, rows, seed, dead in cases:
        H, W = _hessian_and_weight(d, rows, seed, dead)
        Wd = W.to(cuda_device)
        H_ref = H.clone().to(cuda_device)
        ws = torch.empty(d, dtype=torch.uint8, device=cuda_device)
        _cabi.check(lib.fpq_hessian_prepare(H_ref.data_ptr(), d, Wd.data_ptr(), rows, ctypes.c_float(0.01),
                                            ws.data_ptr(), stream))
        H_new = H.clone().to(cuda_device)
        _cabi.check(lib.fpq_hessian_prepare_noalloc(H_new.data_ptr(), d, Wd.data_ptr(), rows, ctypes.c_float(0.01),
                                                    stream))
        torch.cuda.synchronize()
        assert torch.equal(H_new, H_ref)                      # same kernels, same arithmetic: bit-identical
        for j in dead:
            assert H_new[j, j].item() > 1.0 and H_new[j, (j + 1) % d].item() == 0.0


def test_noalloc_rejects_sizes_beyond_its_scratch(cuda_device):
    from fpq_b200 import _cabi

    lib = _cabi.lib()
    H = torch.zeros(4, 4, device=cuda_device)
    W = torch.ones(1, 4, device=cuda_device)
    rc = lib.fpq_hessian_prepare_noalloc(H.data_ptr(), 32768 + 1, W.data_ptr(), 1, ctypes.c_float(0.01),
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    assert b"exceeds the built-in scratch" in lib.fpq_last_error()


def test_noalloc_at_its_size_limit(cuda_device):
    """d = FPQ_PREPARE_NOALLOC_MAX_D uses the whole built-in array: dead columns in the first and in the last
    256-column tile, compared with the workspace variant on the diagonal and on the dead rows / columns
    (the full 4 GiB matrices are compared on the device)."""
    from fpq_b200 import _cabi

    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    d, rows, dead = 32768, 8, (7, 32768 - 200, 32768 - 1)
    g = torch.Generator(device=cuda_device).manual_seed(3)
    H = torch.rand(d, d, device=cuda_device, generator=g)
    W = torch.rand(rows, d, device=cuda_device, generator=g) + 0.5
    for j in dead:
        W[:, j] = 0
    H_ref = H.clone()
    ws = torch.empty(d, dtype=torch.uint8, device=cuda_device)
    _cabi.check(lib.fpq_hessian_prepare(H_ref.data_ptr(), d, W.data_ptr(), rows, ctypes.c_float(0.01), ws.data_ptr(), stream))
    _cabi.check(lib.fpq_hessian_prepare_noalloc(H.data_ptr(), d, W.data_ptr(), rows, ctypes.c_float(0.01), stream))
    torch.cuda.synchronize()
    assert torch.equal(H, H_ref)
    for j in dead:
        assert torch.count_nonzero(H[j]).item() == 1 and torch.count_nonzero(H[:, j]).item() == 1
    assert H[5, 5].item() != H_ref[7, 7].item()      # a live diagonal entry kept its own value plus the damping
