"""GPU parity of the tcgen05 Hessian accumulation against an fp64 X^T X (bf16 products are exact,
so the only error is fp32 accumulation: <= 1e-5 relative Frobenius, far tighter than the
reference's TF32 path)."""
import pytest
import torch

from oracle import gptq as ogptq
from tests import inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,d", [(64, 128), (200, 256), (2048, 512), (1000, 1032), (4096, 4096), (1024, 3080)])   # the last two: 256 x 256 tiles on CTA pairs, the last with ragged edge tiles
def test_xtx_matches_fp64(cuda_device, tokens, d):
    from fpq_b200 import ops

    x = inputs.correlated_activations(tokens, d, seed=tokens + d)
    want = (x.double().t() @ x.double()) * 0.25
    H = torch.zeros(d, d, device=cuda_device)
    ops.hessian_accumulate(H, x.to(cuda_device), alpha=0.25, beta=0.0)
    ops.check_device_errors(cuda_device)
    got = H.cpu().double()
    assert ((got - want).norm() / want.norm()).item() < 1e-5
    assert torch.equal(H.cpu(), H.cpu().t())          # mirrored exactly


def test_running_mean_matches_gptq_update(cuda_device):
    """Five `GPTQ.update` calls (one sequence each) through alpha/beta on H."""
    from fpq_b200 import ops

    d = 384
    xs = [inputs.correlated_activations(256, d, seed=50 + i).view(1, 256, d) for i in range(5)]
    H_ref, n = None, 0
    for x in xs:
        H_ref, n = ogptq.hessian_update(H_ref, n, x)
    exact = ogptq.hessian_exact(xs, 5)
    H = torch.zeros(d, d, device=cuda_device)
    n = 0
    for x in xs:
        b = x.shape[0]
        ops.hessian_accumulate(H, x.to(cuda_device), alpha=2.0 / (n + b), beta=n / (n + b))
        n += b
    ops.check_device_errors(cuda_device)
    got = H.cpu().double()
    assert ((got - exact).norm() / exact.norm()).item() < 1e-5
    assert ((got - H_ref.double()).norm() / exact.norm()).item() < 1e-5


def test_fp32_input_is_split_into_bf16_terms(cuda_device):
    from fpq_b200 import ops

    x = inputs.correlated_activations(512, 256, seed=9, dtype=torch.float32)
    want = x.double().t() @ x.double()
    H = torch.zeros(256, 256, device=cuda_device)
    ops.hessian_accumulate(H, x.to(cuda_device), alpha=1.0, beta=0.0)
    ops.check_device_errors(cuda_device)
    assert ((H.cpu().double() - want).norm() / want.norm()).item() < 1e-5
