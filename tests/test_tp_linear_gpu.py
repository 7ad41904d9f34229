"""Column-split tensor-parallel FPQuantLinear on two GPUs: the gathered output must equal the unsplit
layer's output bit for bit (K is not split, so every product is the same)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_path):
    import sys

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    sys.path.insert(0, os.path.join(os.path.dirname(here), "fp-quant_b200"))
    sys.path.insert(0, os.path.dirname(here))
    import torch.distributed as dist

    import inputs
    from fpq_b200.fp_quant import FPQuantConfig, FPQuantDtype, FPQuantLinear
    from fpq_b200.fp_quant.module.tp_linear import ColumnParallelFPQuantLinear

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok = True
    for fmt, hg, n in ((FPQuantDtype.MXFP4, 32, 1024), (FPQuantDtype.NVFP4, 16, 1152)):   # 1152 = 9 x 128: uneven split
        cfg = FPQuantConfig(forward_dtype=fmt, forward_method="abs_max", backward_dtype=FPQuantDtype.BF16,
                            hadamard_group_size=hg)
        layer = FPQuantLinear(512, n, cfg, bias=True, device=dev, dtype=torch.bfloat16)
        layer.weight.data.copy_(inputs.normal_weight(n, 512, seed=3))
        layer.bias.data.copy_(torch.linspace(-1, 1, n))
        layer.pre_forward()
        x = inputs.outlier_activations(300, 512, seed=5).to(dev)
        want = layer(x)
        got = ColumnParallelFPQuantLinear(layer, None, gather_output=True)(x)
        if not torch.equal(got, want):
            ok = False
            print(f"rank {rank} {fmt} nccl gather differs: {(got.float() - want.float()).abs().max().item()}", flush=True)
        fused = ColumnParallelFPQuantLinear(layer, None, gather_output=True, fused=True)
        for it in range(3):              # repeated calls reuse the symmetric buffer
            got = fused(x)
            if not torch.equal(got, want):
                ok = False
                bad = (got != want)
                print(f"rank {rank} {fmt} fused call {it} differs: {int(bad.sum())} elements, columns "
                      f"{bad.any(dim=0).nonzero().flatten()[:4].tolist()}..{bad.any(dim=0).nonzero().flatten()[-4:].tolist()} "
                      f"rows {bad.any(dim=1).nonzero().flatten()[:4].tolist()}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        torch.save({"equal": ok}, out_path)


def test_column_parallel_linear_equals_full_layer(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    out = str(tmp_path / "result.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert torch.load(out)["equal"]
