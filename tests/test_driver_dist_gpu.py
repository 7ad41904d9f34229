"""Multi-GPU model-level MR-GPTQ: two ranks (one per GPU, NCCL) quantise a tiny Llama with the calibration
sequences, the Cholesky chains and the weight rows partitioned; the result must agree with the single-GPU
run of the same driver (the Hessian sum is reassociated, so agreement is statistical, as for any GPTQ
parity check: a flipped code changes the later errors of its row)."""
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

    from test_driver_gpu import _args, _calibration, _tiny_llama
    from fpq_b200.quantization.driver import gptq_quantization

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    data = _calibration(dev)
    model = _tiny_llama(dev)
    from fpq_b200.quantization import driver as drv

    quantized, _ = gptq_quantization(model, data, _args("nvfp"), dev)
    with torch.no_grad():
        logits = torch.cat([model(x.to(dev)).logits.float() for x in data]).cpu()
    split_exact = drv._split_state.get("exact")
    # the same two-rank run with the second pass in one piece (the down-projection not deferred): the split
    # pass adds the same two bf16 tensors the block adds, so codes and logits must be identical
    plain_args = _args("nvfp")
    plain_args.split_second_pass = False
    model_p = _tiny_llama(dev)
    quantized_p, _ = gptq_quantization(model_p, data, plain_args, dev)
    with torch.no_grad():
        logits_p = torch.cat([model_p(x.to(dev)).logits.float() for x in data]).cpu()
    same_as_plain = all(torch.equal(quantized[k]["qweight"], quantized_p[k]["qweight"]) for k in quantized) \
        and torch.equal(logits, logits_p)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        # the same driver on one GPU, no process group
        model1 = _tiny_llama(dev)
        quantized1, _ = gptq_quantization(model1, data, _args("nvfp"), dev)
        with torch.no_grad():
            logits1 = torch.cat([model1(x.to(dev)).logits.float() for x in data]).cpu()
        def agreement(keys):
            agree, total = 0, 0
            for k in keys:
                a, b = quantized[k]["qweight"], quantized1[k]["qweight"]
                agree += int(((a & 0xF) == (b & 0xF)).sum() + ((a >> 4) == (b >> 4)).sum())
                total += 2 * a.numel()
            return agree / total

        first = [f"model.layers.0.self_attn.{n}_proj" for n in "qkv"]
        torch.save({"agree": agreement(list(quantized1)), "agree_first": agreement(first),
                    "keys": sorted(quantized) == sorted(quantized1), "split_exact": split_exact,
                    "same_as_plain": same_as_plain,
                    "logit_diff": float(((logits - logits1) ** 2).mean() / (logits1 ** 2).mean())}, out_path)


def test_two_rank_driver_matches_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    out = str(tmp_path / "result.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    r = torch.load(out)
    assert r["keys"]
    assert r["split_exact"] is True and r["same_as_plain"], r
    # q/k/v of the first block see identical inputs on both runs: only the order of the Hessian sum differs
    assert r["agree_first"] > 0.99, r
    # later layers: the activation quantiser's running-minimum tensor scale evolves per rank during the
    # calibration pass (as it does with the sequence order in the reference), so their Hessians differ
    # slightly and GPTQ's choices diverge; the models must still be equivalent
    assert r["agree"] > 0.6, r
    assert r["logit_diff"] < 0.05, r
