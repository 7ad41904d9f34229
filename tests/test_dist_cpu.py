"""World-size-2 gloo test of the multi-GPU partitioning logic (token-sharded Hessian + all-reduce,
row-sharded column loop + all-gather).  Runs on CPU tensors; the numeric callbacks are the oracle's,
so this checks the host logic only: the sharded run must reproduce the unsharded one."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world_size, port, tmpdir):
    for p in (ROOT, os.path.join(ROOT, "fp-quant_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world_size)
    try:
        from fpq_b200 import dist as fdist
        from oracle import fp4, gptq as ogptq
        from tests import inputs

        torch.set_num_threads(2)
        R, C, n_seq, T = 320, 256, 6, 128            # 320 rows -> slabs of 256 and 64 (multiples of 128)
        w = fp4.fwht_butterfly(inputs.normal_weight(R, C, seed=0, dtype=torch.float32), 128)
        xs = [fp4.fwht_butterfly(inputs.correlated_activations(T, C, seed=60 + i), 128) for i in range(n_seq)]

        def accumulate(H, x2d, alpha, beta):
            H.mul_(beta).add_(alpha * (x2d.float().t() @ x2d.float()))

        def column_loop(W, s, U, g):
            wq, codes = ogptq.gptq_column_loop(W, s, U, g, 128)
            return wq, fp4.pack_codes(codes)

        sh = fdist.ShardedLayerGPTQ(C, torch.device("cpu"))
        lo, hi = fdist.shard_bounds(n_seq, world_size, rank)
        for i in range(lo, hi):
            sh.update(xs[i].view(1, T, C), n_seq, accumulate)
        H = sh.finish_hessian()
        exact = ogptq.hessian_exact([x.view(1, T, C) for x in xs], n_seq)
        assert ((H.double() - exact).norm() / exact.norm()).item() < 1e-6

        gs = fp4.nvfp4_global_scale(w.abs().max())
        _, _, s = fp4.quantize(w, "nvfp4", gs)
        Hd = ogptq.prepare_hessian(H, w, 0.01)
        U, ok = ogptq.cholesky_inverse_upper(Hd)
        wq, codes = sh.quantize(w, s, U, 16, column_loop)
        wq_full, codes_full = ogptq.gptq_column_loop(w, s, U, 16, 128)
        assert torch.equal(wq, wq_full) and torch.equal(codes, fp4.pack_codes(codes_full))

        # helpers
        assert fdist.all_bounds(10, 3) == [(0, 4), (4, 7), (7, 10)]
        assert fdist.all_bounds(320, 2, 128) == [(0, 256), (256, 320)]
        assert fdist.all_bounds(128, 4, 128) == [(0, 128), (128, 128), (128, 128), (128, 128)]
        t = torch.tensor([float(rank + 1)])
        assert fdist.allreduce_min_(t.clone()).item() == 1.0
        assert fdist.allreduce_sum_(t.clone()).item() == sum(range(1, world_size + 1))
        for dst in range(world_size):       # the sum arrives on `dst`; nobody else may rely on its buffer
            r = fdist.reduce_sum_(t.clone(), dst)
            if rank == dst:
                assert r.item() == sum(range(1, world_size + 1))
        open(os.path.join(tmpdir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_sharded_gptq_matches_unsharded_on_two_gloo_ranks(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_shard_bounds_cover_everything():
    sys.path.insert(0, os.path.join(ROOT, "fp-quant_b200"))
    from fpq_b200 import dist as fdist

    for n in (0, 1, 7, 128, 1000, 14336):
        for ws in (1, 2, 3, 8):
            for mult in (1, 128):
                b = fdist.all_bounds(n, ws, mult)
                assert b[0][0] == 0 and b[-1][1] == n
                assert all(b[i][1] == b[i + 1][0] for i in range(ws - 1))
                assert all((lo % mult == 0) for lo, hi in b if lo < n)


@pytest.mark.parametrize("out_features,world_size,expect", [(1536, 8, False), (384, 2, False), (640, 4, False),
                                                             (2048, 8, True), (17408, 8, True), (512, 2, True)])
def test_fused_tensor_parallel_path_is_chosen_identically_on_all_ranks(out_features, world_size, expect):
    """The epilogue-push path of the column-parallel linear is a collective: either every rank takes it or none.
    Shares of uneven splits differ by 128 rows (1536 over 8 ranks: 256 x 4 + 128 x 4), so a rank-local test
    ("my slice has >= 256 rows") would split the ranks; the decision must come out of the split alone."""
    for p in (ROOT, os.path.join(ROOT, "fp-quant_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from fpq_b200 import dist as fdist
    from fpq_b200.fp_quant.module.tp_linear import fused_path_allowed

    verdict = fused_path_allowed(out_features, world_size)
    assert verdict == expect
    local = [hi - lo >= 256 for lo, hi in fdist.all_bounds(out_features, world_size, 128)]
    assert verdict == all(local)          # and it is the conjunction of what each rank would have said


def test_weighted_bounds_cover_everything_in_order():
    for p in (ROOT, os.path.join(ROOT, "fp-quant_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from fpq_b200 import dist as fdist

    for n, weights in ((128, [0.62] + [7.38 / 7] * 7), (128, [0.89, 1.11]), (6, [0.89, 1.11]), (3, [0.62] + [1.05] * 7),
                       (0, [1.0, 1.0]), (5, [1.0])):
        b = fdist.weighted_bounds(n, weights)
        assert len(b) == len(weights) and b[0][0] == 0 and b[-1][1] == n
        assert all(b[i][1] == b[i + 1][0] for i in range(len(b) - 1)) and all(hi >= lo for lo, hi in b)
    assert [hi - lo for lo, hi in fdist.weighted_bounds(128, [0.62] + [7.38 / 7] * 7)][0] == 10     # the tail owner's share


@pytest.mark.parametrize("world_size", [1, 2, 3, 4, 5, 6, 7, 8, 16])
def test_plan_ranks_invariants(world_size):
    """Every linear of a block gets exactly one rank; the chains of the distinct Hessians go to different ranks
    while there are enough (widest first, so the widest is rank 0's); a group's first linear stays with the
    rank that factors its Hessian; the others only move to ranks that run no chain."""
    from fpq_b200.quantization.driver import plan_ranks

    members = {"qkv": ["q_proj", "k_proj", "v_proj"], "o": ["o_proj"], "gate_up": ["gate_proj", "up_proj"], "down": ["down_proj"]}
    width = {"qkv": 4096, "o": 4096, "gate_up": 4096, "down": 14336}
    order, chain_rank, loop_rank = plan_ranks(members, width, world_size)
    assert order[0] == "down" and chain_rank["down"] == 0
    assert sorted(loop_rank) == sorted(n for names in members.values() for n in names)
    assert all(0 <= r < world_size for r in list(chain_rank.values()) + list(loop_rank.values()))
    if world_size >= 4:
        assert len(set(chain_rank.values())) == 4
    chain_ranks = set(chain_rank.values())
    for grp, names in members.items():
        assert loop_rank[names[0]] == chain_rank[grp]
        for n in names[1:]:
            assert loop_rank[n] == chain_rank[grp] or loop_rank[n] not in chain_ranks
    moved = [loop_rank[n] for grp, names in members.items() for n in names[1:] if loop_rank[n] != chain_rank[grp]]
    assert len(moved) == len(set(moved)) == min(3, max(0, world_size - 4))      # one idle rank per moved linear
