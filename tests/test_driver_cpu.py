"""Host logic of the model-level drivers that needs no GPU: rank planning, Hessian-update batching,
block replay with several sequences per call."""
import types

import torch

from fpq_b200.quantization import driver


LLAMA_GROUPS = {"qkv": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"], "o": ["self_attn.o_proj"],
                "gate_up": ["mlp.gate_proj", "mlp.up_proj"], "down": ["mlp.down_proj"]}
LLAMA_COLS = {"qkv": 4096, "o": 4096, "gate_up": 4096, "down": 14336}


def test_plan_single_rank_keeps_everything_on_rank_zero():
    order, gown, lown = driver.plan_ranks(LLAMA_GROUPS, LLAMA_COLS, 1)
    assert order[0] == "down"
    assert set(gown.values()) == {0} and set(lown.values()) == {0}


def test_plan_spreads_chains_and_members():
    for ws in (2, 4, 8):
        order, gown, lown = driver.plan_ranks(LLAMA_GROUPS, LLAMA_COLS, ws)
        assert gown["down"] == 0                                  # the largest chain first
        assert len(set(gown.values())) == min(ws, 4)
        for g, names in LLAMA_GROUPS.items():
            assert lown[names[0]] == gown[g]                      # leaders stay with their chain
        assert all(0 <= r < ws for r in lown.values())
    _, gown, lown = driver.plan_ranks(LLAMA_GROUPS, LLAMA_COLS, 8)
    assert len(set(lown.values())) == 7                           # seven linears on seven ranks
    _, gown, lown = driver.plan_ranks(LLAMA_GROUPS, LLAMA_COLS, 4)
    assert lown["self_attn.k_proj"] == gown["qkv"]                # no idle rank: members stay


def test_hessian_sink_batches_updates():
    calls = []
    handle = types.SimpleNamespace(update=lambda x: calls.append(tuple(x.shape)))
    sink = driver._HessianSink(handle, tokens_per_update=3 * 16)
    for _ in range(7):
        sink(torch.zeros(1, 16, 8))
    sink.flush()
    assert calls == [(3, 16, 8), (3, 16, 8), (1, 16, 8)]
    calls.clear()
    sink(torch.zeros(1, 16, 8))
    sink(torch.zeros(1, 24, 8))          # a different sequence length flushes what is pending
    sink.flush()
    assert calls == [(1, 16, 8), (1, 24, 8)]


class _Scale(torch.nn.Module):
    def forward(self, hidden_states, factor=2.0):
        return (hidden_states * factor,)


def test_run_block_batches_and_writes_back():
    for batch in (1, 2, 5):
        args = types.SimpleNamespace(calibration_batch=batch, amp=False)
        xs = [torch.full((1, 4, 3), float(i)) for i in range(5)]
        input_args = [(x.clone(),) for x in xs]
        input_kwargs = [{"factor": 3.0} for _ in xs]
        driver._run_block(_Scale(), input_args, input_kwargs, "cpu", args, keep_outputs=True, offload_device="cpu")
        for i, (a,) in enumerate(input_args):
            assert torch.equal(a, xs[i] * 3.0)
        input_args = [() for _ in xs]
        input_kwargs = [{"hidden_states": x.clone(), "factor": 0.5} for x in xs]
        driver._run_block(_Scale(), input_args, input_kwargs, "cpu", args, keep_outputs=True, offload_device="cpu")
        for i, kw in enumerate(input_kwargs):
            assert torch.equal(kw["hidden_states"], xs[i] * 0.5)
