"""The tiny model and synthetic per-layer export entries shared by the export tests and by the script
that lists what the reference's exporter writes for them (tests/golden/make_export_listing.py)."""
import types

import torch

CASES = ("realquant_nvfp", "pseudoquant_mxfp_tied")
LINEARS = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
           "mlp.up_proj", "mlp.down_proj"]


def tiny_llama(tie: bool):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=160, max_position_embeddings=128, tie_word_embeddings=tie)
    model = LlamaForCausalLM(cfg).to(dtype=torch.bfloat16).eval()
    model.config.use_cache = False
    return model


def build(case: str):
    """(model, quantized_state_dict, non_quantized_state_dict, args) with seeded contents."""
    real = case.startswith("realquant")
    nv = "nvfp" in case
    model = tiny_llama(tie=case.endswith("tied"))
    g = torch.Generator().manual_seed(11)
    group, hg = (16 if nv else 32), 128
    quantized = {}
    for b, block in enumerate(model.model.layers):
        for name in LINEARS:
            lin = block.get_submodule(name)
            n, k = lin.out_features, lin.in_features
            had = torch.eye(hg, dtype=torch.bfloat16)
            entry = {}
            if real:
                entry["qweight"] = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g)
                entry["scales"] = torch.randint(1, 120, (n, k // group), dtype=torch.uint8, generator=g).view(
                    torch.float8_e4m3fn if nv else torch.float8_e8m0fnu)
            else:
                entry["dqweight"] = torch.randn(n, k, generator=g).to(torch.bfloat16)
            entry["forward_hadamard_matrix"] = had
            entry["backward_hadamard_matrix"] = had.clone()
            entry["weight_global_scale"] = torch.tensor([3.0 + b])
            entry["act_global_scale"] = torch.tensor([5.0])
            quantized[f"model.layers.{b}.{name}"] = entry
    # one block tensor overridden from outside, as the block-wise fine-tuning path of the reference does
    non_quantized = {"model.layers.1.input_layernorm.weight": torch.full((256,), 0.5, dtype=torch.bfloat16)}
    args = types.SimpleNamespace(save_path=None, max_shard_size=300_000, hadamard_group_size=hg,
                                 format="nvfp" if nv else "mxfp",
                                 export_quantized_model="realquant" if real else "pseudoquant")
    return model, quantized, non_quantized, args
