"""Published configuration files and tensor layouts of the newer decoder families load through ``Model.load``."""
import json

import pytest
import torch

from flyingfish_b200.api import Model
from flyingfish_b200.config import ConfigError, Settings, spec_from_hf_config
from flyingfish_b200.loaders.checkpoint import CheckpointError, manifest, save_decoder_checkpoint

FLINT_CONFIG = {
    "architectures": ["FlintForCausalLM"], "model_type": "flint", "attention_bias": False, "attention_dropout": 0.0,
    "bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0, "decoder_sparse_step": 1, "head_dim": 128, "hidden_act": "silu",
    "hidden_size": 256, "initializer_range": 0.02, "intermediate_size": 512,
    "layer_types": ["full_attention", "full_attention", "sliding_attention", "sliding_attention", "full_attention"],
    "max_position_embeddings": 4096, "mlp_only_layers": [0, 1], "moe_intermediate_size": 128, "norm_topk_prob": True,
    "num_attention_heads": 4, "num_experts": 8, "num_experts_per_tok": 2, "num_hidden_layers": 5, "num_key_value_heads": 1,
    "no_rope_layer_indices": [0, 1, 4], "output_router_logits": False, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
    "router_aux_loss_coef": 0.0005, "router_score_function": "sigmoid", "shared_expert_intermediate_size": 256,
    "sliding_window": 33, "softmax_type": "learnable", "tie_word_embeddings": False, "torch_dtype": "bfloat16",
    "use_cache": True, "use_sliding_window": True, "vocab_size": 512,
}


def test_flint_config_and_checkpoint(tmp_path):
    spec = spec_from_hf_config(FLINT_CONFIG, "flint-test")
    assert spec.arch == "flint" and spec.qk_norm and spec.extra["flint"] == {"window": 33, "no_rope_layers": [0, 1, 4]}
    assert (spec.moe.num_experts, spec.moe.top_k, spec.moe.score, spec.moe.first_dense_layers, spec.moe.shared_ffn) == (8, 2, "sigmoid", 2, 256)
    m = manifest(spec)
    assert "model.layers.2.mlp.shared_expert.up_proj.weight" in m and not any(".shared_experts." in k for k in m)
    assert m["model.layers.4.self_attn.softmax_offset"] == ((4,), "float") and "model.layers.2.mlp.experts.7.down_proj.weight" in m
    assert "model.layers.0.mlp.gate_proj.weight" in m and "model.layers.2.mlp.gate.weight" in m
    for bad in (dict(FLINT_CONFIG, router_score_function="softmax"), dict(FLINT_CONFIG, mlp_only_layers=[1]),
                dict(FLINT_CONFIG, layer_types=["sliding_attention"] * 5), dict(FLINT_CONFIG, no_rope_layer_indices=[7])):
        with pytest.raises(ConfigError):
            spec_from_hf_config(bad, "x")
    g = torch.Generator().manual_seed(0)
    tensors = {}
    for name, (shape, _) in m.items():
        t = torch.randn(*shape, generator=g) * 0.05
        if name.endswith("norm.weight"):
            t = t + 1.0
        tensors[name] = t.to(torch.bfloat16)
    d = tmp_path / "flint"
    save_decoder_checkpoint(d, spec, tensors, FLINT_CONFIG)
    model = Model.load(str(d), Settings(capacity=256, max_batch=2, graph=False), device="cpu")
    assert model.spec.arch == "flint"
    net = model.engine.model
    assert torch.equal(net.sinks[3].cpu(), tensors["model.layers.3.self_attn.softmax_offset"].float())
    ids = [5, 6, 7, 8, 9, 10]
    first = model.prefill(ids)
    assert first == model.prefill(ids) and isinstance(model.decode(), int)
    # the offsets are part of the model: other offsets, other logits
    other = dict(tensors)
    for i in range(5):
        other[f"model.layers.{i}.self_attn.softmax_offset"] = (tensors[f"model.layers.{i}.self_attn.softmax_offset"].float() + 4.0).to(torch.bfloat16)
    d2 = tmp_path / "flint2"
    save_decoder_checkpoint(d2, spec, other, FLINT_CONFIG)
    model2 = Model.load(str(d2), Settings(capacity=256, max_batch=2, graph=False), device="cpu")
    assert not torch.equal(model2.engine.model.sinks[0], net.sinks[0])
    # a checkpoint in the plural spelling is not a published Flint checkpoint
    wrong = {k.replace(".shared_expert.", ".shared_experts."): v for k, v in tensors.items()}
    d3 = tmp_path / "flint3"
    save_decoder_checkpoint(d3, spec, wrong, FLINT_CONFIG)
    with pytest.raises(CheckpointError):
        Model.load(str(d3), Settings(capacity=256, max_batch=2, graph=False), device="cpu")
