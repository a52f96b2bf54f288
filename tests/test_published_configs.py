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


LOOPVL_TEXT = {
    "model_type": "hrm_text", "architectures": ["HrmTextForCausalLM"], "dtype": "bfloat16", "hidden_act": "silu", "prefix_lm": True,
    "tie_word_embeddings": False, "attention_bias": False, "mlp_bias": False, "use_cache": False, "hidden_size": 256,
    "intermediate_size": 512, "vocab_size": 2048, "num_attention_heads": 2, "num_key_value_heads": 2, "head_dim": 128, "H_cycles": 2,
    "L_cycles": 3, "num_layers_per_stack": 2, "num_hidden_layers": 16, "max_position_embeddings": 128, "bos_token_id": 6,
    "eos_token_id": 11, "pad_token_id": 5, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "embedding_scale": 16.0,
    "attention_dropout": 0.0,
    "rope_parameters": {"rope_type": "yarn", "rope_theta": 10000, "factor": 2, "original_max_position_embeddings": 64,
                        "beta_fast": 32, "beta_slow": 1},
}
LOOPVL_CONFIG = {"model_type": "loopvl", "architectures": ["LoopVLForConditionalGeneration"], "format_version": 2,
                 "text_config": LOOPVL_TEXT, "loopvl_config": {"language": {k: LOOPVL_TEXT[k] for k in ("hidden_size", "num_attention_heads", "H_cycles")}},
                 "vision_config": {"model_type": "penguinvl_vision_encoder"}}


def test_loopvl_text_config_and_checkpoint(tmp_path):
    from flyingfish_b200.config import loop_tiny
    spec = spec_from_hf_config(LOOPVL_CONFIG, "loop-test")
    tiny = loop_tiny()
    assert spec.arch == "loop_vl" and spec.layers == 16 and spec.extra["hrm"]["layers_per_stack"] == 2
    assert spec.extra["hrm"]["yarn"] == {"factor": 2.0, "original_max": 64, "beta_fast": 32.0, "beta_slow": 1.0}
    assert spec.extra["hrm"]["embedding_scale"] == 16.0 and spec.eos_token_id == 11 and spec.max_position == 128
    assert (spec.hidden, spec.heads, spec.ffn, spec.vocab) == (tiny.hidden, tiny.heads, tiny.ffn, tiny.vocab)
    bad = json.loads(json.dumps(LOOPVL_CONFIG))
    bad["text_config"]["num_hidden_layers"] = 12
    with pytest.raises(ConfigError):
        spec_from_hf_config(bad, "x")
    bad = json.loads(json.dumps(LOOPVL_CONFIG))
    bad["loopvl_config"]["language"]["H_cycles"] = 3
    with pytest.raises(ConfigError):
        spec_from_hf_config(bad, "x")
    g = torch.Generator().manual_seed(1)
    h, f = spec.hidden, spec.ffn
    tensors = {"language_model.model.embed_tokens.weight": torch.randn(spec.vocab, h, generator=g) * 0.05,
               "language_model.lm_head.weight": torch.randn(spec.vocab, h, generator=g) * 0.05,
               "language_model.model.z_L_init": torch.randn(h, generator=g) * 0.05,
               "projector.fc1.bias": torch.zeros(8)}                         # vision-side tensors are left alone
    for stack in ("L", "H"):
        for i in range(2):
            p = f"language_model.model.{stack}_module.layers.{i}"
            for r in ("q", "k", "v", "o", "gate"):
                tensors[f"{p}.self_attn.{r}_proj.weight"] = torch.randn(h, h, generator=g) * 0.05
            tensors[f"{p}.mlp.gate_proj.weight"] = torch.randn(f, h, generator=g) * 0.05
            tensors[f"{p}.mlp.up_proj.weight"] = torch.randn(f, h, generator=g) * 0.05
            tensors[f"{p}.mlp.down_proj.weight"] = torch.randn(h, f, generator=g) * 0.05
    tensors = {k: v.to(torch.bfloat16) for k, v in tensors.items()}
    d = tmp_path / "loopvl"
    save_decoder_checkpoint(d, spec, tensors, LOOPVL_CONFIG)
    model = Model.load(str(d), Settings(capacity=128, max_batch=2, graph=False), device="cpu")
    w = model.engine.model.w
    assert torch.equal(w.embed.cpu(), tensors["language_model.model.embed_tokens.weight"])
    assert torch.equal(w.layers[0].wqkv[:h].cpu(), tensors["language_model.model.L_module.layers.0.self_attn.q_proj.weight"])
    assert torch.equal(w.layers[2].wo.cpu(), tensors["language_model.model.H_module.layers.0.self_attn.o_proj.weight"])
    ids = [6, 20, 21, 22, 23]
    first = model.prefill(ids)
    assert first == model.prefill(ids) and isinstance(model.decode(), int)
    del tensors["language_model.model.z_L_init"]
    d2 = tmp_path / "loopvl2"
    save_decoder_checkpoint(d2, spec, tensors, LOOPVL_CONFIG)
    with pytest.raises(CheckpointError):
        Model.load(str(d2), Settings(capacity=128, max_batch=2, graph=False), device="cpu")
