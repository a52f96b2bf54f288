"""Checkpoint formats: safetensors audit, manifests, sharded directories, FP8/NVFP4 checkpoints,
GGUF Q4_0 -- all on synthetic files written to a temp dir."""
import json
import struct

import pytest
import torch

from flyingfish_b200.config import named_shape, spec_from_hf_config
from flyingfish_b200.loaders import quant
from flyingfish_b200.loaders.checkpoint import (audit, has_mtp_component, inspect_checkpoint, load_decoder_weights,
                                                manifest, save_decoder_checkpoint)
from flyingfish_b200.loaders.gguf import GgufError, GgufFile, T_F32, T_Q4_0, q4_0_dequant, q4_0_quant, write_gguf
from flyingfish_b200.loaders.safetensors_io import CheckpointError, MappedCheckpoint, SafetensorsFile, save_safetensors

HF_TINY = {"architectures": ["LlamaForCausalLM"], "hidden_size": 512, "num_attention_heads": 4, "num_key_value_heads": 1,
           "head_dim": 128, "intermediate_size": 1024, "num_hidden_layers": 2, "vocab_size": 2048, "rope_theta": 500000.0,
           "rms_norm_eps": 1e-5, "torch_dtype": "bfloat16", "hidden_act": "silu"}


def _tensors(spec, seed=0, fmt=None):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, cls) in manifest(spec).items():
        if cls == "float":
            t = (torch.ones(shape) if name.endswith("norm.weight") else torch.randn(shape, generator=g) * 0.02)
            out[name] = t.to(torch.bfloat16)
        elif cls == "f32":
            out[name] = torch.rand(shape, generator=g) + 0.5
    return out


def test_roundtrip_and_model_equivalence(tmp_path):
    from flyingfish_b200.api import Model, generate_plain
    from flyingfish_b200.config import Settings
    spec = spec_from_hf_config(HF_TINY, "tiny")
    tensors = _tensors(spec)
    for shards, name in ((1, "single"), (3, "sharded")):
        d = tmp_path / name
        save_decoder_checkpoint(d, spec, tensors, HF_TINY, shards=shards)
        ck = MappedCheckpoint(d)
        audit(ck, spec)
        assert len(ck.names()) == len(tensors)
        assert torch.equal(ck.tensor("model.layers.1.mlp.up_proj.weight"), tensors["model.layers.1.mlp.up_proj.weight"])
        ck.close()
        m = Model.load(str(d), Settings(capacity=128, max_batch=2, graph=False), device="cpu")
        out = generate_plain(m, [1, 2, 3, 4, 5], 4, ignore_eos=True).ids
        assert len(out) == 4
        info = inspect_checkpoint(d)
        assert info["tensors"] == len(tensors) and info["shards"] == shards and not info["mtp"]
    assert not has_mtp_component(tmp_path / "single")


def test_manifest_rejects_mutants(tmp_path):
    spec = spec_from_hf_config(HF_TINY, "tiny")
    base = _tensors(spec)
    def write(name, tensors):
        d = tmp_path / name
        save_decoder_checkpoint(d, spec, tensors, HF_TINY)
        return MappedCheckpoint(d)
    t = dict(base); del t["model.layers.0.self_attn.k_proj.weight"]
    with pytest.raises(CheckpointError, match="missing"):
        audit(write("missing", t), spec)
    t = dict(base); t["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(1023, 512, dtype=torch.bfloat16)
    with pytest.raises(CheckpointError, match="shape"):
        audit(write("shape", t), spec)
    t = dict(base); t["model.layers.7.rogue.weight"] = torch.zeros(4, dtype=torch.bfloat16)
    with pytest.raises(CheckpointError, match="unexpected"):
        audit(write("extra", t), spec)
    t = dict(base); t["model.norm.weight"] = torch.zeros(512, dtype=torch.int32)
    with pytest.raises(CheckpointError, match="dtype"):
        audit(write("dtype", t), spec)


def test_header_audit_detects_holes_overlaps_and_escapes(tmp_path):
    good = tmp_path / "good.safetensors"
    save_safetensors(good, {"a": torch.arange(4, dtype=torch.float32), "b": torch.ones(2, 2, dtype=torch.bfloat16)})
    f = SafetensorsFile(good)
    assert f.tensor("a").tolist() == [0, 1, 2, 3] and f.byte_range("b")[1] - f.byte_range("b")[0] == 8
    f.close()

    def craft(name, header, data=b"\0" * 32):
        hj = json.dumps(header).encode()
        p = tmp_path / name
        p.write_bytes(struct.pack("<Q", len(hj)) + hj + data)
        return p
    with pytest.raises(CheckpointError, match="hole"):
        SafetensorsFile(craft("hole.safetensors", {"a": {"dtype": "F32", "shape": [4], "data_offsets": [16, 32]}}))
    with pytest.raises(CheckpointError, match="overlap"):
        SafetensorsFile(craft("ovl.safetensors", {"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]},
                                                  "b": {"dtype": "F32", "shape": [4], "data_offsets": [8, 24]}}))
    with pytest.raises(CheckpointError, match="bytes"):
        SafetensorsFile(craft("size.safetensors", {"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 32]}}))
    with pytest.raises(CheckpointError, match="cover"):
        SafetensorsFile(craft("tail.safetensors", {"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}))
    # sharded index pointing outside the model directory
    d = tmp_path / "models_dir"; d.mkdir()
    outside = tmp_path / "outside.safetensors"
    save_safetensors(outside, {"x": torch.zeros(1)})
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "../outside.safetensors"}}))
    with pytest.raises(CheckpointError, match="outside"):
        MappedCheckpoint(d)


def test_fp8_block_checkpoint_loads_dequantised(tmp_path):
    cfg = dict(HF_TINY, quantization_config={"quant_method": "fp8", "weight_block_size": [128, 128]})
    spec = spec_from_hf_config(cfg, "tiny-fp8")
    assert spec.linear_format == "fp8_block"
    g = torch.Generator().manual_seed(1)
    tensors, dense = {}, {}
    for name, (shape, cls) in manifest(spec).items():
        if cls == "fp8":
            w = torch.randn(shape, generator=g) * 0.02
            codes, scale = quant.quantize_fp8_block_weight(w)
            tensors[name] = codes.view(torch.float8_e4m3fn)
            tensors[name + "_scale_inv"] = scale
            dense[name] = quant.dequantize_fp8_block(codes, scale)
        elif cls == "float":
            tensors[name] = (torch.ones(shape) if name.endswith("norm.weight") else torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16)
    d = tmp_path / "fp8"
    save_decoder_checkpoint(d, spec, tensors, cfg)
    w = load_decoder_weights(d, spec, "cpu")
    q0 = dense["model.layers.0.self_attn.q_proj.weight"]
    assert torch.equal(w.layers[0].wqkv[: q0.shape[0]], q0)


def test_mtp_probe(tmp_path):
    cfg = dict(HF_TINY, num_nextn_predict_layers=1)
    spec = spec_from_hf_config(cfg, "tiny-mtp")
    assert spec.mtp_layers == 1
    d = tmp_path / "mtp"
    save_decoder_checkpoint(d, spec, _tensors(spec), cfg)
    assert has_mtp_component(d)
    audit(MappedCheckpoint(d), spec)


def test_gguf_q4_0(tmp_path):
    g = torch.Generator().manual_seed(2)
    w = torch.randn(8, 64, generator=g)
    p = tmp_path / "m.gguf"
    write_gguf(p, {"general.architecture": "llama", "llama.block_count": 2, "tokenizer.ggml.tokens": ["a", "b"]},
               {"blk.0.w": (w, T_Q4_0), "norm": (torch.ones(64), T_F32)})
    f = GgufFile(p)
    assert f.metadata["general.architecture"] == "llama" and f.metadata["llama.block_count"] == 2
    assert f.metadata["tokenizer.ggml.tokens"] == ["a", "b"]
    assert f.tensors["blk.0.w"].shape == (8, 64) and f.tensors["blk.0.w"].nbytes == 8 * 2 * 18
    deq = f.tensor("blk.0.w", torch.float32)
    assert (deq - w).abs().max() <= w.abs().max() / 8 + 1e-3
    assert torch.equal(f.tensor("norm", torch.float32), torch.ones(64))
    assert torch.equal(q4_0_dequant(q4_0_quant(w), (8, 64), torch.float32), deq)
    f.close()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUX" + b"\0" * 64)
    with pytest.raises(GgufError):
        GgufFile(bad)
    trunc = tmp_path / "trunc.gguf"
    trunc.write_bytes(p.read_bytes()[:-40])
    with pytest.raises(GgufError):
        GgufFile(trunc)
