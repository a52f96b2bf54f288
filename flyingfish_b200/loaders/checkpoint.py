"""Checkpoint loading: expected-tensor manifests per architecture, load policies, assembly of
the fused / sharded weights from a mapped safetensors directory.

``manifest(spec)`` lists every tensor a decoder of that geometry must ship, with shape and dtype
class; ``audit`` compares it with what the directory holds and rejects missing tensors, shape
mismatches and unexpected extras (the reference's per-architecture manifests,
src/checkpoint.rs:3951-4008, 5857-6153, exercised by its contract tests). Quantised checkpoints
carry their scale tensors (``weight_scale_inv`` for block FP8, ``weight_scale`` /
``weight_scale_2`` for NVFP4) which are part of the manifest.
"""
from __future__ import annotations

import enum
import json
from pathlib import Path

import torch

from ..config import ModelSpec, read_model_spec
from ..models.weights import DTYPES, ModelWeights, TPInfo, build_decoder_weights
from .safetensors_io import CheckpointError, MappedCheckpoint


class LoadPolicy(enum.Enum):
    TEXT_ONLY = "text"
    ALL = "all"


def _linear_entries(name: str, out_f: int, in_f: int, fmt: str) -> dict[str, tuple[tuple[int, ...], str]]:
    if fmt == "fp8_block":
        return {name + ".weight": ((out_f, in_f), "fp8"),
                name + ".weight_scale_inv": (((out_f + 127) // 128, (in_f + 127) // 128), "f32")}
    if fmt == "nvfp4":
        return {name + ".weight": ((out_f, in_f // 2), "u8"), name + ".weight_scale": ((out_f, in_f // 16), "fp8"),
                name + ".weight_scale_2": ((), "f32")}
    return {name + ".weight": ((out_f, in_f), "float")}


def manifest(spec: ModelSpec, policy: LoadPolicy = LoadPolicy.TEXT_ONLY) -> dict[str, tuple[tuple[int, ...], str]]:
    """name -> (shape, dtype class in {float, f32, fp8, u8})."""
    m: dict[str, tuple[tuple[int, ...], str]] = {}
    h, d = spec.hidden, spec.head_dim
    m["model.embed_tokens.weight"] = ((spec.vocab, h), "float")
    m["model.norm.weight"] = ((h,), "float")
    if not spec.tie_embeddings:
        m["lm_head.weight"] = ((spec.vocab, h), "float")
    lf = spec.linear_format
    n_layers = spec.layers + spec.mtp_layers
    for i in range(n_layers):
        p = f"model.layers.{i}."
        m[p + "input_layernorm.weight"] = ((h,), "float")
        m[p + "post_attention_layernorm.weight"] = ((h,), "float")
        if spec.mla is not None:
            a = spec.mla
            qk = a.qk_nope_dim + a.qk_rope_dim
            if a.q_lora_rank:
                m.update(_linear_entries(p + "self_attn.q_a_proj", a.q_lora_rank, h, lf))
                m[p + "self_attn.q_a_layernorm.weight"] = ((a.q_lora_rank,), "float")
                m.update(_linear_entries(p + "self_attn.q_b_proj", spec.heads * qk, a.q_lora_rank, lf))
            else:
                m.update(_linear_entries(p + "self_attn.q_proj", spec.heads * qk, h, lf))
            m.update(_linear_entries(p + "self_attn.kv_a_proj_with_mqa", a.kv_lora_rank + a.qk_rope_dim, h, lf))
            m[p + "self_attn.kv_a_layernorm.weight"] = ((a.kv_lora_rank,), "float")
            m.update(_linear_entries(p + "self_attn.kv_b_proj", spec.heads * (a.qk_nope_dim + a.v_head_dim),
                                     a.kv_lora_rank, lf))
            m.update(_linear_entries(p + "self_attn.o_proj", h, spec.heads * a.v_head_dim, lf))
        else:
            m.update(_linear_entries(p + "self_attn.q_proj", spec.q_dim, h, lf))
            m.update(_linear_entries(p + "self_attn.k_proj", spec.kv_dim, h, lf))
            m.update(_linear_entries(p + "self_attn.v_proj", spec.kv_dim, h, lf))
            m.update(_linear_entries(p + "self_attn.o_proj", h, spec.q_dim, lf))
            if spec.qk_norm:
                m[p + "self_attn.q_norm.weight"] = ((d,), "float")
                m[p + "self_attn.k_norm.weight"] = ((d,), "float")
        moe = spec.moe
        is_moe = moe is not None and i >= moe.first_dense_layers
        if not is_moe:
            f = moe.dense_ffn if (moe is not None and moe.dense_ffn) else spec.ffn
            for nm, (o, k) in {"gate_proj": (f, h), "up_proj": (f, h), "down_proj": (h, f)}.items():
                m.update(_linear_entries(p + "mlp." + nm, o, k, lf))
        else:
            m[p + "mlp.gate.weight"] = ((moe.num_experts, h), "float")
            if moe.score == "noaux":
                m[p + "mlp.gate.e_score_correction_bias"] = ((moe.num_experts,), "f32")
            ef = moe.expert_format
            f = moe.expert_ffn
            for e in range(moe.num_experts):
                q = p + f"mlp.experts.{e}."
                for nm, (o, k) in {"gate_proj": (f, h), "up_proj": (f, h), "down_proj": (h, f)}.items():
                    m.update(_linear_entries(q + nm, o, k, ef))
            if moe.n_shared:
                sf = moe.shared_ffn
                for nm, (o, k) in {"gate_proj": (sf, h), "up_proj": (sf, h), "down_proj": (h, sf)}.items():
                    m.update(_linear_entries(p + "mlp.shared_experts." + nm, o, k, lf))
        if spec.arch == "flint":
            m[p + "self_attn.softmax_offset"] = ((spec.heads,), "float")
        if i >= spec.layers:   # MTP module extras
            m[p + "enorm.weight"] = ((h,), "float")
            m[p + "hnorm.weight"] = ((h,), "float")
            m[p + "eh_proj.weight"] = ((h, 2 * h), "float")
            m[p + "shared_head.norm.weight"] = ((h,), "float")
    if spec.arch == "flint":
        # published Flint checkpoints name the shared expert in the singular
        m = {k.replace(".mlp.shared_experts.", ".mlp.shared_expert."): v for k, v in m.items()}
    return m


def published_name(spec: ModelSpec, name: str) -> str:
    """The tensor name a published checkpoint of ``spec.arch`` uses for the canonical ``name``."""
    if spec.arch == "flint":
        return name.replace(".mlp.shared_experts.", ".mlp.shared_expert.")
    return name


_CLASS = {"float": ("BF16", "F16", "F32"), "f32": ("F32",), "fp8": ("F8_E4M3",), "u8": ("U8",)}


def audit(ckpt: MappedCheckpoint, spec: ModelSpec, allow_extra: tuple[str, ...] = ("rotary_emb.inv_freq",)) -> None:
    """Raise ``CheckpointError`` unless the directory holds exactly the manifest."""
    exp = manifest(spec)
    have = set(ckpt.names())
    missing = sorted(set(exp) - have)
    if missing:
        raise CheckpointError(f"checkpoint is missing {len(missing)} tensors, e.g. {missing[:3]}")
    for name, (shape, cls) in exp.items():
        info = ckpt.info(name)
        if tuple(info.shape) != tuple(shape):
            raise CheckpointError(f"{name}: shape {tuple(info.shape)} != expected {tuple(shape)}")
        if info.dtype not in _CLASS[cls]:
            raise CheckpointError(f"{name}: dtype {info.dtype} not allowed here ({cls})")
    vision = ("visual.", "model.visual.") if spec.extra.get("vision") else ()
    extra = sorted(n for n in have - set(exp)
                   if not any(n.endswith(a) for a in allow_extra) and not n.startswith(vision or ("\0",)))
    if extra:
        raise CheckpointError(f"checkpoint holds {len(extra)} unexpected tensors, e.g. {extra[:3]}")


def load_prefixed_tensors(model_dir: str | Path, prefixes: tuple[str, ...]) -> dict[str, torch.Tensor]:
    """All tensors whose name starts with one of ``prefixes`` (first match), keyed without the prefix -- the
    vision tower of a vision-language checkpoint lives under ``visual.``."""
    ck = MappedCheckpoint(model_dir)
    try:
        out: dict[str, torch.Tensor] = {}
        for n in ck.names():
            for pre in prefixes:
                if n.startswith(pre):
                    out.setdefault(n[len(pre):], ck.tensor(n).clone())
                    break
        if not out:
            raise CheckpointError(f"no tensors under {prefixes}")
        return out
    finally:
        ck.close()


def has_mtp_component(model_dir: str | Path) -> bool:
    """True when the checkpoint ships a multi-token-prediction module (probe by tensor name, like
    the reference's ``checkpoint::has_mtp_component``)."""
    ck = MappedCheckpoint(model_dir)
    try:
        return any(".enorm.weight" in n or n.startswith("mtp.") for n in ck.names())
    finally:
        ck.close()


def inspect_checkpoint(model_dir: str | Path) -> dict:
    ck = MappedCheckpoint(model_dir)
    try:
        by_dtype: dict[str, int] = {}
        total = 0
        for n in ck.names():
            i = ck.info(n)
            by_dtype[i.dtype] = by_dtype.get(i.dtype, 0) + i.nbytes
            total += i.nbytes
        return {"tensors": len(ck.names()), "bytes": total, "bytes_by_dtype": by_dtype, "shards": len(ck.files),
                "mtp": any(".enorm.weight" in n for n in ck.names())}
    finally:
        ck.close()


def load_decoder_weights(model_dir: str | Path, spec: ModelSpec | None, device: torch.device | str,
                         tp: TPInfo | None = None, ep: TPInfo | None = None, strict: bool = True) -> ModelWeights:
    """Map the directory, audit it against the manifest and assemble the fused weights on
    ``device``. 16/32-bit float checkpoints are cast to the model's compute dtype; block-FP8 and
    NVFP4 linears are dequantised to BF16 here when the model runs BF16 kernels for them."""
    model_dir = Path(model_dir)
    spec = spec or read_model_spec(model_dir)
    ck = MappedCheckpoint(model_dir)
    if strict:
        audit(ck, spec)
    device = torch.device(device)
    dtype = DTYPES["bf16" if spec.dtype == "f16" and device.type == "cuda" else spec.dtype]

    def source(name: str, shape: tuple[int, ...]) -> torch.Tensor:
        name = published_name(spec, name)
        if not ck.has(name):
            raise CheckpointError(f"missing tensor {name}")
        info = ck.info(name)
        if info.dtype == "F8_E4M3":
            from . import quant
            codes = ck.tensor(name).view(torch.uint8)
            scale = ck.tensor(name + "_scale_inv").to(torch.float32)
            return quant.dequantize_fp8_block(codes, scale, dtype=dtype).to(device)
        if info.dtype == "U8" and ck.has(name + "_scale"):
            from . import quant
            t = quant.dequantize_nvfp4(ck.tensor(name), ck.tensor(name + "_scale").view(torch.uint8),
                                       ck.tensor(name + "_scale_2").to(torch.float32), dtype)
            return t.to(device)
        t = ck.tensor(name)
        if tuple(t.shape) != tuple(shape):
            raise CheckpointError(f"{name}: shape {tuple(t.shape)} != expected {tuple(shape)}")
        return t.to(device=device, dtype=dtype)

    try:
        w = build_decoder_weights(spec, source, device, tp, ep)
        if spec.moe is not None and spec.moe.score == "noaux":
            for i, lw in enumerate(w.layers):
                nm = f"model.layers.{i}.mlp.gate.e_score_correction_bias"
                if lw.router is not None and ck.has(nm):
                    lw.router_bias = ck.tensor(nm).to(device=device, dtype=torch.float32)
        if spec.arch == "flint":
            # the learnable soft-max offsets ride along for the model class (one logit per query head and layer)
            w.extra["state"] = {f"model.layers.{i}.self_attn.sinks": ck.tensor(f"model.layers.{i}.self_attn.softmax_offset").float().clone()
                                for i in range(spec.layers)}
        return w
    finally:
        ck.close()


def checkpoint_source(model_dir: str | Path, spec: ModelSpec, device: torch.device | str):
    """(source, close): ``source(name, shape)`` reads one 16/32-bit float tensor of the directory, checks its shape and
    casts it to the model's compute dtype on ``device`` -- for model classes that assemble their own weight sets."""
    ck = MappedCheckpoint(Path(model_dir))
    device = torch.device(device)
    dtype = DTYPES["bf16" if spec.dtype == "f16" and device.type == "cuda" else spec.dtype]

    def source(name: str, shape: tuple[int, ...]) -> torch.Tensor:
        if not ck.has(name):
            raise CheckpointError(f"missing tensor {name}")
        t = ck.tensor(name)
        if tuple(t.shape) != tuple(shape):
            raise CheckpointError(f"{name}: shape {tuple(t.shape)} != expected {tuple(shape)}")
        if ck.info(name).dtype not in ("BF16", "F16", "F32"):
            raise CheckpointError(f"{name}: dtype {ck.info(name).dtype} is not a float tensor")
        return t.to(device=device, dtype=dtype)
    return source, ck.close


def save_decoder_checkpoint(model_dir: str | Path, spec: ModelSpec, tensors: dict[str, torch.Tensor],
                            hf_config: dict, shards: int = 1) -> None:
    """Write a model directory (config.json + safetensors, optionally sharded with an index) --
    used by tests and by ``ff`` tools that export synthetic checkpoints."""
    from .safetensors_io import save_safetensors
    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=False)
    (d / "config.json").write_text(json.dumps(hf_config))
    names = sorted(tensors)
    if shards == 1:
        save_safetensors(d / "model.safetensors", tensors)
        return
    wm = {}
    for s in range(shards):
        part = {n: tensors[n] for n in names[s::shards]}
        fname = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        save_safetensors(d / fname, part)
        wm.update({n: fname for n in part})
    (d / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wm}))
