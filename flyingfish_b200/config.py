"""Model geometry and engine settings.

``ModelSpec`` is the normalised description of a decoder that the rest of the framework works
from (the counterpart of the reference's ``ModelSpec`` / ``Config``: src/model_spec.rs:8-104,
469-510; src/config.rs:5-104). It can be read from a Hugging Face ``config.json`` or taken from
the table of named benchmark shapes below. ``Settings`` carries the engine options of the CLI
(src/backend/mod.rs:196-224).
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any


@dataclass
class MoeSpec:
    num_experts: int
    top_k: int
    expert_ffn: int
    score: str = "softmax"            # softmax | sigmoid | noaux | sqrt_softplus
    n_shared: int = 0                 # shared experts (each of width shared_ffn)
    shared_ffn: int = 0
    n_groups: int = 1
    topk_groups: int = 1
    routed_scaling: float = 1.0
    renormalize: bool = True
    first_dense_layers: int = 0       # leading layers with a dense FFN
    dense_ffn: int = 0
    shared_gate: bool = False         # sigmoid gate on the shared expert (Qwen-style)
    expert_format: str = "bf16"       # bf16 | fp8_block | nvfp4


@dataclass
class MlaSpec:
    q_lora_rank: int
    kv_lora_rank: int
    qk_nope_dim: int
    qk_rope_dim: int
    v_head_dim: int


@dataclass
class ModelSpec:
    name: str
    arch: str                         # llama | qwen3 | qwen3_moe | deepseek_v3 | deepseek_v41 | glm5_next | flint | loop_vl | tiny_moe | qwen3_vl | embedding | diffusion_lm | qwen35_text | gemma
    layers: int
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rope_theta: float = 10000.0
    rms_eps: float = 1e-6
    dtype: str = "bf16"               # storage / compute dtype of dense weights
    linear_format: str = "bf16"       # bf16 | fp8_block | nvfp4
    tie_embeddings: bool = False
    qk_norm: bool = False
    swiglu_mode: int = 0
    max_position: int = 131072
    eos_token_id: int | None = None
    moe: MoeSpec | None = None
    mla: MlaSpec | None = None
    mtp_layers: int = 0               # multi-token-prediction heads shipped with the checkpoint
    extra: dict[str, Any] = field(default_factory=dict)

    @property
    def q_dim(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    def dense_param_count(self) -> int:
        per_layer = self.hidden * self.qkv_dim + self.q_dim * self.hidden + 3 * self.hidden * self.ffn + 2 * self.hidden
        return self.layers * per_layer + (1 if self.tie_embeddings else 2) * self.vocab * self.hidden + self.hidden

    def decode_weight_bytes(self) -> int:
        """Bytes of weights read by one decode step (embedding row gathers excluded, lm_head
        included) -- the numerator of the reference's decode roofline (src/bench.rs:137-160)."""
        per_layer = self.hidden * self.qkv_dim + self.q_dim * self.hidden + 3 * self.hidden * self.ffn + 2 * self.hidden
        return 2 * (self.layers * per_layer + self.vocab * self.hidden + self.hidden)

    def to_json(self) -> dict[str, Any]:
        return dataclasses.asdict(self)


# ------------------------------------------------------------------------------------------
# named shapes (the benchmark configurations; random-init, no checkpoint needed)
# ------------------------------------------------------------------------------------------
def tiny_moe() -> ModelSpec:
    return ModelSpec(
        name="tiny-moe", arch="tiny_moe", layers=2, hidden=256, heads=4, kv_heads=2, head_dim=64, ffn=512,
        vocab=1024, rope_theta=1e4, rms_eps=1e-6, dtype="fp32",
        moe=MoeSpec(num_experts=8, top_k=2, expert_ffn=512, score="softmax", n_shared=1, shared_ffn=512))


def tiny_llama() -> ModelSpec:
    """Small dense shape with the production head geometry (head_dim 128, GQA 4:1) for tests."""
    return ModelSpec(name="tiny-llama", arch="llama", layers=2, hidden=512, heads=4, kv_heads=1, head_dim=128,
                     ffn=1024, vocab=2048, rope_theta=5e5, rms_eps=1e-5)


def llama3_8b() -> ModelSpec:
    return ModelSpec(name="llama3-8b-shape", arch="llama", layers=32, hidden=4096, heads=32, kv_heads=8,
                     head_dim=128, ffn=14336, vocab=128256, rope_theta=5e5, rms_eps=1e-5)


def llama3_70b() -> ModelSpec:
    return ModelSpec(name="llama3-70b-shape", arch="llama", layers=80, hidden=8192, heads=64, kv_heads=8,
                     head_dim=128, ffn=28672, vocab=128256, rope_theta=5e5, rms_eps=1e-5)


def deepseek_v3() -> ModelSpec:
    return ModelSpec(
        name="deepseek-v3-shape", arch="deepseek_v3", layers=61, hidden=7168, heads=128, kv_heads=128, head_dim=128,
        ffn=18432, vocab=129280, rope_theta=1e4, rms_eps=1e-6, linear_format="fp8_block", mtp_layers=1,
        mla=MlaSpec(q_lora_rank=1536, kv_lora_rank=512, qk_nope_dim=128, qk_rope_dim=64, v_head_dim=128),
        moe=MoeSpec(num_experts=256, top_k=8, expert_ffn=2048, score="noaux", n_shared=1, shared_ffn=2048,
                    n_groups=8, topk_groups=4, routed_scaling=2.5, first_dense_layers=3, dense_ffn=18432,
                    expert_format="fp8_block"))


def deepseek_v3_tiny() -> ModelSpec:
    """Same structure as :func:`deepseek_v3` (MLA + grouped noaux routing + MTP head) at test size."""
    return ModelSpec(
        name="deepseek-v3-tiny", arch="deepseek_v3", layers=3, hidden=256, heads=4, kv_heads=4, head_dim=128,
        ffn=512, vocab=1024, rope_theta=1e4, rms_eps=1e-6, mtp_layers=1,
        mla=MlaSpec(q_lora_rank=96, kv_lora_rank=64, qk_nope_dim=32, qk_rope_dim=16, v_head_dim=32),
        moe=MoeSpec(num_experts=16, top_k=4, expert_ffn=128, score="noaux", n_shared=1, shared_ffn=128,
                    n_groups=4, topk_groups=2, routed_scaling=2.5, first_dense_layers=1, dense_ffn=512))


def deepseek_v3_mini() -> ModelSpec:
    """DeepSeek-V3 attention geometry (kv_lora 512, rope 64, nope 128, v 128) with a handful of
    heads and layers: the smallest shape the MLA CUDA kernel serves."""
    return ModelSpec(
        name="deepseek-v3-mini", arch="deepseek_v3", layers=2, hidden=512, heads=4, kv_heads=4, head_dim=128,
        ffn=1024, vocab=2048, rope_theta=1e4, rms_eps=1e-6,
        mla=MlaSpec(q_lora_rank=256, kv_lora_rank=512, qk_nope_dim=128, qk_rope_dim=64, v_head_dim=128),
        moe=MoeSpec(num_experts=16, top_k=4, expert_ffn=256, score="noaux", n_shared=1, shared_ffn=256,
                    n_groups=4, topk_groups=2, routed_scaling=2.5, first_dense_layers=1, dense_ffn=1024))


def deepseek_v3_fp8_mini() -> ModelSpec:
    """:func:`deepseek_v3_mini` with the published quantisation of DeepSeek-V3: every projection and expert as E4M3
    codes with 128x128 block scales (activations quantised 1x128 inside the linears), plus one MTP module."""
    s = deepseek_v3_mini()
    s.name, s.layers, s.linear_format, s.mtp_layers = "deepseek-v3-fp8-mini", 3, "fp8_block", 1
    s.moe.expert_format = "fp8_block"
    return s


def qwen3_moe_235b() -> ModelSpec:
    return ModelSpec(
        name="qwen3-moe-235b-shape", arch="qwen3_moe", layers=94, hidden=4096, heads=64, kv_heads=4, head_dim=128,
        ffn=12288, vocab=151936, rope_theta=1e6, rms_eps=1e-6, qk_norm=True,
        moe=MoeSpec(num_experts=128, top_k=8, expert_ffn=1536, score="softmax", expert_format="nvfp4"))


def qwen3_moe_tiny() -> ModelSpec:
    return ModelSpec(
        name="qwen3-moe-tiny", arch="qwen3_moe", layers=2, hidden=512, heads=4, kv_heads=1, head_dim=128, ffn=1024,
        vocab=2048, rope_theta=1e6, rms_eps=1e-6, qk_norm=True,
        moe=MoeSpec(num_experts=16, top_k=4, expert_ffn=256, score="softmax"))


def tiny_vl() -> ModelSpec:
    """Small vision-language shape: the tiny dense decoder plus a vision tower (``extra["vision"]`` holds the
    fields of ``models.vision.VisionSpec``; ``extra["image_token_id"]`` marks the rows the tower fills)."""
    spec = tiny_llama()
    spec.name, spec.arch = "tiny-vl", "qwen3_vl"
    spec.extra = {"image_token_id": 2047,
                  "vision": {"hidden": 256, "heads": 2, "depth": 2, "intermediate": 512, "patch": 16, "temporal": 2,
                             "merge": 2, "out_hidden": spec.hidden, "pos_side": 16}}
    return spec


def tiny_minicpm() -> ModelSpec:
    """Small sliced-image vision-language shape: the tiny dense decoder plus a MiniCPM-V style tower
    (``extra["vision"]``: ``kind`` "minicpm" and the fields of ``models.minicpm_vision.MiniCpmVisionSpec``); a large
    image is shown whole and as tiles, each view wrapped in marker tokens."""
    spec = tiny_llama()
    spec.name, spec.arch = "tiny-minicpm", "qwen3_vl"
    spec.extra = {"image_token_id": 2047, "image_start_id": 2040, "image_end_id": 2041, "slice_start_id": 2042, "slice_end_id": 2043,
                  "newline_id": 10, "max_slices": 4, "slice_scale": 32,
                  "vision": {"kind": "minicpm", "hidden": 64, "heads": 2, "depth": 3, "intermediate": 96, "patch": 2, "channels": 3,
                             "image_size": 32, "insert_layer": 0, "out_hidden": spec.hidden}}
    return spec


def tiny_embed() -> ModelSpec:
    """Small bidirectional text encoder (embedding model): mean pooling, optional dense head, L2 normalisation."""
    spec = tiny_llama()
    spec.name, spec.arch = "tiny-embed", "embedding"
    spec.extra = {"bidirectional": True, "embed_dense": [1024, 256]}
    return spec


def tiny_diffusion() -> ModelSpec:
    """Small masked-diffusion language model: a bidirectional decoder stack that denoises a canvas of mask tokens."""
    spec = tiny_llama()
    spec.name, spec.arch = "tiny-diffusion", "diffusion_lm"
    spec.extra = {"bidirectional": True, "mask_token_id": 2046}
    return spec


def tiny_hybrid() -> ModelSpec:
    """Small hybrid shape: gated-delta-net mixers with full attention in every fourth layer."""
    spec = tiny_llama()
    spec.name, spec.arch, spec.layers = "tiny-hybrid", "qwen35_text", 4
    spec.extra = {"gdn": {"v_heads": 4, "k_heads": 2, "full_attention_interval": 4}}
    return spec


def qwen3_moe_fp4_tiny() -> ModelSpec:
    """The tiny MoE shape with NVFP4 experts (decode reads the packed experts, prefill their BF16 expansion)."""
    spec = qwen3_moe_tiny()
    spec.name = "qwen3-moe-fp4-tiny"
    spec.moe.expert_format = "nvfp4"
    return spec


def tiny_gemma() -> ModelSpec:
    """Small Gemma-layout shape: five local layers (window 48) per global layer, tanh-GELU gate, soft-capped logits."""
    spec = tiny_llama()
    spec.name, spec.arch, spec.layers = "tiny-gemma", "gemma", 6
    spec.qk_norm, spec.swiglu_mode, spec.tie_embeddings, spec.rope_theta = True, 2, True, 1e6
    spec.extra = {"gemma": {"window": 48, "global_every": 6, "local_rope_theta": 1e4, "final_softcap": 30.0}}
    return spec


def deepseek_v41_tiny() -> ModelSpec:
    """Small DeepSeek-V4.1-style shape: four hyper-connection streams, a latent mixer with an FP8 window ring (window 32),
    one top-k sparse layer with a pooled indexer, n-gram memory rows in the first layer, shared + routed experts with
    square-root-soft-plus routing after a dense first layer."""
    return ModelSpec(
        name="deepseek-v41-tiny", arch="deepseek_v41", layers=3, hidden=256, heads=4, kv_heads=1, head_dim=128, ffn=512,
        vocab=2048, rope_theta=1e4, rms_eps=1e-6,
        moe=MoeSpec(num_experts=8, top_k=2, expert_ffn=128, score="sqrt_softplus", n_shared=1, shared_ffn=128,
                    routed_scaling=1.5, first_dense_layers=1, dense_ffn=512),
        extra={"v41": {"hc_mult": 4, "hc_iters": 3, "hc_eps": 1e-6, "q_lora": 128, "rope_tail": 32, "window": 32,
                       "o_groups": 2, "o_rank": 128, "sparse_layers": [1], "index_topk": 4,
                       "engram": {"layers": [0], "ngram": 3, "heads": 2, "compressed_vocab": 512, "table_rows": 509,
                                  "cache_rows": 256}}})


def flint_tiny() -> ModelSpec:
    """Small Flint-style shape: local layers (window 33, rotary) and global layers without positions, QK-norm, a
    learnable soft-max sink per head, two dense layers then sigmoid-routed experts with a shared expert."""
    return ModelSpec(
        name="flint-tiny", arch="flint", layers=5, hidden=512, heads=4, kv_heads=1, head_dim=128, ffn=1024, vocab=2048,
        rope_theta=1e4, rms_eps=1e-6, qk_norm=True,
        moe=MoeSpec(num_experts=8, top_k=2, expert_ffn=128, score="sigmoid", n_shared=1, shared_ffn=256,
                    first_dense_layers=2, dense_ffn=1024),
        extra={"flint": {"window": 33, "no_rope_layers": [0, 1, 4]}})


def _loop_spec(name: str, hidden: int, heads: int, ffn: int, vocab: int, per_stack: int, h_cycles: int, l_cycles: int,
               original_max: int) -> ModelSpec:
    return ModelSpec(
        name=name, arch="loop_vl", layers=h_cycles * (l_cycles + 1) * per_stack, hidden=hidden, heads=heads, kv_heads=heads,
        head_dim=128, ffn=ffn, vocab=vocab, rope_theta=1e4, rms_eps=1e-6,
        extra={"hrm": {"layers_per_stack": per_stack, "h_cycles": h_cycles, "l_cycles": l_cycles,
                       "embedding_scale": float(hidden) ** 0.5,
                       "yarn": {"factor": 2.0, "original_max": original_max, "beta_fast": 32.0, "beta_slow": 1.0}}})


def loop_tiny() -> ModelSpec:
    """Small looped two-stack decoder: two weight stacks of 2 layers, 2 H cycles of 3 L calls + 1 H call = 16 cache
    layers, gated full attention, YaRN positions."""
    return _loop_spec("loop-tiny", 256, 2, 512, 2048, per_stack=2, h_cycles=2, l_cycles=3, original_max=64)


def loopvl_text() -> ModelSpec:
    """The published LoopVL text geometry: 1536 hidden, 12 heads, two stacks of 16 layers applied 2 x (3 + 1) times
    (128 cache layers), vocabulary 65536."""
    return _loop_spec("loopvl-text-shape", 1536, 12, 4096, 65536, per_stack=16, h_cycles=2, l_cycles=3, original_max=4096)


def glm5_next_tiny() -> ModelSpec:
    """Small GLM-5-style shape: the hyper-connection program with every stage collapsing on its own pre-mix, top-k sparse
    attention with the pooled indexer in every layer, sigmoid routing with selection bias."""
    s = deepseek_v41_tiny()
    s.name, s.arch = "glm5-next-tiny", "glm5_next"
    s.moe.score, s.moe.routed_scaling = "noaux", 1.0
    s.extra = {"v41": dict(s.extra["v41"], hc_policy="own", sparse_layers=[0, 1, 2], engram=None)}
    return s


NAMED_SHAPES = {
    "tiny-gemma": tiny_gemma, "qwen3-moe-fp4-tiny": qwen3_moe_fp4_tiny, "tiny-hybrid": tiny_hybrid, "tiny-embed": tiny_embed, "tiny-diffusion": tiny_diffusion, "tiny-vl": tiny_vl, "tiny-minicpm": tiny_minicpm, "tiny-moe": tiny_moe, "tiny-llama": tiny_llama, "llama3-8b-shape": llama3_8b, "llama3-70b-shape": llama3_70b,
    "deepseek-v3-shape": deepseek_v3, "deepseek-v3-tiny": deepseek_v3_tiny, "deepseek-v3-mini": deepseek_v3_mini,
    "deepseek-v3-fp8-mini": deepseek_v3_fp8_mini, "deepseek-v41-tiny": deepseek_v41_tiny, "glm5-next-tiny": glm5_next_tiny, "flint-tiny": flint_tiny,
    "loop-tiny": loop_tiny, "loopvl-text-shape": loopvl_text,
    "qwen3-moe-235b-shape": qwen3_moe_235b, "qwen3-moe-tiny": qwen3_moe_tiny,
}


def named_shape(name: str) -> ModelSpec:
    if name not in NAMED_SHAPES:
        raise KeyError(f"unknown shape {name!r}; known: {sorted(NAMED_SHAPES)}")
    return NAMED_SHAPES[name]()


# ------------------------------------------------------------------------------------------
# config.json normalisation
# ------------------------------------------------------------------------------------------
class ConfigError(ValueError):
    pass


_ARCH_MAP = {
    "LlamaForCausalLM": "llama", "MistralForCausalLM": "llama", "Qwen2ForCausalLM": "qwen3",
    "Qwen3ForCausalLM": "qwen3", "Qwen3MoeForCausalLM": "qwen3_moe", "DeepseekV3ForCausalLM": "deepseek_v3",
    "DeepseekV2ForCausalLM": "deepseek_v3", "FlintForCausalLM": "flint", "LoopVLForConditionalGeneration": "loop_vl",
}


def _loopvl_spec(cfg: dict[str, Any], name: str) -> ModelSpec:
    """``LoopVLForConditionalGeneration`` (src/model_spec.rs:2273-2400 of the reference), text side: the looped two-stack
    decoder described by ``text_config`` (``hrm_text``); the vision encoder and projector of the checkpoint are not
    loaded."""
    t = cfg.get("text_config")
    if not isinstance(t, dict) or t.get("model_type") != "hrm_text":
        raise ConfigError("LoopVL text_config (hrm_text) missing")
    if cfg.get("quantization_config") is not None:
        raise ConfigError("LoopVL checkpoints are BF16 / F32")
    for key, want in (("hidden_act", "silu"), ("prefix_lm", True), ("tie_word_embeddings", False), ("attention_bias", False),
                      ("mlp_bias", False)):
        if t.get(key, want) != want:
            raise ConfigError(f"unsupported LoopVL setting {key}={t.get(key)!r}")
    rope = t.get("rope_parameters") or {}
    if rope.get("rope_type") != "yarn":
        raise ConfigError("LoopVL positions are YaRN-scaled")
    language = (cfg.get("loopvl_config") or {}).get("language") or {}
    for key in ("hidden_size", "num_attention_heads", "head_dim", "H_cycles", "L_cycles", "max_position_embeddings"):
        if key in language and language[key] != t.get(key):
            raise ConfigError(f"LoopVL language / text_config mismatch: {key}")
    if int(t["head_dim"]) != 128 or int(t["num_key_value_heads"]) != int(t["num_attention_heads"]):
        raise ConfigError("LoopVL heads are 128 wide without grouping")
    per, hc, lc = int(t["num_layers_per_stack"]), int(t["H_cycles"]), int(t["L_cycles"])
    if int(t.get("num_hidden_layers", hc * (lc + 1) * per)) != hc * (lc + 1) * per:
        raise ConfigError("num_hidden_layers differs from H_cycles * (L_cycles + 1) * num_layers_per_stack")
    spec = _loop_spec(name, int(t["hidden_size"]), int(t["num_attention_heads"]), int(t["intermediate_size"]), int(t["vocab_size"]),
                      per_stack=per, h_cycles=hc, l_cycles=lc, original_max=int(rope["original_max_position_embeddings"]))
    spec.rope_theta, spec.rms_eps = float(t.get("rope_theta", 10000.0)), float(t.get("rms_norm_eps", 1e-6))
    spec.max_position = int(t["max_position_embeddings"])
    spec.eos_token_id = t.get("eos_token_id")
    hrm = spec.extra["hrm"]
    hrm["embedding_scale"] = float(t.get("embedding_scale", hrm["embedding_scale"]))
    hrm["yarn"] = {"factor": float(rope["factor"]), "original_max": int(rope["original_max_position_embeddings"]),
                   "beta_fast": float(rope.get("beta_fast", 32.0)), "beta_slow": float(rope.get("beta_slow", 1.0))}
    return spec


def _flint_spec(cfg: dict[str, Any], name: str) -> ModelSpec:
    """``FlintForCausalLM`` (src/model_spec.rs:2723-2905 of the reference): sliding-window layers with rotary positions,
    the listed layers global and without positions, QK-norm, a learnable soft-max offset per head, dense FFNs in the
    ``mlp_only_layers`` prefix and sigmoid-routed experts with one shared expert after it."""
    for key, want in (("hidden_act", "silu"), ("attention_bias", False), ("router_score_function", "sigmoid"),
                      ("softmax_type", "learnable"), ("norm_topk_prob", True), ("use_sliding_window", True), ("decoder_sparse_step", 1)):
        if cfg.get(key, want) != want:
            raise ConfigError(f"unsupported Flint setting {key}={cfg.get(key)!r}")
    layers = int(cfg["num_hidden_layers"])
    no_rope = sorted(int(i) for i in cfg["no_rope_layer_indices"])
    if any(not (0 <= i < layers) for i in no_rope) or len(set(no_rope)) != len(no_rope):
        raise ConfigError("no_rope_layer_indices outside the layer range")
    types = cfg.get("layer_types")
    if types is not None:
        want = ["full_attention" if i in set(no_rope) else "sliding_attention" for i in range(layers)]
        if list(types) != want:
            raise ConfigError("layer_types disagree with no_rope_layer_indices (global layers carry no positions)")
    dense = sorted(int(i) for i in cfg.get("mlp_only_layers", []))
    if dense != list(range(len(dense))):
        raise ConfigError("mlp_only_layers must be a prefix of the layers")
    if int(cfg["head_dim"]) != 128:
        raise ConfigError("Flint heads are 128 wide")
    td = cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))
    dtype = {"bfloat16": "bf16", "float16": "f16", "float32": "fp32"}.get(td)
    if dtype is None:
        raise ConfigError(f"unsupported torch_dtype {td!r}")
    eos = cfg.get("eos_token_id")
    extra: dict[str, Any] = {"flint": {"window": int(cfg["sliding_window"]), "no_rope_layers": no_rope}}
    if isinstance(eos, list):
        extra["eos_token_ids"] = eos
        eos = eos[0] if eos else None
    heads, kv_heads = int(cfg["num_attention_heads"]), int(cfg["num_key_value_heads"])
    if heads % kv_heads:
        raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads")
    return ModelSpec(
        name=name, arch="flint", layers=layers, hidden=int(cfg["hidden_size"]), heads=heads, kv_heads=kv_heads, head_dim=128,
        ffn=int(cfg["intermediate_size"]), vocab=int(cfg["vocab_size"]), rope_theta=float(cfg.get("rope_theta", 10000.0)),
        rms_eps=float(cfg.get("rms_norm_eps", 1e-6)), dtype=dtype, tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        qk_norm=True, max_position=int(cfg.get("max_position_embeddings", 262144)), eos_token_id=eos,
        moe=MoeSpec(num_experts=int(cfg["num_experts"]), top_k=int(cfg["num_experts_per_tok"]),
                    expert_ffn=int(cfg["moe_intermediate_size"]), score="sigmoid", n_shared=1,
                    shared_ffn=int(cfg["shared_expert_intermediate_size"]), first_dense_layers=len(dense),
                    dense_ffn=int(cfg["intermediate_size"])),
        extra=extra)


def spec_from_hf_config(cfg: dict[str, Any], name: str = "model") -> ModelSpec:
    """Normalise a Hugging Face ``config.json``. Hard checks mirror the reference's: SiLU
    activation only, 16-bit or 32-bit floats, no unsupported rope scaling for plain Llama."""
    archs = cfg.get("architectures") or []
    arch = next((_ARCH_MAP[a] for a in archs if a in _ARCH_MAP), None)
    if arch is None:
        raise ConfigError(f"unsupported architectures {archs}")
    if arch == "flint":
        return _flint_spec(cfg, name)
    if arch == "loop_vl":
        return _loopvl_spec(cfg, name)
    act = cfg.get("hidden_act", "silu")
    if act not in ("silu", "swish"):
        raise ConfigError(f"unsupported activation {act!r}")
    td = cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))
    dtype = {"bfloat16": "bf16", "float16": "f16", "float32": "fp32"}.get(td)
    if dtype is None:
        raise ConfigError(f"unsupported torch_dtype {td!r}")
    hidden = int(cfg["hidden_size"])
    heads = int(cfg["num_attention_heads"])
    kv_heads = int(cfg.get("num_key_value_heads", heads))
    head_dim = int(cfg.get("head_dim") or hidden // heads)
    if heads % kv_heads:
        raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads")
    scaling = cfg.get("rope_scaling")
    extra: dict[str, Any] = {}
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind not in ("llama3", "yarn", "default", None):
            raise ConfigError(f"unsupported rope scaling {kind!r}")
        extra["rope_scaling"] = scaling
    quant = cfg.get("quantization_config") or {}
    linear_format = "bf16"
    if quant.get("quant_method") == "fp8" and quant.get("weight_block_size") == [128, 128]:
        linear_format = "fp8_block"
    elif quant.get("quant_algo") == "NVFP4" or quant.get("quant_method") == "modelopt":
        linear_format = "nvfp4"
    moe = None
    if arch == "qwen3_moe":
        moe = MoeSpec(num_experts=int(cfg["num_experts"]), top_k=int(cfg["num_experts_per_tok"]),
                      expert_ffn=int(cfg["moe_intermediate_size"]), score="softmax",
                      renormalize=bool(cfg.get("norm_topk_prob", True)),
                      expert_format=linear_format if linear_format != "bf16" else "bf16")
    mla = None
    if arch == "deepseek_v3":
        moe = MoeSpec(num_experts=int(cfg["n_routed_experts"]), top_k=int(cfg["num_experts_per_tok"]),
                      expert_ffn=int(cfg["moe_intermediate_size"]),
                      score="noaux" if cfg.get("topk_method", "noaux_tc") == "noaux_tc" else "softmax",
                      n_shared=int(cfg.get("n_shared_experts", 0)),
                      shared_ffn=int(cfg["moe_intermediate_size"]) * int(cfg.get("n_shared_experts", 0) or 0),
                      n_groups=int(cfg.get("n_group", 1)), topk_groups=int(cfg.get("topk_group", 1)),
                      routed_scaling=float(cfg.get("routed_scaling_factor", 1.0)),
                      renormalize=bool(cfg.get("norm_topk_prob", True)),
                      first_dense_layers=int(cfg.get("first_k_dense_replace", 0)),
                      dense_ffn=int(cfg["intermediate_size"]),
                      expert_format=linear_format)
        mla = MlaSpec(q_lora_rank=int(cfg.get("q_lora_rank") or 0), kv_lora_rank=int(cfg["kv_lora_rank"]),
                      qk_nope_dim=int(cfg["qk_nope_head_dim"]), qk_rope_dim=int(cfg["qk_rope_head_dim"]),
                      v_head_dim=int(cfg["v_head_dim"]))
    eos = cfg.get("eos_token_id")
    if isinstance(eos, list):
        extra["eos_token_ids"] = eos
        eos = eos[0] if eos else None
    return ModelSpec(
        name=name, arch=arch, layers=int(cfg["num_hidden_layers"]), hidden=hidden, heads=heads, kv_heads=kv_heads,
        head_dim=head_dim, ffn=int(cfg.get("intermediate_size", 0)), vocab=int(cfg["vocab_size"]),
        rope_theta=float(cfg.get("rope_theta", 10000.0)), rms_eps=float(cfg.get("rms_norm_eps", 1e-6)), dtype=dtype,
        linear_format=linear_format, tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        qk_norm=arch in ("qwen3", "qwen3_moe"), max_position=int(cfg.get("max_position_embeddings", 131072)),
        eos_token_id=eos, moe=moe, mla=mla, mtp_layers=int(cfg.get("num_nextn_predict_layers", 0)), extra=extra)


def read_model_spec(model_dir: str | Path) -> ModelSpec:
    p = Path(model_dir)
    cfg = json.loads((p / "config.json").read_text())
    return spec_from_hf_config(cfg, name=p.name)


# ------------------------------------------------------------------------------------------
# engine settings
# ------------------------------------------------------------------------------------------
@dataclass
class Settings:
    """Engine options shared by every entry point (CLI flags of the same names)."""
    device: int = 0
    capacity: int = 4096                  # tokens of KV per sequence the engine plans for
    chunk: int | None = None              # prefill chunk rows (planner-derived when None)
    device_budget_gib: float | None = None
    draft_model: str | None = None
    tree_builder: str = "waves"           # waves | serial | markov
    spec_budget: str = "chain"            # chain | tree16 | tree32 | tree64
    spec_graph: bool = True
    prefix_cache: bool = False
    kv_format: str = "bf16"               # bf16 | affine8
    kv_recent: int = 2048                 # affine8: tokens behind the newest that stay BF16 (groups older than that are sealed)
    runtime_dir: str | None = None
    dram_gb_s: float = 6550.0             # roofline denominators (measured on the target box)
    gemm_tflops: float = 1385.0
    verbose: bool = False
    tp: int = 1
    ep: int = 1
    max_batch: int = 64
    kv_block: int = 64
    graph: bool = True

    def resolved_runtime_dir(self) -> Path:
        import os
        d = self.runtime_dir or os.environ.get("FLYINGFISH_RUNTIME_DIR") or str(Path.home() / ".flyingfish")
        return Path(d)
