"""Weight containers: seeded random initialisation of a named shape, fusion of the published
per-projection tensors into the layouts the kernels want, and tensor-parallel sharding.

Tensor names follow the Hugging Face checkpoints the loaders read
(``model.layers.N.self_attn.q_proj.weight`` ...), so a safetensors reader and the synthetic
generator feed the same code. Fusions done here, once, at load time:

* ``wqkv``  = [q | k | v] rows (the reference's fused QKV catalog, src/backend/cuda/weights.rs),
  sharded by heads for tensor parallelism;
* ``wgu``   = gate/up rows interleaved per 64 so the GEMM epilogues can apply SwiGLU;
* row-parallel ``wo`` / ``wdown`` shards split the input dimension;
* ``lm_head`` is vocabulary-parallel.

Random weights are N(0, 0.02) from a per-tensor seed derived from (seed, tensor name), so every
rank and every parallel layout sees the same logical model.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Callable

import torch

from ..config import ModelSpec
from ..ops import ref

DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16, "fp32": torch.float32}


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(seed: int, name: str, shape: tuple[int, ...], dtype: torch.dtype, device: torch.device,
                  std: float = 0.02, ones: bool = False) -> torch.Tensor:
    if ones:
        return torch.ones(shape, dtype=dtype, device=device)
    numel = 1
    for d in shape:
        numel *= d
    # Small tensors are always drawn on the host and copied, so a model of a test-sized shape has the same weights on
    # every device (a GPU run can be compared with the CPU oracle); only the tensors of the large benchmark shapes,
    # which would take minutes to draw on the host, come from the device generator.
    draw_dev = device if numel > CPU_DRAW_MAX else torch.device("cpu")
    g = torch.Generator(device=draw_dev)
    g.manual_seed(tensor_seed(seed, name))
    t = torch.empty(shape, dtype=torch.float32 if draw_dev.type == "cpu" else dtype, device=draw_dev)
    t.normal_(0.0, std, generator=g)
    return t.to(dtype).to(device)


CPU_DRAW_MAX = 1 << 22      # elements; larger random tensors are drawn on their device


TensorSource = Callable[[str, tuple[int, ...]], torch.Tensor]


def synthetic_source(spec: ModelSpec, seed: int, device: torch.device, dtype: torch.dtype) -> TensorSource:
    """Tensor source producing N(0, 0.02) weights and unit norm weights by name."""
    def get(name: str, shape: tuple[int, ...]) -> torch.Tensor:
        is_norm = name.endswith("layernorm.weight") or name.endswith("norm.weight")
        return random_tensor(seed, name, shape, dtype, device, ones=is_norm)
    return get


@dataclass
class TPInfo:
    rank: int = 0
    size: int = 1


@dataclass
class LayerWeights:
    input_ln: torch.Tensor = None
    post_ln: torch.Tensor = None
    wqkv: torch.Tensor = None            # [(hq + 2 hkv)/tp * d, hidden]
    wo: torch.Tensor = None              # [hidden, hq/tp * d]
    q_norm: torch.Tensor | None = None
    k_norm: torch.Tensor | None = None
    wgu: torch.Tensor | None = None      # dense FFN, gate/up interleaved per 64 (or [gate|up] if not divisible)
    wgu_interleaved: bool = True
    wdown: torch.Tensor | None = None
    # MoE
    router: torch.Tensor | None = None
    router_bias: torch.Tensor | None = None
    experts_gu: torch.Tensor | None = None      # [E_local, 2f, hidden] (gate | up)
    experts_down: torch.Tensor | None = None    # [E_local, hidden, f]
    shared_gu: torch.Tensor | None = None
    shared_down: torch.Tensor | None = None
    extra: dict = field(default_factory=dict)


@dataclass
class ModelWeights:
    spec: ModelSpec
    embed: torch.Tensor
    final_norm: torch.Tensor
    lm_head: torch.Tensor                 # [vocab/tp (padded), hidden]
    layers: list[LayerWeights]
    tp: TPInfo
    vocab_shard: tuple[int, int] = (0, 0)  # [start, end) of this rank's vocabulary rows
    extra: dict = field(default_factory=dict)

    def nbytes(self) -> int:
        total = 0
        def add(t):
            nonlocal total
            if isinstance(t, torch.Tensor):
                total += t.numel() * t.element_size()
            elif hasattr(t, "nbytes") and callable(t.nbytes):      # FP8-resident weights
                total += t.nbytes()
            elif isinstance(t, dict):
                for v in t.values():
                    add(v)
            elif hasattr(t, "__dataclass_fields__"):
                for v in vars(t).values():
                    add(v)
        add(self.embed); add(self.final_norm); add(self.lm_head)
        for l in self.layers:
            for v in vars(l).values():
                add(v)
        return total


def shard_range(n: int, rank: int, size: int) -> tuple[int, int]:
    assert n % size == 0, f"{n} is not divisible by the parallel degree {size}"
    per = n // size
    return rank * per, (rank + 1) * per


def pack_ffn_fp8(lw: "LayerWeights") -> None:
    """Re-encode a layer's feed-forward matrices as FP8-resident weights (E4M3 codes + 128x128 block scales): the
    dense gate/up and down projections, the shared expert, and the routed experts (gate/up interleaved per 64 rows,
    the layout the grouped kernel's SwiGLU epilogue reads). Done layer by layer while a model is assembled, so only
    one layer ever exists in BF16."""
    from ..ops.quant_ops import Fp8Experts, Fp8Weight
    if isinstance(lw.wgu, torch.Tensor):
        assert not lw.wgu_interleaved, "FP8 dense FFN weights keep the [gate | up] row order of the checkpoint"
        lw.wgu = Fp8Weight.from_dense(lw.wgu)
        lw.wdown = Fp8Weight.from_dense(lw.wdown)
    if isinstance(lw.shared_gu, torch.Tensor):
        lw.shared_gu = Fp8Weight.from_dense(lw.shared_gu)
        lw.shared_down = Fp8Weight.from_dense(lw.shared_down)
    if isinstance(lw.experts_gu, torch.Tensor):
        lw.experts_gu = Fp8Experts.from_dense(lw.experts_gu, interleave=True)
        lw.experts_down = Fp8Experts.from_dense(lw.experts_down)


def build_decoder_weights(spec: ModelSpec, source: TensorSource, device: torch.device, tp: TPInfo | None = None,
                          ep: TPInfo | None = None, fuse_swiglu: bool = True, layer_hook=None) -> ModelWeights:
    """Assemble fused / sharded weights for a GQA decoder (dense or MoE FFN). ``layer_hook(layer_weights)`` runs on
    every finished layer (format conversion that should not wait for the whole model to exist)."""
    tp = tp or TPInfo()
    ep = ep or TPInfo()
    h, d = spec.hidden, spec.head_dim
    hq0, hq1 = shard_range(spec.heads, tp.rank, tp.size)
    if spec.kv_heads >= tp.size:
        kv0, kv1 = shard_range(spec.kv_heads, tp.rank, tp.size)
    else:  # replicate KV heads when there are fewer than ranks
        assert tp.size % spec.kv_heads == 0
        per = tp.size // spec.kv_heads
        kv0 = tp.rank // per
        kv1 = kv0 + 1
    layers: list[LayerWeights] = []
    for i in range(spec.layers):
        p = f"model.layers.{i}."
        lw = LayerWeights()
        lw.input_ln = source(p + "input_layernorm.weight", (h,))
        lw.post_ln = source(p + "post_attention_layernorm.weight", (h,))
        wq = source(p + "self_attn.q_proj.weight", (spec.q_dim, h))[hq0 * d: hq1 * d]
        wk = source(p + "self_attn.k_proj.weight", (spec.kv_dim, h))[kv0 * d: kv1 * d]
        wv = source(p + "self_attn.v_proj.weight", (spec.kv_dim, h))[kv0 * d: kv1 * d]
        lw.wqkv = torch.cat([wq, wk, wv], dim=0).contiguous()
        del wq, wk, wv
        lw.wo = source(p + "self_attn.o_proj.weight", (h, spec.q_dim))[:, hq0 * d: hq1 * d].contiguous()
        if spec.qk_norm:
            lw.q_norm = source(p + "self_attn.q_norm.weight", (d,))
            lw.k_norm = source(p + "self_attn.k_norm.weight", (d,))
        moe = spec.moe
        is_moe = moe is not None and i >= moe.first_dense_layers
        if not is_moe:
            f = moe.dense_ffn if (moe is not None and moe.dense_ffn) else spec.ffn
            f0, f1 = shard_range(f, tp.rank, tp.size)
            wg = source(p + "mlp.gate_proj.weight", (f, h))[f0:f1]
            wu = source(p + "mlp.up_proj.weight", (f, h))[f0:f1]
            if fuse_swiglu and (f1 - f0) % 128 == 0:
                lw.wgu = ref.interleave_gate_up(wg, wu)
                lw.wgu_interleaved = True
            else:
                lw.wgu = torch.cat([wg, wu], dim=0).contiguous()
                lw.wgu_interleaved = False
            del wg, wu
            lw.wdown = source(p + "mlp.down_proj.weight", (h, f))[:, f0:f1].contiguous()
        else:
            lw.router = source(p + "mlp.gate.weight", (moe.num_experts, h))
            if moe.score in ("noaux", "sqrt_softplus"):
                lw.router_bias = torch.zeros(moe.num_experts, dtype=torch.float32, device=device)
            e0, e1 = shard_range(moe.num_experts, ep.rank, ep.size)
            f = moe.expert_ffn
            gus, downs = [], []
            for e in range(e0, e1):
                q = p + f"mlp.experts.{e}."
                gus.append(torch.cat([source(q + "gate_proj.weight", (f, h)), source(q + "up_proj.weight", (f, h))], 0))
                downs.append(source(q + "down_proj.weight", (h, f)))
            lw.experts_gu = torch.stack(gus).contiguous()
            lw.experts_down = torch.stack(downs).contiguous()
            lw.extra["expert_range"] = (e0, e1)
            if moe.n_shared:
                sf = moe.shared_ffn
                s0, s1 = shard_range(sf, tp.rank, tp.size)
                q = p + "mlp.shared_experts."
                lw.shared_gu = torch.cat([source(q + "gate_proj.weight", (sf, h))[s0:s1],
                                          source(q + "up_proj.weight", (sf, h))[s0:s1]], 0).contiguous()
                lw.shared_down = source(q + "down_proj.weight", (h, sf))[:, s0:s1].contiguous()
        if layer_hook is not None:
            layer_hook(lw)
        layers.append(lw)
    embed = source("model.embed_tokens.weight", (spec.vocab, h))
    final_norm = source("model.norm.weight", (h,))
    vpad = (spec.vocab + tp.size - 1) // tp.size
    v0, v1 = tp.rank * vpad, min(spec.vocab, (tp.rank + 1) * vpad)
    if spec.tie_embeddings:
        lm_head = embed[v0:v1].contiguous() if tp.size > 1 else embed
    else:
        lm_head = source("lm_head.weight", (spec.vocab, h))[v0:v1].contiguous()
    return ModelWeights(spec=spec, embed=embed, final_norm=final_norm, lm_head=lm_head, layers=layers, tp=tp,
                        vocab_shard=(v0, v1))


def random_decoder_weights(spec: ModelSpec, seed: int = 0, device: torch.device | str = "cpu",
                           tp: TPInfo | None = None, ep: TPInfo | None = None, fuse_swiglu: bool = True) -> ModelWeights:
    device = torch.device(device)
    dtype = DTYPES[spec.dtype]
    return build_decoder_weights(spec, synthetic_source(spec, seed, device, dtype), device, tp, ep, fuse_swiglu)
