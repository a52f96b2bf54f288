"""Hardware-adaptive planning of the engine's memory: prefill chunk, KV blocks, decode graph
buckets.

Pure functions over a ``DeviceInfo`` so the arithmetic is testable without a GPU. The policy
follows the reference's prefill planner (src/prefill.rs:321-373, 1210-1310): hold back 1/16 of
device memory, cap the rows of a prefill chunk by what the per-row workspace allows, and make the
chunk the largest power-of-two multiple of the attention tile that fits; whatever remains after
weights and workspace becomes KV blocks (the reference sizes one contiguous cache of ``capacity``
tokens; a paged cache takes every spare block, bounded by what ``max_batch`` sequences of
``capacity`` tokens can use).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch

from ..config import ModelSpec, Settings

ATTENTION_TILE = 64
B200_HBM_BYTES = 180 * (1 << 30)


@dataclass
class DeviceInfo:
    """What the planner needs to know about a device (src/backend/setup.rs:21-46)."""
    name: str = "cpu"
    sms: int = 0
    l2_bytes: int = 0
    smem_per_block: int = 0
    total_bytes: int = 0
    free_bytes: int = 0
    memory_bytes_per_second: float = 0.0
    cc: tuple[int, int] = (0, 0)

    def to_json(self) -> dict:
        return dataclasses.asdict(self)


def probe_device(device: torch.device | str) -> DeviceInfo:
    device = torch.device(device)
    if device.type != "cuda":
        import psutil
        vm = psutil.virtual_memory()
        return DeviceInfo(name="cpu", total_bytes=vm.total, free_bytes=vm.available)
    p = torch.cuda.get_device_properties(device)
    free, total = torch.cuda.mem_get_info(device)
    # HBM3e on B200: 8 stacks x 1024 bit; bandwidth = 2 * memory clock * bus width / 8
    clock_hz = getattr(p, "memory_clock_rate", 0) * 1e3
    bus = getattr(p, "memory_bus_width", 0)
    bw = 2.0 * clock_hz * bus / 8.0 if clock_hz and bus else 0.0
    return DeviceInfo(name=p.name, sms=p.multi_processor_count, l2_bytes=getattr(p, "L2_cache_size", 0),
                      smem_per_block=getattr(p, "shared_memory_per_block_optin", 0), total_bytes=total,
                      free_bytes=free, memory_bytes_per_second=bw, cc=(p.major, p.minor))


def workspace_row_bytes(spec: ModelSpec, tp: int = 1) -> int:
    """Bytes of activation workspace per prefill row: residual, normed, attention out, projection
    out (4 x hidden), packed QKV, gate/up + activated (3 x ffn), ids/positions/slots
    (the reference's formula, src/prefill.rs:302-307, with the parallel shards applied)."""
    ffn = spec.moe.expert_ffn * spec.moe.top_k if spec.moe is not None else spec.ffn
    return (4 * spec.hidden + spec.qkv_dim // tp + 3 * ffn // tp) * 2 + 12 + spec.heads * 4


def largest_pow2_multiple(limit: int, tile: int) -> int:
    """Largest ``tile * 2**k`` that does not exceed ``limit`` (0 if even one tile does not fit)."""
    if limit < tile:
        return 0
    c = tile
    while c * 2 <= limit:
        c *= 2
    return c


@dataclass
class EnginePlan:
    prefill_chunk: int
    kv_blocks: int
    kv_bytes: int
    workspace_bytes: int
    reserve_bytes: int
    weights_bytes: int
    budget_bytes: int
    graph_buckets: tuple[int, ...]

    def to_json(self) -> dict:
        return dataclasses.asdict(self)


class PlanError(RuntimeError):
    pass


def plan_memory(spec: ModelSpec, settings: Settings, info: DeviceInfo, weights_bytes: int, tp: int = 1,
                max_chunk: int = 16384) -> EnginePlan:
    total = info.total_bytes
    budget = total
    if settings.device_budget_gib is not None:
        budget = min(total, int(settings.device_budget_gib * (1 << 30)))
    reserve = total // 16
    free_after_weights = min(info.free_bytes, budget - weights_bytes) - reserve
    if free_after_weights <= 0:
        raise PlanError(f"model weights ({weights_bytes >> 20} MiB) leave no room inside the budget "
                        f"({budget >> 20} MiB, reserve {reserve >> 20} MiB)")
    row_bytes = workspace_row_bytes(spec, tp)
    hkv = max(1, spec.kv_heads // tp)
    if spec.mla is not None:
        block_bytes = spec.layers * settings.kv_block * (spec.mla.kv_lora_rank + spec.mla.qk_rope_dim) * 2
    else:
        block_bytes = spec.layers * hkv * settings.kv_block * spec.head_dim * 2 * 2
    blocks_per_seq = (settings.capacity + settings.kv_block - 1) // settings.kv_block
    # one sequence of `capacity` tokens must always fit next to a minimal chunk
    min_need = blocks_per_seq * block_bytes + ATTENTION_TILE * row_bytes
    if free_after_weights < min_need:
        raise PlanError(f"capacity {settings.capacity} needs {min_need >> 20} MiB of KV + workspace, "
                        f"{free_after_weights >> 20} MiB available")
    # workspace gets at most a quarter of what is left; the rest is KV
    ws_cap = free_after_weights // 4
    row_limit = min(settings.chunk or max_chunk, max_chunk, ws_cap // row_bytes)
    chunk = settings.chunk if settings.chunk and settings.chunk <= row_limit else \
        largest_pow2_multiple(row_limit, ATTENTION_TILE)
    if chunk <= 0:
        raise PlanError("no room for a prefill chunk")
    workspace = chunk * row_bytes
    kv_budget = free_after_weights - workspace
    want = blocks_per_seq * settings.max_batch + 1
    kv_blocks = int(min(kv_budget // block_bytes, want))
    if kv_blocks < blocks_per_seq:
        raise PlanError("no room for the KV cache of one full sequence")
    buckets = tuple(b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256) if b <= max(1, settings.max_batch))
    if buckets[-1] < settings.max_batch:
        buckets = buckets + (min(256, 1 << (settings.max_batch - 1).bit_length()),)
    return EnginePlan(prefill_chunk=int(chunk), kv_blocks=kv_blocks, kv_bytes=kv_blocks * block_bytes,
                      workspace_bytes=int(workspace), reserve_bytes=int(reserve), weights_bytes=int(weights_bytes),
                      budget_bytes=int(budget), graph_buckets=buckets)


def plan_engine(spec: ModelSpec, settings: Settings, device: torch.device | str, weights_bytes: int,
                tp: int = 1) -> EnginePlan:
    info = probe_device(device)
    if info.name == "cpu":
        # host execution: memory is not the constraint the planner models; give the tests a
        # small, fixed arena
        blocks_per_seq = (settings.capacity + settings.kv_block - 1) // settings.kv_block
        chunk = settings.chunk or 512
        return EnginePlan(prefill_chunk=chunk, kv_blocks=blocks_per_seq * min(settings.max_batch, 8) + 1, kv_bytes=0,
                          workspace_bytes=0, reserve_bytes=0, weights_bytes=weights_bytes, budget_bytes=0,
                          graph_buckets=())
    # weights are already resident when the planner runs, so `free` excludes them
    info2 = dataclasses.replace(info, free_bytes=info.free_bytes + weights_bytes)
    return plan_memory(spec, settings, info2, weights_bytes, tp)
