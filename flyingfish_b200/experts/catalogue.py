"""Expert catalogue: where every routed expert's bytes live inside the published shards, and how
they are packed into a slot (the reference's src/experts/catalogue.rs:11-325, 524-830).

The tiers copy experts by byte range, straight out of the checkpoint files and without conversion:
host blocks and GPU slots hold ``[gate rows | up rows | down rows]`` (plus the scale tensors of the
quantised formats) in exactly the stored dtype.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

from ..config import ModelSpec
from ..loaders.safetensors_io import CheckpointError, MappedCheckpoint

PARTS = ("gate_proj", "up_proj", "down_proj")


@dataclass(frozen=True)
class ByteRange:
    path: str
    begin: int          # absolute file offset
    end: int
    name: str

    @property
    def nbytes(self) -> int:
        return self.end - self.begin


@dataclass
class SlotLayout:
    """Offsets of the three matrices (and optional scales) inside a slot, in bytes."""
    gate: int
    up: int
    down: int
    total: int
    elem_bytes: int
    ffn: int
    hidden: int


def slot_layout(spec: ModelSpec, elem_bytes: int = 2) -> SlotLayout:
    f, h = spec.moe.expert_ffn, spec.hidden
    m = f * h * elem_bytes
    return SlotLayout(gate=0, up=m, down=2 * m, total=3 * m, elem_bytes=elem_bytes, ffn=f, hidden=h)


# ------------------------------------------------------------------------------------------------
# Native slot layouts of the quantised expert formats (the reference's ExpertLayout::{Fp8W8a16, Fp8W8a16Block,
# Fp4E2m1Block}, src/experts/catalogue.rs:40-330): a slot holds the three code matrices and then their three scale
# tensors, every slice starting on a 16-byte boundary, in exactly the stored dtypes, so that a tier copies an expert by
# byte range and a kernel addresses the slices by these offsets.
# ------------------------------------------------------------------------------------------------
FORMATS = ("bf16", "bf16_separate", "fp8_channel", "fp8_block", "e2m1_block", "nvfp4")


@dataclass(frozen=True)
class QuantSlotLayout:
    """``slices``: name -> (begin, end) byte offsets inside the slot, names ``gate up down`` (codes) and
    ``gate_scale up_scale down_scale`` (and ``global_scale`` for NVFP4)."""
    format: str
    slices: dict
    total: int
    ffn: int
    hidden: int

    def range(self, name: str) -> tuple[int, int]:
        return self.slices[name]

    @property
    def code_bytes(self) -> int:
        return sum(e - b for n, (b, e) in self.slices.items() if n in ("gate", "up", "down"))

    @property
    def scale_bytes(self) -> int:
        return sum(e - b for n, (b, e) in self.slices.items() if n not in ("gate", "up", "down"))


def _align16(n: int) -> int:
    return (n + 15) // 16 * 16


def quant_slot_layout(fmt: str, ffn: int, hidden: int, block: int = 128) -> QuantSlotLayout:
    """Slot layout of one expert (gate/up: [ffn, hidden], down: [hidden, ffn]) in ``fmt``:

    * ``bf16`` / ``bf16_separate``: two-byte elements, no scales (fused = gate and up adjacent, the same bytes);
    * ``fp8_channel``: one-byte E4M3 codes + one FP32 scale per output row (W8A16);
    * ``fp8_block``: one-byte E4M3 codes + one FP32 scale per ``block`` x ``block`` tile (ceil on both sides);
    * ``e2m1_block``: two four-bit E2M1 codes per byte ([rows, cols / 2]) + one E8M0 byte per 32 columns of each row;
    * ``nvfp4``: two codes per byte + one E4M3 byte per 16 columns of each row + one FP32 global scale per matrix."""
    if fmt not in FORMATS:
        raise ValueError(f"unknown expert format {fmt!r}")
    if ffn <= 0 or hidden <= 0:
        raise ValueError("empty expert geometry")
    mats = {"gate": (ffn, hidden), "up": (ffn, hidden), "down": (hidden, ffn)}
    if fmt in ("e2m1_block", "nvfp4") and (hidden % 32 or ffn % 32):
        raise ValueError("four-bit expert formats need both dimensions to be multiples of 32")

    def code_bytes(r, c):
        return r * c * 2 if fmt.startswith("bf16") else r * c if fmt.startswith("fp8") else r * c // 2

    def scale_bytes(r, c):
        if fmt == "fp8_channel":
            return r * 4
        if fmt == "fp8_block":
            return ((r + block - 1) // block) * ((c + block - 1) // block) * 4
        if fmt == "e2m1_block":
            return r * (c // 32)
        if fmt == "nvfp4":
            return r * (c // 16)
        return 0
    off, slices = 0, {}
    for name, (r, c) in mats.items():
        slices[name] = (off, off + code_bytes(r, c))
        off = _align16(off + code_bytes(r, c))
    if not fmt.startswith("bf16"):
        for name, (r, c) in mats.items():
            slices[name + "_scale"] = (off, off + scale_bytes(r, c))
            off = _align16(off + scale_bytes(r, c))
    if fmt == "nvfp4":
        slices["global_scale"] = (off, off + 12)
        off = _align16(off + 12)
    return QuantSlotLayout(fmt, slices, off, ffn, hidden)


def pack_slot(layout: QuantSlotLayout, tensors: dict) -> "bytes":
    """Serialise one expert's tensors (name -> torch tensor of the stored dtype) into slot bytes; the inverse of
    :func:`slot_views`. Used to stage random-init experts of the quantised formats the way a checkpoint would."""
    import torch
    buf = torch.zeros(layout.total, dtype=torch.uint8)
    for name, (b, e) in layout.slices.items():
        raw = tensors[name].contiguous().view(torch.uint8).reshape(-1)
        if raw.numel() != e - b:
            raise ValueError(f"{name}: {raw.numel()} bytes, the layout wants {e - b}")
        buf[b:e] = raw
    return buf


def slot_views(layout: QuantSlotLayout, slot) -> dict:
    """Typed views of the slices of a slot (a uint8 tensor of ``layout.total`` bytes, on any device): codes as uint8
    matrices, FP32 scales as float32, E8M0 / E4M3 scale bytes as uint8."""
    import torch
    f, h, fmt = layout.ffn, layout.hidden, layout.format
    mats = {"gate": (f, h), "up": (f, h), "down": (h, f)}
    out = {}
    for name, (b, e) in layout.slices.items():
        raw = slot[b:e]
        base = name.replace("_scale", "")
        if name == "global_scale":
            out[name] = raw.view(torch.float32)
        elif name in mats:
            r, c = mats[name]
            out[name] = raw.view(torch.bfloat16).view(r, c) if fmt.startswith("bf16") else raw.view(r, -1)
        elif fmt in ("fp8_channel", "fp8_block"):
            out[name] = raw.view(torch.float32).view(mats[base][0] if fmt == "fp8_channel" else -1, *(() if fmt == "fp8_channel" else ((mats[base][1] + 127) // 128,)))
        else:
            out[name] = raw.view(mats[base][0], -1)
    return out


class ExpertCatalogue:
    def __init__(self, spec: ModelSpec, ranges: dict[tuple[int, int], list[ByteRange]]):
        self.spec = spec
        self.ranges = ranges
        self.layers = sorted({l for l, _ in ranges})

    @classmethod
    def from_checkpoint(cls, ckpt: MappedCheckpoint, spec: ModelSpec) -> "ExpertCatalogue":
        if spec.moe is None:
            raise CheckpointError("model has no routed experts")
        out: dict[tuple[int, int], list[ByteRange]] = {}
        for i in range(spec.moe.first_dense_layers, spec.layers):
            for e in range(spec.moe.num_experts):
                rs = []
                for part in PARTS:
                    base = f"model.layers.{i}.mlp.experts.{e}.{part}.weight"
                    for name in (base, base + "_scale_inv", base + "_scale", base + "_scale_2"):
                        if ckpt.has(name):
                            f = ckpt.where[name]
                            b, en = f.byte_range(name)
                            rs.append(ByteRange(str(f.path), b, en, name))
                if len(rs) < 3:
                    raise CheckpointError(f"layer {i} expert {e}: incomplete expert tensors")
                out[(i, e)] = rs
        return cls(spec, out)

    def expert_bytes(self, layer: int, expert: int) -> int:
        return sum(r.nbytes for r in self.ranges[(layer, expert)])

    def slot_bytes(self) -> int:
        return max(self.expert_bytes(l, e) for (l, e) in self.ranges)

    def files(self) -> list[str]:
        return sorted({r.path for rs in self.ranges.values() for r in rs})
