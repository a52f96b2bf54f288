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
