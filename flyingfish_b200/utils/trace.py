"""Operator trace: named FP32 tensors captured after chosen operators, saved as safetensors with
device metadata (the reference's ``--dump`` / ``--trace-layer``, src/trace.rs:11-130). Recording
copies device tensors to the host synchronously, so it is incompatible with CUDA-graph decode;
non-finite values are rejected at record time."""
from __future__ import annotations

from pathlib import Path

import torch

from ..loaders.safetensors_io import save_safetensors


class TraceError(RuntimeError):
    pass


class Trace:
    def __init__(self, device: str = "cpu", only_layer: int | None = None):
        self.device = device
        self.only_layer = only_layer
        self.tensors: dict[str, torch.Tensor] = {}
        self.step = 0

    def record(self, name: str, t: torch.Tensor) -> None:
        if self.only_layer is not None and name.startswith("layer.") and not name.startswith(f"layer.{self.only_layer}"):
            return
        v = t.detach().to(torch.float32).cpu()
        if not torch.isfinite(v).all():
            raise TraceError(f"non-finite values in {name}")
        key = f"step.{self.step}.{name}"
        self.tensors[key] = v
        if name == "logits":
            self.step += 1

    def save(self, path: str | Path) -> None:
        save_safetensors(path, self.tensors, metadata={"device": self.device, "format": "flyingfish-trace-1"})
