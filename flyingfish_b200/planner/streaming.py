"""Dense-layer streaming: run a model whose layers do not all fit in device memory.

``plan_layer_streaming`` decides, from byte counts and measured rates, which layers stay resident on the device,
how many device *slots* the remaining layers cycle through, and whether their home is pinned host memory or the
disk tier; it prices a decode token and a prefill chunk so the planner can compare against a smaller context.
``StreamedLayers`` is the runtime: a list-like object the model indexes as ``layers[i]``; resident layers are
returned as they are, a streamed layer is copied from pinned host memory into the next slot on a copy stream
(prefetching the following streamed layer while the current one computes) and returned as a ``LayerWeights`` whose
tensors are views of the slot. CUDA graphs are not used with streaming (the tensors behind a layer move).
Mirrors the dense-layer placement of the reference's planner (src/prefill.rs:82-208 placement records, :378-680
slot cycling, :269-287 pricing by PCIe and disk rates).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class LayerPlacement:
    resident: tuple[int, ...]            # layer ids kept on the device
    streamed: tuple[int, ...]            # layer ids cycling through the slots, in execution order
    slots: int                           # device slots for streamed layers (0 when nothing streams)
    host_layers: tuple[int, ...]         # streamed layers homed in pinned host memory
    disk_layers: tuple[int, ...]         # streamed layers homed on disk (read through the host staging buffer)
    slot_bytes: int
    device_bytes: int                    # resident + slots
    decode_ms: float                     # estimated time of one decode step over all layers
    bound: str                           # "compute", "pcie" or "disk"


def plan_layer_streaming(layer_bytes: list[int], device_budget: int, host_budget: int, h2d_gbs: float, disk_gbs: float,
                         compute_ms_per_layer: float, min_slots: int = 2) -> LayerPlacement:
    """Layers are executed in order every step, so a streamed layer must be re-copied every step: keep as many
    as fit resident (the LAST layers stream, so that their copies overlap the resident layers' compute at the
    start of the step), give the rest ``min_slots`` slots (double buffering) and add slots while memory is left."""
    n = len(layer_bytes)
    if n == 0 or device_budget <= 0:
        raise ValueError("nothing to place")
    if sum(layer_bytes) <= device_budget:
        return LayerPlacement(tuple(range(n)), (), 0, (), (), 0, sum(layer_bytes), n * compute_ms_per_layer, "compute")
    slot = max(layer_bytes)
    if min_slots * slot > device_budget:
        raise ValueError("device budget is smaller than two layer slots")
    resident, used = [], min_slots * slot
    for i in range(n):
        if used + layer_bytes[i] <= device_budget and n - (i + 1) >= min_slots:
            resident.append(i); used += layer_bytes[i]
        else:
            break
    streamed = [i for i in range(n) if i not in resident]
    slots = min_slots
    while slots < len(streamed) and used + slot <= device_budget:
        slots += 1; used += slot
    host, disk, hb = [], [], host_budget
    for i in streamed:
        if layer_bytes[i] <= hb:
            host.append(i); hb -= layer_bytes[i]
        else:
            disk.append(i)
    copy_ms = sum(layer_bytes[i] for i in streamed) / (h2d_gbs * 1e6)
    disk_ms = sum(layer_bytes[i] for i in disk) / (disk_gbs * 1e6) if disk else 0.0
    compute_ms = n * compute_ms_per_layer
    # copies of streamed layers overlap compute; the slowest of the three pipelines sets the step time
    step = max(compute_ms, copy_ms, disk_ms)
    bound = "compute" if step == compute_ms else ("pcie" if step == copy_ms else "disk")
    return LayerPlacement(tuple(resident), tuple(streamed), slots, tuple(host), tuple(disk), slot, used, step, bound)


def _tensor_fields(lw) -> list[str]:
    return [f.name for f in dataclasses.fields(lw) if isinstance(getattr(lw, f.name), torch.Tensor)]


class StreamedLayers:
    """List-like view over layer weights where some layers live in pinned host memory."""

    def __init__(self, layers: list, placement: LayerPlacement, device: torch.device):
        self.device = device
        self.placement = placement
        self.n = len(layers)
        self.resident = {i: layers[i] for i in placement.resident}
        self.host = {}
        for i in placement.streamed:
            lw = layers[i]
            h = dataclasses.replace(lw)
            for name in _tensor_fields(lw):
                t = getattr(lw, name).detach().to("cpu")
                setattr(h, name, t.pin_memory() if device.type == "cuda" else t)
            self.host[i] = h
        self.order = list(placement.streamed)
        self.slot_of: dict[int, int] = {}
        self.slots = []
        for _ in range(placement.slots):
            bufs = {}
            for i in self.order:
                for name in _tensor_fields(self.host[i]):
                    t = getattr(self.host[i], name)
                    cur = bufs.get(name)
                    if cur is None or cur.numel() * cur.element_size() < t.numel() * t.element_size():
                        bufs[name] = torch.empty(t.numel(), dtype=t.dtype, device=device)
            self.slots.append(bufs)
        self.copy_stream = torch.cuda.Stream(device) if device.type == "cuda" else None
        self.ready: dict[int, object] = {}            # layer -> event of its copy
        self.released: list[object] = [None] * placement.slots   # per slot: event after its last consumer
        self.next_slot = 0
        self._current: int | None = None
        self.stats = {"copies": 0, "bytes": 0}

    def __len__(self) -> int:
        return self.n

    def _issue(self, layer: int) -> None:
        if layer in self.slot_of:
            return
        slot = self.next_slot
        self.next_slot = (self.next_slot + 1) % len(self.slots)
        for l, s in list(self.slot_of.items()):
            if s == slot:
                del self.slot_of[l]; self.ready.pop(l, None)
        self.slot_of[layer] = slot
        h = self.host[layer]
        ctx = torch.cuda.stream(self.copy_stream) if self.copy_stream is not None else None
        if ctx is not None:
            if self.released[slot] is not None:
                self.copy_stream.wait_event(self.released[slot])       # the slot's previous layer has been consumed
            ctx.__enter__()
        try:
            for name in _tensor_fields(h):
                src = getattr(h, name)
                dst = self.slots[slot][name][: src.numel()].view(src.shape)
                dst.copy_(src, non_blocking=True)
                self.stats["bytes"] += src.numel() * src.element_size()
            self.stats["copies"] += 1
            if self.copy_stream is not None:
                ev = torch.cuda.Event(); ev.record(self.copy_stream); self.ready[layer] = ev
        finally:
            if ctx is not None:
                ctx.__exit__(None, None, None)

    def _release_current(self) -> None:
        """The kernels that read the layer handed out last are enqueued by now (the model asks for layers in
        execution order): after them its slot may be overwritten."""
        cur = self._current
        if cur is not None and cur in self.slot_of and self.copy_stream is not None:
            ev = torch.cuda.Event(); ev.record(torch.cuda.current_stream(self.device))
            self.released[self.slot_of[cur]] = ev
        self._current = None

    def __getitem__(self, i: int):
        if i != self._current:
            self._release_current()
        if i in self.resident:
            return self.resident[i]
        if i not in self.host:
            raise IndexError(i)
        self._issue(i)
        # keep the pipeline full: request the streamed layers that follow, one per remaining slot
        k = self.order.index(i)
        for j in range(1, len(self.slots)):
            self._issue(self.order[(k + j) % len(self.order)])
        slot = self.slot_of[i]
        if self.copy_stream is not None:
            torch.cuda.current_stream(self.device).wait_event(self.ready[i])
        self._current = i
        h = self.host[i]
        lw = dataclasses.replace(h)
        for name in _tensor_fields(h):
            src = getattr(h, name)
            setattr(lw, name, self.slots[slot][name][: src.numel()].view(src.shape))
        return lw

