"""NVMe tier: experts that fit neither HBM nor the pinned host arena are read on demand from the
checkpoint shards with aligned O_DIRECT reads into a small ring of pinned slots (the reference's
src/experts/disk.rs:440-770, 844-1830). A ring slot is leased until the caller releases it; reads
for upcoming layers can be queued ahead of time (bounded prefetch, demand reads first).
"""
from __future__ import annotations

from collections import OrderedDict

import torch

from .catalogue import ExpertCatalogue, slot_layout
from .native import DirectReader


class DiskExperts:
    def __init__(self, catalogue: ExpertCatalogue, disk_set: set[tuple[int, int]], ring_slots: int = 8,
                 threads: int = 4, pin: bool = False, layer_base: int = 0):
        self.cat = catalogue
        self.disk_set = disk_set              # (MoE layer ordinal, expert)
        self.layer_base = layer_base          # model layer number of MoE ordinal 0
        self.layout = slot_layout(catalogue.spec)
        self.reader = DirectReader(threads)
        self.ring = [torch.empty(self.layout.total, dtype=torch.uint8, pin_memory=pin) for _ in range(ring_slots)]
        self.free = list(range(ring_slots))
        self.cached: "OrderedDict[tuple[int, int], int]" = OrderedDict()     # key -> ring slot (LRU)
        self.pending: dict[tuple[int, int], tuple[int, list[int]]] = {}      # key -> (slot, tickets)
        self.stats = {"reads": 0, "bytes": 0, "hits": 0, "prefetched": 0}

    def on_disk(self, layer: int, expert: int) -> bool:
        return (layer, expert) in self.disk_set

    def _slot(self) -> int:
        if self.free:
            return self.free.pop()
        if not self.cached:
            raise RuntimeError("direct-IO ring exhausted: every slot has a read in flight")
        _, slot = self.cached.popitem(last=False)
        return slot

    def _submit(self, layer: int, expert: int) -> tuple[int, list[int]]:
        slot = self._slot()
        buf = self.ring[slot]
        L = self.layout
        dst_off = {"gate_proj": L.gate, "up_proj": L.up, "down_proj": L.down}
        tickets = []
        for r in self.cat.ranges[(self.layer_base + layer, expert)]:
            part = next(p for p in dst_off if f".{p}.weight" in r.name)
            if not r.name.endswith(".weight"):
                continue                      # scale tensors of quantised formats travel with the codes (not used here)
            fd = self.reader.open(r.path)
            tickets.append(self.reader.submit(fd, r.begin, r.nbytes, buf[dst_off[part]: dst_off[part] + r.nbytes]))
            self.stats["bytes"] += r.nbytes
        self.stats["reads"] += 1
        return slot, tickets

    def prefetch(self, layer: int, experts: list[int], limit: int = 2) -> None:
        """Queue reads for experts of an upcoming layer (at most ``limit`` outstanding)."""
        for e in experts:
            key = (layer, e)
            if len(self.pending) >= limit:
                break
            if key in self.cached or key in self.pending or not self.on_disk(layer, e):
                continue
            self.pending[key] = self._submit(layer, e)
            self.stats["prefetched"] += 1

    def fetch(self, layer: int, expert: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Blocking: (gate|up [2f, h], down [h, f]) views into the ring slot holding the expert."""
        key = (layer, expert)
        if key in self.cached:
            self.cached.move_to_end(key)
            self.stats["hits"] += 1
            slot = self.cached[key]
        else:
            slot, tickets = self.pending.pop(key) if key in self.pending else self._submit(layer, expert)
            for t in tickets:
                self.reader.wait(t)
            self.cached[key] = slot
        L = self.layout
        dt = torch.bfloat16 if L.elem_bytes == 2 else torch.float32
        buf = self.ring[slot]
        gu = buf[: L.down].view(dt).view(2 * L.ffn, L.hidden)
        down = buf[L.down: L.total].view(dt).view(L.hidden, L.ffn)
        return gu, down

    def close(self) -> None:
        self.reader.close()
