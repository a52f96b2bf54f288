"""Tiered expert provider: serves a MoE layer's routed experts from GPU slots, the pinned host
tier (CPU expert FFN for this token, promotion later) and the NVMe tier (direct-IO ring, then CPU).

Per MoE layer call (the reference's decode executor, src/backend/cuda/engine_moe.rs:1404-1830):

1. the routed ids / weights are read back to the host (one small D2H: the only host round trip,
   skipped entirely when every expert is resident),
2. ``Residency.dispatch`` splits the routes into slot hits, host misses and disk misses,
3. hits run on the device: ids are remapped to slot numbers (misses become -1 and are skipped by
   the dispatch kernels), then dispatch -> grouped GEMMs over the slot arena,
4. misses run on the host worker pool with the host copy of the weights (disk-tier experts are
   first read through the direct-IO ring); their outputs are uploaded behind the device outputs,
5. ONE combine sums every contribution of a row in ascending expert id.

At token end ``finish_token`` returns the admissions; the provider copies those experts into their
slots and updates the slot table (slot generations guard against stale tables).
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import moe_ops, ref
from .native import ExpertPool
from .plan import Admission, Capacity, ExpertGeometry
from .runtime import EMPTY, Move, Residency, Route


class ExpertStore:
    """Host-side home of one layer's expert weights: a pinned tensor for the host tier, optionally a
    disk reader for experts that do not fit."""

    def __init__(self, gate_up: torch.Tensor, down: torch.Tensor, pin: bool = False, disk=None):
        self.gate_up = gate_up.pin_memory() if pin and not gate_up.is_pinned() else gate_up     # [E, 2f, h]
        self.down = down.pin_memory() if pin and not down.is_pinned() else down                 # [E, h, f]
        self.disk = disk                                                                        # DiskExperts or None

    def weights(self, layer: int, expert: int) -> tuple[torch.Tensor, torch.Tensor]:
        if self.disk is not None and self.disk.on_disk(layer, expert):
            return self.disk.fetch(layer, expert)
        return self.gate_up[expert], self.down[expert]


class TieredExpertProvider:
    def __init__(self, geo: ExpertGeometry, cap: Capacity, adm: Admission, stores: list[ExpertStore],
                 device: torch.device | str, hidden: int, ffn: int, mode: str = "score", swiglu_mode: int = 0,
                 threads: int = 8, disk_experts: set[tuple[int, int]] | None = None):
        self.geo, self.cap = geo, cap
        self.device = torch.device(device)
        self.stores = stores
        self.hidden, self.ffn, self.swiglu_mode = hidden, ffn, swiglu_mode
        self.res = Residency(geo, cap, adm, mode=mode, host_backed=True, disk_experts=disk_experts)
        dt = stores[0].gate_up.dtype
        self.arena_gu = [torch.zeros(cap.slots_per_layer[l], 2 * ffn, hidden, dtype=dt, device=self.device)
                         for l in range(geo.layers)]
        self.arena_down = [torch.zeros(cap.slots_per_layer[l], hidden, ffn, dtype=dt, device=self.device)
                           for l in range(geo.layers)]
        self.table = [torch.full((geo.experts_per_layer,), EMPTY, dtype=torch.int32, device=self.device)
                      for _ in range(geo.layers)]
        self.pool = ExpertPool(threads) if dt == torch.bfloat16 else None
        self.layer_index: dict[int, int] = {}      # model layer number -> MoE layer ordinal
        self.copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.stats = {"cpu_rows": 0, "gpu_rows": 0, "h2d_expert_bytes": 0, "layers_all_hit": 0, "layer_calls": 0}
        self.freq = [[0.0] * geo.experts_per_layer for _ in range(geo.layers)]
        self.collect_freq = False

    # -- slot maintenance ----------------------------------------------------------------------
    def apply_moves(self, moves: list[Move]) -> None:
        for m in moves:
            wgu, wd = self.stores[m.layer].weights(m.layer, m.expert_in)
            if self.device.type == "cuda":
                from ..ops import moe_cuda
                with torch.cuda.stream(self.copy_stream):
                    g = wgu.to(self.device, non_blocking=True)
                    self.arena_gu[m.layer][m.slot].copy_(moe_cuda.interleave64(g[None])[0])
                    self.arena_down[m.layer][m.slot].copy_(wd.to(self.device, non_blocking=True))
            else:
                self.arena_gu[m.layer][m.slot].copy_(wgu)
                self.arena_down[m.layer][m.slot].copy_(wd)
            if m.expert_out != EMPTY:
                self.table[m.layer][m.expert_out] = EMPTY
            self.table[m.layer][m.expert_in] = m.slot
            self.stats["h2d_expert_bytes"] += self.geo.slot_bytes
        if moves and self.copy_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.copy_stream)

    def begin_request(self, prefill_freq: list[list[float]] | None = None) -> None:
        f = prefill_freq if prefill_freq is not None else self.freq
        self.apply_moves(self.res.begin_request(f))
        self.res.freeze_prefill_rank(f)

    def begin_token(self) -> None:
        self.res.begin_token()

    def finish_token(self) -> None:
        self.apply_moves(self.res.finish_token())

    # -- one layer -----------------------------------------------------------------------------
    def forward(self, model_layer: int, x: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        l = self.layer_index[model_layer]
        rows, k = ids.shape
        self.stats["layer_calls"] += 1
        ids_h = ids.cpu()
        w_h = weights.cpu()
        if self.collect_freq:
            for e in ids_h.flatten().tolist():
                self.freq[l][e] += 1.0
        opened = False
        if not self.res.in_token:          # prefill chunks: no decay / admission, plain dispatch
            self.res.in_token = True
            self.res.routed[l].clear()
            opened = True
        routes = [Route(r, j, int(ids_h[r, j]), float(w_h[r, j])) for r in range(rows) for j in range(k)]
        d = self.res.dispatch(l, routes)
        if opened:
            self.res.in_token = False
        misses = d.host + d.disk
        self.stats["cpu_rows"] += len(misses)
        self.stats["gpu_rows"] += len(d.hits)
        if not misses:
            self.stats["layers_all_hit"] += 1
        if self.device.type == "cuda":
            return self._forward_cuda(l, x, weights, ids, misses)
        return self._forward_host(l, x, w_h, ids_h, d, misses)

    def _cpu_contributions(self, l: int, x_host: torch.Tensor, misses: list[Route]) -> dict[tuple[int, int], torch.Tensor]:
        """Run the missed (row, choice) assignments on the host pool; returns outputs keyed by
        (row, choice)."""
        by_expert: dict[int, list[Route]] = {}
        for r in misses:
            by_expert.setdefault(r.expert, []).append(r)
        jobs, keep = [], []
        for e, rs in by_expert.items():
            wgu, wd = self.stores[l].weights(l, e)
            xs = x_host[[r.row for r in rs]].contiguous()
            if self.pool is not None:
                y = torch.empty(len(rs), self.hidden, dtype=torch.bfloat16)
                jobs.append((xs, wgu.contiguous(), wd.contiguous(), y))
            else:
                y = ref.expert_ffn(xs, wgu, wd, self.swiglu_mode)
            keep.append((rs, y))
        if jobs:
            self.pool.run(jobs, self.swiglu_mode)
        out = {}
        for rs, y in keep:
            for i, r in enumerate(rs):
                out[(r.row, r.choice)] = y[i]
        return out

    def _forward_host(self, l, x, w_h, ids_h, d, misses) -> torch.Tensor:
        rows, k = ids_h.shape
        contrib = torch.zeros(rows, k, self.hidden, dtype=torch.float32)
        for r, s in zip(d.hits, d.hit_slots):
            y = ref.expert_ffn(x[r.row: r.row + 1], self.arena_gu[l][s], self.arena_down[l][s], self.swiglu_mode)
            contrib[r.row, r.choice] = y[0].to(torch.float32) * r.weight
        for (row, ch), y in self._cpu_contributions(l, x, misses).items():
            contrib[row, ch] = y.to(torch.float32) * float(w_h[row, ch])
        order = torch.argsort(ids_h.long(), dim=-1, stable=True)
        ordered = torch.gather(contrib, 1, order[:, :, None].expand_as(contrib))
        acc = torch.zeros(rows, self.hidden, dtype=torch.float32)
        for j in range(k):
            acc = acc + ordered[:, j]
        return acc.to(x.dtype)

    def _forward_cuda(self, l, x, weights, ids, misses) -> torch.Tensor:
        from ..ops import moe_cuda
        rows, k = ids.shape
        slot_ids = self.table[l][ids.long()].to(torch.int32)                 # misses -> -1
        n_slots = self.cap.slots_per_layer[l]
        xs, pos, seg_off, counts, cap_rows = moe_cuda.dispatch_local(x.contiguous(), slot_ids.contiguous(), n_slots, 0, n_slots)
        h = moe_cuda.grouped_gemm(xs, self.arena_gu[l], seg_off, counts, cap_rows, epi=1)
        y = moe_cuda.grouped_gemm(h, self.arena_down[l], seg_off, counts, cap_rows, epi=0)
        if misses:
            x_host = x.cpu()
            outs = self._cpu_contributions(l, x_host, misses)
            keys = list(outs)
            y_cpu = torch.stack([outs[kk] for kk in keys]).to(self.device)
            y = torch.cat([y, y_cpu], dim=0)
            idx = torch.tensor([row * k + ch for row, ch in keys], dtype=torch.long, device=self.device)
            pos[idx] = torch.arange(cap_rows, cap_rows + len(keys), dtype=torch.int32, device=self.device)
        return moe_cuda.combine(y, pos, ids.contiguous(), weights.contiguous(), rows, self.hidden)


def build_provider_from_weights(model, resident_fraction: float, device=None, mode: str = "score", threads: int = 8,
                                admission_cap: int | None = None) -> TieredExpertProvider:
    """Move a loaded model's routed experts to the host tier and serve them through GPU slots
    holding ``resident_fraction`` of them (the Qwen3-MoE benchmark runs with 0.5)."""
    from .plan import CpuService, TransferRates, admission_budget, plan_capacity
    spec = model.spec
    w = model.w
    device = torch.device(device) if device is not None else w.embed.device
    moe_layers = [i for i, lw in enumerate(w.layers) if lw.router is not None]
    e_local = w.layers[moe_layers[0]].experts_gu.shape[0]
    f = spec.moe.expert_ffn
    slot_bytes = 3 * f * spec.hidden * w.embed.element_size()
    geo = ExpertGeometry(len(moe_layers), e_local, spec.moe.top_k, slot_bytes)
    cap = plan_capacity(geo, device_expert_bytes=1 << 62, host_bytes=1 << 62, rates=TransferRates(),
                        resident_fraction=resident_fraction)
    adm = admission_budget(geo, TransferRates(), CpuService())
    if admission_cap is not None:
        adm = Admission(adm.bytes_per_token, admission_cap)
    stores = []
    for i in moe_layers:
        lw = w.layers[i]
        stores.append(ExpertStore(lw.experts_gu.cpu(), lw.experts_down.cpu(), pin=device.type == "cuda"))
    prov = TieredExpertProvider(geo, cap, adm, stores, device, spec.hidden, f, mode=mode,
                                swiglu_mode=spec.swiglu_mode, threads=threads)
    prov.layer_index = {ml: j for j, ml in enumerate(moe_layers)}
    for i in moe_layers:                       # the device copies of the experts are no longer needed
        w.layers[i].experts_gu = None
        w.layers[i].experts_down = None
    model.expert_provider = prov
    return prov
