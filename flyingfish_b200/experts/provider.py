"""Tiered expert provider: serves a MoE layer's routed experts from GPU slots, the pinned host
tier (CPU expert FFN for this token, promotion later) and the NVMe tier (direct-IO ring, then CPU).

Per MoE layer call (the reference's decode executor, src/backend/cuda/engine_moe.rs:1404-1830):

1. on the device the routed ids are remapped to slot numbers through the layer's slot table (misses
   become -1, the dispatch kernels skip them) and a fixed-size summary is built: number of misses,
   bitmap of routed experts, the missed (position, expert) pairs compacted to the front; ONE small
   device-to-host copy carries it,
2. meanwhile the hits run on the device: dispatch -> grouped GEMMs over the slot arena (BF16 slots, or
   packed NVFP4 slots expanded inside the GEMM),
3. the host reads the summary and updates the residency scores in array form (``Residency.account``;
   the CPU path of the tests still walks ``Residency.dispatch`` route by route),
4. misses (if any) run on the host worker pool with the host copy of the weights (disk-tier experts
   are first read through the direct-IO ring); their outputs are uploaded behind the device outputs,
5. ONE combine sums every contribution of a row in ascending expert id.

Calls with many assignments (prefill chunks, large decode batches: ``FF_EXPERT_STREAM_MIN`` or more) do not use
the host FFN at all: the layer's non-resident experts are streamed from the pinned host tier into a staging arena
(two arenas: the next MoE layer's experts are copied while this layer computes), one dispatch covers resident
slots and staged experts, and nothing is read back inside the step (the accounting summary is copied
asynchronously and processed at the token's end). The reference's prefill streams experts through the device the
same way (src/backend/cuda/moe/prefill.rs).

At token end ``finish_token`` returns the admissions; the provider copies those experts into their
slots on a copy stream and records one event per layer, which the next token's call for that layer
waits on (copies for late layers overlap the early layers' compute; the reference orders slot
lifetimes with events the same way, src/experts/arena.rs:485-560).
"""
from __future__ import annotations

import os

import torch

from .. import ops
from ..ops import moe_ops, ref
from .native import ExpertPool
from .plan import Admission, Capacity, ExpertGeometry
from .runtime import EMPTY, Move, Residency, Route


class ExpertStore:
    """Host-side home of one layer's expert weights: a pinned tensor for the host tier, optionally a
    disk reader for experts that do not fit. ``packed``: (gate/up, down) packed NVFP4 stacks on the host (gate/up
    already interleaved for the SwiGLU epilogue) that are uploaded into slots instead of the BF16 matrices; the BF16
    tensors then hold the dequantised (effective) weights the host FFN computes with."""

    def __init__(self, gate_up: torch.Tensor, down: torch.Tensor, pin: bool = False, disk=None, packed=None):
        self.gate_up = gate_up.pin_memory() if pin and not gate_up.is_pinned() else gate_up     # [E, 2f, h]
        self.down = down.pin_memory() if pin and not down.is_pinned() else down                 # [E, h, f]
        self.disk = disk                                                                        # DiskExperts or None
        self.packed = packed
        if packed is not None and pin:
            for st in packed:
                st.codes, st.scales = st.codes.pin_memory(), st.scales.pin_memory()

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
        self.fp4 = stores[0].packed is not None and self.device.type == "cuda"
        if self.fp4:
            from ..ops.moe_cuda import Nvfp4Experts
            u8 = dict(dtype=torch.uint8, device=self.device)

            def arena(n, rows, cols):
                return Nvfp4Experts(torch.zeros(n, rows, cols // 2, **u8), torch.zeros(n, rows, cols // 16, **u8),
                                    torch.ones(n, device=self.device))
            self.arena_gu = [arena(cap.slots_per_layer[l], 2 * ffn, hidden) for l in range(geo.layers)]
            self.arena_down = [arena(cap.slots_per_layer[l], hidden, ffn) for l in range(geo.layers)]
        else:
            self.arena_gu = [torch.zeros(cap.slots_per_layer[l], 2 * ffn, hidden, dtype=dt, device=self.device)
                             for l in range(geo.layers)]
            self.arena_down = [torch.zeros(cap.slots_per_layer[l], hidden, ffn, dtype=dt, device=self.device)
                               for l in range(geo.layers)]
        self.table = [torch.full((geo.experts_per_layer,), EMPTY, dtype=torch.int32, device=self.device)
                      for _ in range(geo.layers)]
        # the inverse map, slot -> expert (EMPTY for a free slot): expert-parallel owners run their grouped GEMMs
        # over the slots and pick each slot's row segment through it
        self.slot_expert = [torch.full((cap.slots_per_layer[l],), EMPTY, dtype=torch.int32, device=self.device)
                            for l in range(geo.layers)]
        self.pool = ExpertPool(threads) if dt == torch.bfloat16 else None
        self.layer_index: dict[int, int] = {}      # model layer number -> MoE layer ordinal
        self.copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.layer_event: list = [None] * geo.layers     # slot copies of a layer still in flight on the copy stream
        self.summary_host: torch.Tensor | None = None    # pinned landing buffer of the per-layer summary
        self.stats = {"cpu_rows": 0, "gpu_rows": 0, "h2d_expert_bytes": 0, "layers_all_hit": 0, "layer_calls": 0,
                      "d2h_summary_bytes": 0}
        self.freq = [[0.0] * geo.experts_per_layer for _ in range(geo.layers)]
        self.collect_freq = False
        # streaming mode (calls with many assignments): staging arenas for a layer's non-resident experts
        self.stream_min = int(os.environ.get("FF_EXPERT_STREAM_MIN", "64"))
        self.stage = None
        self.stage_layer = [-1, -1]
        self.stage_ready: list = [None, None]          # copies into the buffer done (copy stream)
        self.stage_free: list = [None, None]           # last GEMMs reading the buffer done (compute stream)
        self.vtable: list = [None] * geo.layers        # expert -> virtual slot (resident slot, or slots + staged index)
        self.nonres: list = [None] * geo.layers
        self.nonres_dev: list = [None] * geo.layers
        self.pending_acc: dict[int, tuple] = {}        # layer -> (pinned summary, event, assignments) of this token
        self.freq_dev = None
        self.stats.update(streamed_bytes=0, stream_calls=0)

    # -- slot maintenance ----------------------------------------------------------------------
    def apply_moves(self, moves: list[Move]) -> None:
        if not moves:
            return
        cuda = self.device.type == "cuda"
        if cuda:
            # the copies may start once the compute queued so far (which still reads the old slot contents) is done
            self.copy_stream.wait_stream(torch.cuda.current_stream(self.device))
        touched = set()
        for m in moves:
            st = self.stores[m.layer]
            if self.fp4:
                pg, pd = st.packed
                with torch.cuda.stream(self.copy_stream):
                    ag, ad = self.arena_gu[m.layer], self.arena_down[m.layer]
                    ag.codes[m.slot].copy_(pg.codes[m.expert_in], non_blocking=True)
                    ag.scales[m.slot].copy_(pg.scales[m.expert_in], non_blocking=True)
                    ag.global_scale[m.slot: m.slot + 1].copy_(pg.global_scale[m.expert_in: m.expert_in + 1], non_blocking=True)
                    ad.codes[m.slot].copy_(pd.codes[m.expert_in], non_blocking=True)
                    ad.scales[m.slot].copy_(pd.scales[m.expert_in], non_blocking=True)
                    ad.global_scale[m.slot: m.slot + 1].copy_(pd.global_scale[m.expert_in: m.expert_in + 1], non_blocking=True)
            else:
                wgu, wd = st.weights(m.layer, m.expert_in)
                if cuda:
                    from ..ops import moe_cuda
                    with torch.cuda.stream(self.copy_stream):
                        g = wgu.to(self.device, non_blocking=True)
                        self.arena_gu[m.layer][m.slot].copy_(moe_cuda.interleave64(g[None])[0])
                        self.arena_down[m.layer][m.slot].copy_(wd.to(self.device, non_blocking=True))
                else:
                    self.arena_gu[m.layer][m.slot].copy_(wgu)
                    self.arena_down[m.layer][m.slot].copy_(wd)
            if cuda:
                with torch.cuda.stream(self.copy_stream):     # the table entry changes together with the slot
                    if m.expert_out != EMPTY:
                        self.table[m.layer][m.expert_out] = EMPTY
                    self.table[m.layer][m.expert_in] = m.slot
                    self.slot_expert[m.layer][m.slot] = m.expert_in
            else:
                if m.expert_out != EMPTY:
                    self.table[m.layer][m.expert_out] = EMPTY
                self.table[m.layer][m.expert_in] = m.slot
                self.slot_expert[m.layer][m.slot] = m.expert_in
            self.stats["h2d_expert_bytes"] += self.geo.slot_bytes
            touched.add(m.layer)
            self.vtable[m.layer] = None                 # the layer's resident set changed
            for b in range(2):
                if self.stage_layer[b] == m.layer:
                    self.stage_layer[b] = -1
        if cuda:
            # one event per touched layer (copies are queued in move order, so a layer's event also covers it when a
            # later layer's copies follow): the next call for that layer waits on it, nobody else does
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
            for l in touched:
                self.layer_event[l] = ev

    def begin_request(self, prefill_freq: list[list[float]] | None = None) -> None:
        if prefill_freq is None and self.freq_dev is not None:
            fd = self.freq_dev.cpu().tolist()             # routing counts gathered on the device by streamed calls
            self.freq = [[a + b for a, b in zip(fa, fb)] for fa, fb in zip(self.freq, fd)]
            self.freq_dev.zero_()
        f = prefill_freq if prefill_freq is not None else self.freq
        self.apply_moves(self.res.begin_request(f))
        self.res.freeze_prefill_rank(f)

    def begin_token(self) -> None:
        self.res.begin_token()

    def finish_token(self) -> None:
        self._drain_accounting()
        self.apply_moves(self.res.finish_token())

    # -- streaming mode ------------------------------------------------------------------------
    def _drain_accounting(self) -> None:
        """Summaries of this token's streamed layer calls (copied asynchronously while the step ran)."""
        import numpy as np
        for l, (host, ev, n_assign) in sorted(self.pending_acc.items()):
            ev.synchronize()
            sh = host.numpy()                              # [misses, assignments, routed bitmap]
            if self.res.in_token:
                self.res.account_counts(l, np.nonzero(sh[2:])[0], int(sh[1]) - int(sh[0]), int(sh[0]))
        self.pending_acc.clear()

    def _arena_like(self, n: int):
        if self.fp4:
            from ..ops.moe_cuda import Nvfp4Experts
            u8 = dict(dtype=torch.uint8, device=self.device)
            return (Nvfp4Experts(torch.zeros(n, 2 * self.ffn, self.hidden // 2, **u8),
                                 torch.zeros(n, 2 * self.ffn, self.hidden // 16, **u8), torch.ones(n, device=self.device)),
                    Nvfp4Experts(torch.zeros(n, self.hidden, self.ffn // 2, **u8),
                                 torch.zeros(n, self.hidden, self.ffn // 16, **u8), torch.ones(n, device=self.device)))
        dt = self.stores[0].gate_up.dtype
        return (torch.zeros(n, 2 * self.ffn, self.hidden, dtype=dt, device=self.device),
                torch.zeros(n, self.hidden, self.ffn, dtype=dt, device=self.device))

    @staticmethod
    def _first(arena, n: int):
        """The first ``n`` experts of an arena as the grouped kernels' operand."""
        if isinstance(arena, torch.Tensor):
            return arena[:n]
        from ..ops.moe_cuda import Nvfp4Experts
        return Nvfp4Experts(arena.codes[:n], arena.scales[:n], arena.global_scale[:n])

    def _virtual_table(self, l: int) -> None:
        E, n_slots = self.geo.experts_per_layer, self.cap.slots_per_layer[l]
        slot_of = self.res.slot_of[l]
        nonres = [e for e in range(E) if slot_of[e] == EMPTY]
        vt = list(slot_of)
        for i, e in enumerate(nonres):
            vt[e] = n_slots + i
        self.nonres[l] = nonres
        self.vtable[l] = torch.tensor(vt, dtype=torch.int32, device=self.device)
        self.nonres_dev[l] = torch.tensor(nonres, dtype=torch.long, device=self.device)

    def _stage_fill(self, l: int, b: int) -> None:
        """Copy layer ``l``'s non-resident experts from the pinned host tier into staging buffer ``b`` (copy stream)."""
        if self.vtable[l] is None:
            self._virtual_table(l)
        if self.stage is None:
            # sized for a whole layer: before the first request boundary no slot is filled and everything is staged
            n_stage = self.geo.experts_per_layer
            self.stage = [self._arena_like(n_stage), self._arena_like(n_stage)]
        gu, dn = self.stage[b]
        st = self.stores[l]
        cs = self.copy_stream
        if self.stage_free[b] is not None:
            cs.wait_event(self.stage_free[b])
        with torch.cuda.stream(cs):
            for i, e in enumerate(self.nonres[l]):
                if self.fp4:
                    pg, pd = st.packed
                    gu.codes[i].copy_(pg.codes[e], non_blocking=True); gu.scales[i].copy_(pg.scales[e], non_blocking=True)
                    dn.codes[i].copy_(pd.codes[e], non_blocking=True); dn.scales[i].copy_(pd.scales[e], non_blocking=True)
                else:
                    from ..ops import moe_cuda
                    wgu, wd = st.weights(l, e)
                    gu[i].copy_(moe_cuda.interleave64(wgu.to(self.device, non_blocking=True)[None])[0])
                    dn[i].copy_(wd, non_blocking=True)
            if self.fp4 and self.nonres[l]:
                idx = torch.tensor(self.nonres[l], dtype=torch.long)
                n = len(self.nonres[l])
                gu.global_scale[:n].copy_(st.packed[0].global_scale[idx], non_blocking=True)
                dn.global_scale[:n].copy_(st.packed[1].global_scale[idx], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(cs)
        self.stage_ready[b], self.stage_layer[b] = ev, l
        self.stats["streamed_bytes"] += len(self.nonres[l]) * self.geo.slot_bytes

    def _stage_for(self, l: int) -> int:
        """Buffer holding layer ``l``'s non-resident experts (filled now if it is not there), with the next MoE
        layer's copy started into the other buffer."""
        if self.vtable[l] is None:
            self._virtual_table(l)
        b = 0 if self.stage_layer[0] == l else 1 if self.stage_layer[1] == l else (0 if self.stage_layer[0] == -1 else 1)
        if self.stage_layer[b] != l:
            self._stage_fill(l, b)
        nxt = (l + 1) % self.geo.layers
        if nxt != l and self.stage_layer[1 - b] != nxt:
            self._stage_fill(nxt, 1 - b)
        return b

    def _grouped(self, xs, arena, seg_off, counts, capacity, epi, out=None):
        from ..ops import moe_cuda
        if isinstance(arena, torch.Tensor):
            return moe_cuda.grouped_gemm(xs, arena, seg_off, counts, capacity, epi=epi, out=out)
        return moe_cuda.grouped_gemm_nvfp4(xs, arena, seg_off, counts, capacity, epi=epi, out=out)

    def _note_routing(self, l: int, flat: torch.Tensor, n_miss: torch.Tensor, n_assign: int) -> None:
        """Asynchronous accounting summary [misses | routed bitmap] of a streamed call; read at the token's end."""
        E = self.geo.experts_per_layer
        if self.collect_freq:
            if self.freq_dev is None:
                self.freq_dev = torch.zeros(self.geo.layers, E, dtype=torch.float32, device=self.device)
            self.freq_dev[l] += torch.bincount(flat, minlength=E).to(torch.float32)
        if not self.res.in_token:
            return
        routed = torch.zeros(E, dtype=torch.int32, device=self.device)
        routed[flat] = 1
        host = torch.empty(2 + E, dtype=torch.int32, pin_memory=True)
        host.copy_(torch.cat([n_miss.reshape(1).to(torch.int32),
                              torch.tensor([n_assign], dtype=torch.int32, device=self.device), routed]), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self.pending_acc[l] = (host, ev, n_assign)
        self.stats["d2h_summary_bytes"] += 4 * (1 + E)

    def _forward_stream(self, l: int, x: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        from ..ops import moe_cuda
        rows, k = ids.shape
        E, n_slots = self.geo.experts_per_layer, self.cap.slots_per_layer[l]
        cur = torch.cuda.current_stream(self.device)
        if self.layer_event[l] is not None:
            cur.wait_event(self.layer_event[l])
            self.layer_event[l] = None
        b = self._stage_for(l)
        cur.wait_event(self.stage_ready[b])
        flat = ids.reshape(-1).long()
        vs = self.vtable[l][flat].view(rows, k)
        self._note_routing(l, flat, (vs.reshape(-1) >= n_slots).sum(), rows * k)
        # virtual slots: the layer's resident slots (some may still be empty) followed by the staged experts
        n_stage = len(self.nonres[l])
        nv = n_slots + n_stage
        xs, pos, seg_off, counts, cap_rows = moe_cuda.dispatch_local(x.contiguous(), vs.contiguous(), nv, 0, nv)
        gu_s, dn_s = self.stage[b]
        h = torch.empty(cap_rows, self.ffn, dtype=torch.bfloat16, device=self.device)
        y = torch.empty(cap_rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        if n_slots:
            self._grouped(xs, self._first(self.arena_gu[l], n_slots), seg_off, counts, cap_rows, 1, out=h)
        if n_stage:
            self._grouped(xs, self._first(gu_s, n_stage), seg_off[n_slots:], counts[n_slots:], cap_rows, 1, out=h)
        if n_slots:
            self._grouped(h, self._first(self.arena_down[l], n_slots), seg_off, counts, cap_rows, 0, out=y)
        if n_stage:
            self._grouped(h, self._first(dn_s, n_stage), seg_off[n_slots:], counts[n_slots:], cap_rows, 0, out=y)
        fe = torch.cuda.Event()
        fe.record(cur)
        self.stage_free[b] = fe
        self.stats["stream_calls"] += 1
        self.stats["gpu_rows"] += rows * k
        return moe_cuda.combine(y, pos, ids.contiguous(), weights.contiguous(), rows, self.hidden)

    # -- one layer -----------------------------------------------------------------------------
    def forward(self, model_layer: int, x: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        l = self.layer_index[model_layer]
        rows, k = ids.shape
        self.stats["layer_calls"] += 1
        if self.device.type == "cuda":
            if rows * k >= self.stream_min:
                return self._forward_stream(l, x, weights, ids)
            return self._forward_cuda_vec(l, x, weights, ids)
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

    def _forward_cuda_vec(self, l: int, x: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """Device-resolved form of a layer call: no per-route host objects, one small D2H (the summary) per call, a
        second one (the activations of the missed rows) only when something missed."""
        import numpy as np
        from ..ops import moe_cuda
        rows, k = ids.shape
        E = self.geo.experts_per_layer
        n_assign = rows * k
        dev = self.device
        cur = torch.cuda.current_stream(dev)
        if self.layer_event[l] is not None:
            cur.wait_event(self.layer_event[l])
            self.layer_event[l] = None
        flat = ids.reshape(-1).long()
        slot_ids = self.table[l][flat].to(torch.int32).view(rows, k)              # misses -> -1
        miss = slot_ids.reshape(-1) < 0
        routed = torch.zeros(E, dtype=torch.int32, device=dev)
        routed[flat] = 1
        order = torch.argsort(miss.to(torch.int8), descending=True, stable=True)    # missed positions first, ascending
        summary = torch.cat([miss.sum().reshape(1).to(torch.int32), routed, order.to(torch.int32),
                             flat[order].to(torch.int32)])
        need = 1 + E + 2 * n_assign
        if self.summary_host is None or self.summary_host.numel() < need:
            self.summary_host = torch.empty(max(need, 4096), dtype=torch.int32, pin_memory=True)
        self.summary_host[:need].copy_(summary, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(cur)
        self.stats["d2h_summary_bytes"] += 4 * need
        # hits on the device while the summary travels
        n_slots = self.cap.slots_per_layer[l]
        xs, pos, seg_off, counts, cap_rows = moe_cuda.dispatch_local(x.contiguous(), slot_ids.contiguous(), n_slots, 0, n_slots)
        if self.fp4:
            h = moe_cuda.grouped_gemm_nvfp4(xs, self.arena_gu[l], seg_off, counts, cap_rows, epi=1)
            y = moe_cuda.grouped_gemm_nvfp4(h, self.arena_down[l], seg_off, counts, cap_rows, epi=0)
        else:
            h = moe_cuda.grouped_gemm(xs, self.arena_gu[l], seg_off, counts, cap_rows, epi=1)
            y = moe_cuda.grouped_gemm(h, self.arena_down[l], seg_off, counts, cap_rows, epi=0)
        ev.synchronize()
        sh = self.summary_host.numpy()
        n_miss = int(sh[0])
        routed_e = np.nonzero(sh[1: 1 + E])[0]
        miss_pos = sh[1 + E: 1 + E + n_miss].copy()
        miss_exp = sh[1 + E + n_assign: 1 + E + n_assign + n_miss].copy()
        if self.collect_freq:
            f = self.freq[l]
            for e in sh[1 + E + n_assign: 1 + E + 2 * n_assign].tolist():        # every assignment's expert
                f[e] += 1.0
        opened = False
        if not self.res.in_token:          # prefill chunks: no decay / admission, plain accounting
            self.res.in_token = True
            self.res.routed[l].clear()
            opened = True
        self.res.account(l, routed_e, n_assign - n_miss, miss_exp)
        if opened:
            self.res.in_token = False
        self.stats["cpu_rows"] += n_miss
        self.stats["gpu_rows"] += n_assign - n_miss
        if n_miss == 0:
            self.stats["layers_all_hit"] += 1
        else:
            # host FFN of the missed assignments, grouped by expert with array operations
            miss_rows = miss_pos // k
            x_host = x.cpu()
            by = np.argsort(miss_exp, kind="stable")
            y_cpu = torch.empty(n_miss, self.hidden, dtype=x.dtype)
            jobs, i = [], 0
            exp_sorted = miss_exp[by]
            while i < n_miss:
                j = i
                while j < n_miss and exp_sorted[j] == exp_sorted[i]:
                    j += 1
                sel = by[i:j]
                wgu, wd = self.stores[l].weights(l, int(exp_sorted[i]))
                xs_h = x_host[torch.from_numpy(miss_rows[sel].astype(np.int64))].contiguous()
                if self.pool is not None:
                    out = torch.empty(j - i, self.hidden, dtype=torch.bfloat16)
                    jobs.append((xs_h, wgu.contiguous(), wd.contiguous(), out, sel))
                else:
                    y_cpu[torch.from_numpy(sel.astype(np.int64))] = ref.expert_ffn(xs_h, wgu, wd, self.swiglu_mode).to(x.dtype)
                i = j
            if jobs:
                self.pool.run([(a, b, c, d) for a, b, c, d, _ in jobs], self.swiglu_mode)
                for _, _, _, out, sel in jobs:
                    y_cpu[torch.from_numpy(sel.astype(np.int64))] = out
            y = torch.cat([y, y_cpu.to(dev, non_blocking=True)], dim=0)
            idx = torch.from_numpy(miss_pos.astype(np.int64)).to(dev, non_blocking=True)
            pos[idx] = torch.arange(cap_rows, cap_rows + n_miss, dtype=torch.int32, device=dev)
        return moe_cuda.combine(y, pos, ids.contiguous(), weights.contiguous(), rows, self.hidden)

    def ep_experts(self, model_layer: int, recv_x: torch.Tensor, seg_off: torch.Tensor, counts: torch.Tensor,
                   capacity: int, out_y: torch.Tensor, expected_rows: float = 0.0) -> None:
        """Expert phase of an expert-parallel layer on a rank that tiers its own experts. ``recv_x`` holds the rows
        that arrived for this rank's experts, one 16-row padded segment per local expert (``seg_off`` / ``counts`` on
        the device). Resident experts run as grouped GEMMs over the slot arena (slot s takes the segment of the expert
        it holds); the segments of experts that are not resident are computed by the host FFN and written into
        ``out_y`` (the symmetric buffer the peers combine from) behind them. One small D2H (counts and offsets)."""
        import numpy as np
        from ..ops import moe_cuda
        l = self.layer_index[model_layer]
        dev = self.device
        cur = torch.cuda.current_stream(dev)
        if self.layer_event[l] is not None:
            cur.wait_event(self.layer_event[l])
            self.layer_event[l] = None
        self.stats["layer_calls"] += 1
        el = self.geo.experts_per_layer
        if expected_rows >= self.stream_min:
            # many rows: the non-resident experts are streamed through the staging arena, nothing is read back
            b = self._stage_for(l)
            cur.wait_event(self.stage_ready[b])
            n_slots = self.cap.slots_per_layer[l]
            se = self.slot_expert[l].long()
            live = se >= 0
            sel = se.clamp_min(0)
            cnt = counts[:el]
            counts_s = torch.where(live, cnt[sel], torch.zeros_like(sel, dtype=cnt.dtype)).to(torch.int32).contiguous()
            off_s = seg_off[:el][sel].to(torch.int32).contiguous()
            nr = self.nonres_dev[l]
            counts_n = cnt[nr].to(torch.int32).contiguous()
            off_n = seg_off[:el][nr].to(torch.int32).contiguous()
            gu_s, dn_s = self.stage[b]
            h = torch.empty(capacity, self.ffn, dtype=torch.bfloat16, device=dev)
            if n_slots:
                self._grouped(recv_x, self._first(self.arena_gu[l], n_slots), off_s, counts_s, capacity, 1, out=h)
            if nr.numel():
                self._grouped(recv_x, self._first(gu_s, nr.numel()), off_n, counts_n, capacity, 1, out=h)
            if n_slots:
                self._grouped(h, self._first(self.arena_down[l], n_slots), off_s, counts_s, capacity, 0, out=out_y)
            if nr.numel():
                self._grouped(h, self._first(dn_s, nr.numel()), off_n, counts_n, capacity, 0, out=out_y)
            fe = torch.cuda.Event()
            fe.record(cur)
            self.stage_free[b] = fe
            self.stats["stream_calls"] += 1
            if self.collect_freq:
                if self.freq_dev is None:
                    self.freq_dev = torch.zeros(self.geo.layers, el, dtype=torch.float32, device=dev)
                self.freq_dev[l] += cnt.to(torch.float32)
            if self.res.in_token:
                host = torch.empty(2 + el, dtype=torch.int32, pin_memory=True)
                host.copy_(torch.cat([counts_n.sum().reshape(1).to(torch.int32), cnt.sum().reshape(1).to(torch.int32),
                                      (cnt > 0).to(torch.int32)]), non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(cur)
                self.pending_acc[l] = (host, ev, 0)
            return
        meta_h = torch.cat([counts[:el], seg_off[:el]]).cpu().numpy()         # the one synchronising copy
        self.stats["d2h_summary_bytes"] += 8 * el
        counts_h, off_h = meta_h[:el], meta_h[el:]
        # slot-ordered segment arrays for the grouped GEMMs over the arena
        se = self.slot_expert[l].long()
        live = se >= 0
        sel = se.clamp_min(0)
        counts_s = torch.where(live, counts[:el][sel], torch.zeros_like(sel, dtype=counts.dtype)).to(torch.int32).contiguous()
        off_s = seg_off[:el][sel].to(torch.int32).contiguous()
        if self.fp4:
            h = moe_cuda.grouped_gemm_nvfp4(recv_x, self.arena_gu[l], off_s, counts_s, capacity, epi=1)
            moe_cuda.grouped_gemm_nvfp4(h, self.arena_down[l], off_s, counts_s, capacity, epi=0, out=out_y)
        else:
            h = moe_cuda.grouped_gemm(recv_x, self.arena_gu[l], off_s, counts_s, capacity, epi=1)
            moe_cuda.grouped_gemm(h, self.arena_down[l], off_s, counts_s, capacity, epi=0, out=out_y)
        # accounting and the host tier
        slot_of = self.res.slot_of[l]
        routed = np.nonzero(counts_h > 0)[0]
        miss_e = [int(e) for e in routed if slot_of[int(e)] == EMPTY]
        n_hit = int(sum(int(counts_h[e]) for e in routed if slot_of[int(e)] != EMPTY))
        opened = False
        if not self.res.in_token:
            self.res.in_token = True
            self.res.routed[l].clear()
            opened = True
        miss_rows = [e for e in miss_e for _ in range(int(counts_h[e]))]
        self.res.account(l, routed, n_hit, miss_rows)
        if opened:
            self.res.in_token = False
        self.stats["gpu_rows"] += n_hit
        self.stats["cpu_rows"] += len(miss_rows)
        if not miss_e:
            self.stats["layers_all_hit"] += 1
            return
        jobs = []
        for e in miss_e:
            o, c = int(off_h[e]), int(counts_h[e])
            xs_h = recv_x[o: o + c].cpu()
            wgu, wd = self.stores[l].weights(l, e)
            if self.pool is not None:
                out = torch.empty(c, self.hidden, dtype=torch.bfloat16)
                jobs.append((xs_h.contiguous(), wgu.contiguous(), wd.contiguous(), out, o))
            else:
                out_y[o: o + c].copy_(ref.expert_ffn(xs_h, wgu, wd, self.swiglu_mode).to(out_y.dtype))
        if jobs:
            self.pool.run([(a, b, c_, d) for a, b, c_, d, _ in jobs], self.swiglu_mode)
            for _, _, _, out, o in jobs:
                out_y[o: o + out.shape[0]].copy_(out.to(dev, non_blocking=True))

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


def rates_from_calibration(model, settings, device):
    """(TransferRates, CpuService) from ``ff calibrate``'s cache for this model and device (largest measured copy size,
    one-row host FFN time), or the defaults when the cache does not exist."""
    from .plan import CpuService, TransferRates
    rates, cpu = TransferRates(), CpuService()
    if settings is None:
        return rates, cpu
    try:
        from ..planner.calibrate import load_calibration
        cal = load_calibration(getattr(model.spec, "name", None), settings, torch.device(device))
    except Exception:
        cal = None
    if not cal:
        return rates, cpu
    copies = cal.get("copy_rates") or {}
    if copies:
        big = copies[max(copies, key=lambda k: int(k))]
        rates.h2d_bytes_s, rates.d2h_bytes_s = float(big["h2d_bytes_s"]), float(big["d2h_bytes_s"])
    if cal.get("copy_engines"):
        rates.copy_engines = int(cal["copy_engines"])
    if cal.get("disk_bytes_s"):
        rates.disk_bytes_s = float(cal["disk_bytes_s"])
    svc = cal.get("cpu_service") or {}
    table = svc.get("seconds_per_expert_by_rows") or {}
    if table:
        cpu.per_expert_s = float(table[min(table, key=lambda k: int(k))])
        cpu.workers = int(svc.get("workers", cpu.workers))
    return rates, cpu


def _deinterleave64_rows(t: torch.Tensor) -> torch.Tensor:
    """Inverse of the per-64 gate/up row interleave: [2f, ...] rows back to [gate | up]."""
    n = t.shape[0]
    g = t.view(n // 128, 2, 64, *t.shape[1:])
    return torch.cat([g[:, 0].reshape(n // 2, *t.shape[1:]), g[:, 1].reshape(n // 2, *t.shape[1:])], dim=0)


def build_provider_from_weights(model, resident_fraction: float, device=None, mode: str = "score", threads: int = 8,
                                admission_cap: int | None = None, settings=None) -> TieredExpertProvider:
    """Move a loaded model's routed experts to the host tier and serve them through GPU slots
    holding ``resident_fraction`` of them (the Qwen3-MoE benchmark runs with 0.5)."""
    from .plan import CpuService, TransferRates, admission_budget, plan_capacity
    spec = model.spec
    w = model.w
    device = torch.device(device) if device is not None else w.embed.device
    moe_layers = [i for i, lw in enumerate(w.layers) if lw.router is not None]
    e_local = w.layers[moe_layers[0]].experts_gu.shape[0]
    f = spec.moe.expert_ffn
    nvfp4 = spec.moe.expert_format == "nvfp4" and device.type == "cuda" and f % 128 == 0 and spec.hidden % 128 == 0
    slot_bytes = 3 * f * spec.hidden * w.embed.element_size()
    if nvfp4:
        slot_bytes = 3 * f * spec.hidden // 2 + 3 * f * spec.hidden // 16 + 8       # packed codes + E4M3 scales
    geo = ExpertGeometry(len(moe_layers), e_local, spec.moe.top_k, slot_bytes)
    # transfer and host-FFN rates: the calibration cache of this machine when there is one, defaults otherwise
    rates, cpu = rates_from_calibration(model, settings, device)
    cap = plan_capacity(geo, device_expert_bytes=1 << 62, host_bytes=1 << 62, rates=rates,
                        resident_fraction=resident_fraction)
    adm = admission_budget(geo, rates, cpu)
    if admission_cap is not None:
        adm = Admission(adm.bytes_per_token, admission_cap)
    stores = []
    for i in moe_layers:
        lw = w.layers[i]
        packed = None
        if not nvfp4:
            gu_h, dn_h = lw.experts_gu.cpu(), lw.experts_down.cpu()
        else:
            # slots hold the packed codes; the host tier computes with the same effective (dequantised) weights
            from ..loaders import quant as qref
            from ..ops import moe_cuda
            fp4 = lw.extra.pop("experts_fp4", None)
            if fp4 is None:
                fp4 = (moe_cuda.Nvfp4Experts.quantize(lw.experts_gu, gate_up=True), moe_cuda.Nvfp4Experts.quantize(lw.experts_down))
            pg, pd = fp4
            inv = _deinterleave64_rows
            from ..ops.quant_ops import dequant_nvfp4
            gu_h = torch.stack([dequant_nvfp4(inv(pg.codes[e]), inv(pg.scales[e]), pg.global_scale[e]).cpu()
                                for e in range(e_local)])
            dn_h = torch.stack([dequant_nvfp4(pd.codes[e], pd.scales[e], pd.global_scale[e]).cpu() for e in range(e_local)])
            for st in (pg, pd):
                st.codes, st.scales, st.global_scale = st.codes.cpu(), st.scales.cpu(), st.global_scale.cpu()
            packed = (pg, pd)
        stores.append(ExpertStore(gu_h, dn_h, pin=device.type == "cuda", packed=packed))
    prov = TieredExpertProvider(geo, cap, adm, stores, device, spec.hidden, f, mode=mode,
                                swiglu_mode=spec.swiglu_mode, threads=threads)
    prov.layer_index = {ml: j for j, ml in enumerate(moe_layers)}
    for i in moe_layers:                       # the device copies of the experts are no longer needed
        w.layers[i].experts_gu = None
        w.layers[i].experts_down = None
    model.expert_provider = prov
    return prov
