"""Residency runtime: which experts sit in GPU slots, request-boundary installs, per-token
dispatch and decayed-frequency admission (host state machine; device copies are issued by the
provider through the callbacks).

Policy of the reference (src/experts/runtime.rs:464-650, 654-804, 1003-1125):

* ``begin_request(prefill frequency)``: experts ranked per layer by the request's prefill routing
  frequency; the top ``slots_per_layer`` are installed, scores seeded with
  ``12 * freq * top_k / total``.
* per token: ``begin_token`` decays every score by 0.98; ``dispatch(layer, routes)`` adds 1 to every
  routed expert and splits the routes into GPU hits (with the slot's generation), host-tier misses
  and disk-tier misses; ``finish_token`` admits candidates whose score is at least 1.05 and higher
  than the victim's, up to the hard per-token cap; the victim is the lowest-score resident of the
  layer that was not routed this token; every slot change bumps the slot's generation so a stale
  pointer table can be detected.
* GLM / DeepSeek style ``rank`` mode admits decode misses by the frozen prefill expert rank
  instead of the decayed score (src/experts/runtime.rs:1229-1342, 1409-1448).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

from .plan import Admission, Capacity, ExpertGeometry, F_DECAY, THETA_MIN, Tier, TierLedger, initial_residency, seed_scores

EMPTY = -1


@dataclass
class Route:
    row: int
    choice: int
    expert: int
    weight: float


@dataclass
class Dispatch:
    """Result of routing one layer's token rows against the current residency."""
    hits: list[Route] = field(default_factory=list)
    hit_slots: list[int] = field(default_factory=list)          # slot index inside the layer
    hit_generations: list[int] = field(default_factory=list)
    host: list[Route] = field(default_factory=list)
    disk: list[Route] = field(default_factory=list)
    host_experts: list[int] = field(default_factory=list)       # distinct, in first-seen order
    disk_experts: list[int] = field(default_factory=list)


@dataclass
class Move:
    """One slot change decided at a token / request boundary."""
    layer: int
    slot: int
    expert_in: int
    expert_out: int            # EMPTY when the slot was free
    generation: int
    write_back: bool = False   # evicted expert must be copied to a free host block


class Residency:
    def __init__(self, geo: ExpertGeometry, cap: Capacity, admission: Admission, mode: str = "score",
                 host_backed: bool = True, disk_experts: set[tuple[int, int]] | None = None):
        assert mode in ("score", "rank")
        self.geo, self.cap, self.adm, self.mode = geo, cap, admission, mode
        self.host_backed = host_backed              # every expert also has a host copy (no write-back needed)
        L, E = geo.layers, geo.experts_per_layer
        self.slot_of = [[EMPTY] * E for _ in range(L)]                      # expert -> slot
        self.expert_in = [[EMPTY] * cap.slots_per_layer[l] for l in range(L)]   # slot -> expert
        self.generation = [[0] * cap.slots_per_layer[l] for l in range(L)]
        self.score = [[0.0] * E for _ in range(L)]
        self.routed = [set() for _ in range(L)]                              # experts routed this token
        self.rank = [[0] * E for _ in range(L)]                              # frozen prefill rank (lower = better)
        self.disk = disk_experts or set()
        self.ledger = TierLedger(geo.slot_bytes)
        for l in range(L):
            for e in range(E):
                self.ledger.place(l, e, Tier.DISK if (l, e) in self.disk else Tier.HOST)
        self.stats = {"hits": 0, "host_misses": 0, "disk_misses": 0, "admitted": 0, "evicted": 0, "tokens": 0}
        self.in_token = False

    # -- request boundary ----------------------------------------------------------------------
    def begin_request(self, prefill_freq: list[list[float]]) -> list[Move]:
        """Install the request's hottest experts; returns the slot moves to perform."""
        want = initial_residency(prefill_freq, self.cap.slots_per_layer)
        moves: list[Move] = []
        for l, experts in enumerate(want):
            seeds = seed_scores(prefill_freq[l], self.geo.top_k)
            self.score[l] = list(seeds)
            order = sorted(range(len(prefill_freq[l])), key=lambda e: (-prefill_freq[l][e], e))
            for r, e in enumerate(order):
                self.rank[l][e] = r
            keep = set(experts)
            free = [s for s, e in enumerate(self.expert_in[l]) if e == EMPTY or e not in keep]
            for e in experts:
                if self.slot_of[l][e] != EMPTY:
                    continue
                s = free.pop(0)
                moves.append(self._install(l, s, e))
        return moves

    def freeze_prefill_rank(self, prefill_freq: list[list[float]]) -> None:
        for l, f in enumerate(prefill_freq):
            order = sorted(range(len(f)), key=lambda e: (-f[e], e))
            for r, e in enumerate(order):
                self.rank[l][e] = r

    def _install(self, l: int, s: int, e: int) -> Move:
        out = self.expert_in[l][s]
        if out != EMPTY:
            self.slot_of[l][out] = EMPTY
            self.ledger.place(l, out, Tier.DISK if (l, out) in self.disk and not self.host_backed else Tier.HOST)
            self.stats["evicted"] += 1
        self.expert_in[l][s] = e
        self.slot_of[l][e] = s
        self.generation[l][s] += 1
        self.ledger.place(l, e, Tier.GPU)
        return Move(l, s, e, out, self.generation[l][s], write_back=(out != EMPTY and not self.host_backed))

    # -- token loop ----------------------------------------------------------------------------
    def begin_token(self) -> None:
        assert not self.in_token, "finish_token was not called"
        self.in_token = True
        for l in range(self.geo.layers):
            sc = self.score[l]
            for e in range(len(sc)):
                sc[e] *= F_DECAY
            self.routed[l].clear()
        self.stats["tokens"] += 1

    def dispatch(self, layer: int, routes: list[Route]) -> Dispatch:
        assert self.in_token, "dispatch outside begin_token / finish_token"
        d = Dispatch()
        seen_host, seen_disk = set(), set()
        counted = set()
        for r in routes:
            if not 0 <= r.expert < self.geo.experts_per_layer:
                raise ValueError(f"route names expert {r.expert} outside the layer")
            if r.expert not in counted:                      # +1 per token per expert, not per row
                self.score[layer][r.expert] += 1.0
                counted.add(r.expert)
            self.routed[layer].add(r.expert)
            s = self.slot_of[layer][r.expert]
            if s != EMPTY:
                d.hits.append(r); d.hit_slots.append(s); d.hit_generations.append(self.generation[layer][s])
                self.stats["hits"] += 1
            elif (layer, r.expert) in self.disk:
                d.disk.append(r)
                if r.expert not in seen_disk:
                    seen_disk.add(r.expert); d.disk_experts.append(r.expert)
                self.stats["disk_misses"] += 1
            else:
                d.host.append(r)
                if r.expert not in seen_host:
                    seen_host.add(r.expert); d.host_experts.append(r.expert)
                self.stats["host_misses"] += 1
        return d

    def account_counts(self, layer: int, routed_experts, n_hits: int, n_miss: int) -> None:
        """Accounting of a layer call whose misses were served by streaming the experts through the staging arena:
        scores and routed marks as in :meth:`account`, misses counted against the host tier."""
        assert self.in_token
        sc, rt = self.score[layer], self.routed[layer]
        for e in routed_experts:
            e = int(e)
            sc[e] += 1.0
            rt.add(e)
        self.stats["hits"] += int(n_hits)
        self.stats["host_misses"] += int(n_miss)

    def account(self, layer: int, routed_experts, n_hits: int, miss_experts) -> tuple[list[int], list[int]]:
        """Array form of :meth:`dispatch` for callers that resolved the slots on the device: ``routed_experts`` are the
        distinct experts the token rows named (+1 score each, marked as routed this token), ``n_hits`` the
        assignments served from slots, ``miss_experts`` the expert of every missed assignment. Returns the positions
        (into ``miss_experts``) that go to the host tier and to the disk tier."""
        assert self.in_token, "account outside begin_token / finish_token"
        sc, rt = self.score[layer], self.routed[layer]
        for e in routed_experts:
            e = int(e)
            sc[e] += 1.0
            rt.add(e)
        host, disk = [], []
        for i, e in enumerate(miss_experts):
            (disk if (layer, int(e)) in self.disk else host).append(i)
        self.stats["hits"] += int(n_hits)
        self.stats["host_misses"] += len(host)
        self.stats["disk_misses"] += len(disk)
        return host, disk

    def finish_token(self) -> list[Move]:
        """Admit up to ``hard_cap`` experts across all layers; returns the slot moves."""
        assert self.in_token
        self.in_token = False
        cands: list[tuple[float, int, int]] = []
        for l in range(self.geo.layers):
            for e in self.routed[l]:
                if self.slot_of[l][e] == EMPTY:
                    key = self.score[l][e] if self.mode == "score" else -float(self.rank[l][e])
                    cands.append((key, l, e))
        cands.sort(key=lambda t: (-t[0], t[1], t[2]))
        moves: list[Move] = []
        for key, l, e in cands:
            if len(moves) >= self.adm.hard_cap:
                break
            victim_slot, victim_key = self._victim(l)
            if victim_slot is None:
                continue
            if self.mode == "score":
                if self.score[l][e] < THETA_MIN or self.score[l][e] - victim_key <= 0.0:
                    continue
            else:
                if victim_key is not None and -float(self.rank[l][e]) <= victim_key:
                    continue
            moves.append(self._install(l, victim_slot, e))
            self.stats["admitted"] += 1
        return moves

    def _victim(self, l: int):
        """Free slot first; else the lowest-score resident that was not routed this token."""
        best_slot, best_key = None, None
        for s, e in enumerate(self.expert_in[l]):
            if e == EMPTY:
                return s, float("-inf")
            if e in self.routed[l]:
                continue
            key = self.score[l][e] if self.mode == "score" else -float(self.rank[l][e])
            if best_key is None or key < best_key or (key == best_key and e < self.expert_in[l][best_slot]):
                best_slot, best_key = s, key
        return best_slot, best_key

    # -- views ---------------------------------------------------------------------------------
    def resident(self, layer: int) -> list[int]:
        return sorted(e for e in self.expert_in[layer] if e != EMPTY)

    def slot_table(self, layer: int) -> list[int]:
        """expert -> slot (or -1) for the device-side id remap."""
        return list(self.slot_of[layer])

    def hit_rate(self) -> float:
        total = self.stats["hits"] + self.stats["host_misses"] + self.stats["disk_misses"]
        return self.stats["hits"] / total if total else 1.0
