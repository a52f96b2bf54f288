"""Expert capacity planning across HBM / pinned host / NVMe (pure arithmetic, no device calls).

Follows the reference's planner (src/experts/plan.rs:338-405, 1254-1452, 2016-2081):

* **Capacity**: device bytes minus the persistent reserves give the number of GPU slots; slots are
  split equally over the MoE layers with the remainder going to the low layers; host blocks hold
  every expert that is not GPU-resident (plus span headroom, minus the spare blocks kept for
  admissions); whatever does not fit the host arena becomes the disk tier.
* **Admission budget**: bytes per token = (CPU time of one missed expert in every layer) x the
  slower of the H2D / D2H rates (harmonic mean when there is a single copy engine); the hard cap is
  that budget divided by the slot size, in experts per token.
* **Initial residency**: experts ranked per layer by the request's prefill routing frequency, the
  top ``slots_per_layer`` are installed, scores are seeded with ``12 * freq * top_k / total``.

Under expert parallelism every rank plans its own share (``experts_per_layer`` = E / world).
"""
from __future__ import annotations

import dataclasses
import enum
from dataclasses import dataclass, field

F_DECAY = 0.98
THETA_MIN = 1.05
F_SEED_SCALE = 12.0


class Tier(enum.IntEnum):
    GPU = 0
    HOST = 1
    DISK = 2


@dataclass
class ExpertGeometry:
    layers: int                 # MoE layers
    experts_per_layer: int      # experts this rank owns per layer
    top_k: int
    slot_bytes: int             # bytes of one expert's weights in its stored format

    @property
    def total_experts(self) -> int:
        return self.layers * self.experts_per_layer


@dataclass
class TransferRates:
    """Measured by ``ff calibrate`` (src/backend/cuda/calibrate.rs:1292-1620)."""
    h2d_bytes_s: float = 50e9
    d2h_bytes_s: float = 50e9
    copy_engines: int = 2
    disk_bytes_s: float = 5e9
    pinned_extent_bytes: int = 1 << 40       # how much host memory can be page-locked


@dataclass
class CpuService:
    """seconds(rows, experts) table of the CPU expert path; ``per_expert_s`` is the time of one
    missed expert for one row with the planned worker count."""
    per_expert_s: float = 2e-4
    workers: int = 8


@dataclass
class Capacity:
    gpu_slots: int
    slots_per_layer: list[int]
    host_blocks: int
    spare_blocks: int
    disk_experts: int
    host_pinned: bool
    device_expert_bytes: int
    host_bytes: int

    @property
    def all_resident(self) -> bool:
        return self.host_blocks == 0 and self.disk_experts == 0

    def to_json(self) -> dict:
        return dataclasses.asdict(self)


@dataclass
class Admission:
    bytes_per_token: float
    hard_cap: int                 # experts admitted per token at most

    def to_json(self) -> dict:
        return dataclasses.asdict(self)


class PlanError(RuntimeError):
    pass


def admission_budget(geo: ExpertGeometry, rates: TransferRates, cpu: CpuService) -> Admission:
    """How many bytes of expert weights may be promoted per decode token without the copies
    costing more than the CPU work they save."""
    cpu_time = cpu.per_expert_s * geo.layers
    if rates.copy_engines >= 2:
        rate = min(rates.h2d_bytes_s, rates.d2h_bytes_s)
    else:
        rate = 1.0 / (1.0 / rates.h2d_bytes_s + 1.0 / rates.d2h_bytes_s)
    budget = cpu_time * rate
    return Admission(bytes_per_token=budget, hard_cap=int(budget // max(geo.slot_bytes, 1)))


def plan_capacity(geo: ExpertGeometry, device_expert_bytes: int, host_bytes: int, rates: TransferRates,
                  admission_cap: int = 0, span_headroom_blocks: int = 0, resident_fraction: float | None = None
                  ) -> Capacity:
    """``device_expert_bytes``: HBM left for expert slots after weights / KV / workspace reserves.
    ``resident_fraction`` forces the GPU share (e.g. 0.5 = only half of the experts resident)."""
    if geo.layers <= 0 or geo.experts_per_layer <= 0 or geo.slot_bytes <= 0:
        raise PlanError("empty expert geometry")
    max_slots = device_expert_bytes // geo.slot_bytes
    if resident_fraction is not None:
        max_slots = min(max_slots, int(geo.total_experts * resident_fraction))
    gpu_slots = int(min(max_slots, geo.total_experts))
    if gpu_slots < geo.layers * geo.top_k:
        raise PlanError(f"{gpu_slots} GPU slots cannot hold top_k={geo.top_k} experts for each of {geo.layers} layers")
    base, rem = divmod(gpu_slots, geo.layers)
    base = min(base, geo.experts_per_layer)
    per_layer = [min(geo.experts_per_layer, base + (1 if i < rem else 0)) for i in range(geo.layers)]
    gpu_slots = sum(per_layer)
    non_gpu = geo.total_experts - gpu_slots
    if non_gpu == 0:
        return Capacity(gpu_slots, per_layer, 0, 0, 0, True, device_expert_bytes, host_bytes)
    want_blocks = non_gpu + span_headroom_blocks
    spare = min(admission_cap, want_blocks)
    fit = host_bytes // geo.slot_bytes
    host_blocks = int(min(want_blocks, fit))
    disk = max(0, non_gpu - max(0, host_blocks - span_headroom_blocks))
    pinned = host_blocks * geo.slot_bytes <= rates.pinned_extent_bytes
    return Capacity(gpu_slots, per_layer, host_blocks, spare if disk else 0, disk, pinned, device_expert_bytes, host_bytes)


def initial_residency(freq: list[list[float]], slots_per_layer: list[int]) -> list[list[int]]:
    """Per layer: expert ids ranked by routing frequency (ties -> lower id), top ``slots`` kept."""
    out = []
    for layer_freq, slots in zip(freq, slots_per_layer):
        order = sorted(range(len(layer_freq)), key=lambda e: (-layer_freq[e], e))
        out.append(sorted(order[:slots]))
    return out


def seed_scores(freq: list[float], top_k: int) -> list[float]:
    total = sum(freq)
    if total <= 0:
        return [0.0] * len(freq)
    return [F_SEED_SCALE * f * top_k / total for f in freq]


@dataclass
class PeerDecision:
    """Whether serving a layer's experts from another GPU beats the host tier: compare the
    measured hop time with the miss service time (the reference's 2-GPU peer-layer decision,
    src/experts/plan.rs:1322-1369). With NVSwitch expert parallelism this is the EP degree choice."""
    hop_s: float
    miss_service_s: float

    @property
    def use_peer(self) -> bool:
        return self.hop_s < self.miss_service_s


@dataclass
class TierLedger:
    """Exact byte accounting of where every expert lives (src/experts/plan.rs:1470-1830)."""
    slot_bytes: int
    tier: dict[tuple[int, int], Tier] = field(default_factory=dict)

    def place(self, layer: int, expert: int, tier: Tier) -> None:
        self.tier[(layer, expert)] = tier

    def bytes_in(self, tier: Tier) -> int:
        return sum(1 for t in self.tier.values() if t == tier) * self.slot_bytes

    def count(self, tier: Tier) -> int:
        return sum(1 for t in self.tier.values() if t == tier)

    def where(self, layer: int, expert: int) -> Tier:
        return self.tier[(layer, expert)]

    def check(self, cap: Capacity, geo: ExpertGeometry) -> None:
        assert len(self.tier) == geo.total_experts, "every expert must be placed exactly once"
        assert self.count(Tier.GPU) <= cap.gpu_slots
        assert self.count(Tier.DISK) <= cap.disk_experts + cap.spare_blocks
