"""Prefill span planning: for a whole span of prompt rows, decide per layer how each routed expert
is served -- already resident, staged (streamed into staging slots in cohorts that are reused by
every row wave of the span) or computed on the CPU -- by comparing the measured copy time of the
expert with the CPU service time at its routed row count (src/experts/span.rs:14-45, 97-336).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

from .plan import CpuService, TransferRates


class ExpertClass(enum.Enum):
    RESIDENT = 0
    STAGED = 1
    CPU = 2


@dataclass
class Cohort:
    experts: list[int]
    bytes: int


@dataclass
class LayerSpanPlan:
    classes: dict[int, ExpertClass] = field(default_factory=dict)
    cohorts: list[Cohort] = field(default_factory=list)
    cpu_rows: int = 0
    staged_bytes: int = 0


def plan_layer(routed_rows: dict[int, int], resident: set[int], slot_bytes: int, staging_slots: int,
               rates: TransferRates, cpu: CpuService, forced_waves: int | None = None) -> LayerSpanPlan:
    """``routed_rows``: expert -> number of span rows routed to it. Experts whose H2D copy is cheaper
    than running their rows on the host are staged; cohorts hold at most ``staging_slots`` experts
    and are ordered by decreasing row count (the busiest experts stream first)."""
    plan = LayerSpanPlan()
    copy_s = slot_bytes / rates.h2d_bytes_s
    staged: list[tuple[int, int]] = []
    for e, rows in routed_rows.items():
        if rows <= 0:
            continue
        if e in resident:
            plan.classes[e] = ExpertClass.RESIDENT
            continue
        cpu_s = cpu.per_expert_s * rows / max(cpu.workers, 1) + cpu.per_expert_s * 0.25
        if staging_slots > 0 and copy_s < cpu_s:
            plan.classes[e] = ExpertClass.STAGED
            staged.append((rows, e))
        else:
            plan.classes[e] = ExpertClass.CPU
            plan.cpu_rows += rows
    staged.sort(key=lambda t: (-t[0], t[1]))
    per = staging_slots if forced_waves is None else max(1, -(-len(staged) // forced_waves))
    for i in range(0, len(staged), max(per, 1)):
        chunk = [e for _, e in staged[i: i + per]]
        plan.cohorts.append(Cohort(chunk, len(chunk) * slot_bytes))
        plan.staged_bytes += len(chunk) * slot_bytes
    return plan
