"""Per-machine calibration and the setup closure.

``ff calibrate`` measures, once per machine + model, what the planners need and cannot know
statically: host<->device copy rates at one-slot and top-k-slot sizes, peer (NVLink) copy rates at
4 KiB / 8 MiB / 68 MiB, decode-attention timings per capacity bucket, the skinny / large GEMM
crossover, the CPU expert service table ``seconds(rows)`` for the worker pool, host memory under
the cgroup limit, and the disk read rate. Results are cached as JSON in the runtime directory
under a key of (device uuid, driver, kernel-library hash) and re-used by every later start; the
runtime directory must not sit inside a ``models`` directory. (Reference:
src/backend/cuda/calibrate.rs:396-580, 1292-1854; cache key src/backend/setup.rs:223-262.)

``Closure`` is the small state machine that keeps measurement out of normal start-up:
``Setup`` (measuring allowed) -> ``Frozen`` (plans fixed, graphs may be captured, captures are
counted) -> ``Ready`` (serving; any attempt to measure or to plan a new shape raises). Mirrors
src/backend/cuda/closure.rs:19-35, 293-400.
"""
from __future__ import annotations

import enum
import hashlib
import json
import os
import time
from dataclasses import dataclass, field
from pathlib import Path

import torch

from ..config import Settings, named_shape, read_model_spec
from ..utils.log import log_json

CAPACITY_BUCKETS = (2048, 16384, 49152, 98304, 131072)       # decode-attention plan buckets


class ClosureError(RuntimeError):
    pass


class ClosureState(enum.Enum):
    SETUP = 0
    FROZEN = 1
    READY = 2


@dataclass
class Closure:
    state: ClosureState = ClosureState.SETUP
    shapes: set = field(default_factory=set)         # declared (rows, out, in) linear shapes
    captures: int = 0
    measurements: int = 0

    def measure(self, what: str) -> None:
        if self.state is not ClosureState.SETUP:
            raise ClosureError(f"measurement {what!r} attempted after setup was frozen; run `ff calibrate` first")
        self.measurements += 1

    def declare_shape(self, shape: tuple) -> None:
        if self.state is ClosureState.READY and shape not in self.shapes:
            raise ClosureError(f"shape {shape} was not declared during setup")
        self.shapes.add(shape)

    def freeze(self) -> None:
        if self.state is not ClosureState.SETUP:
            raise ClosureError("closure is already frozen")
        self.state = ClosureState.FROZEN

    def capture(self) -> None:
        if self.state is ClosureState.SETUP:
            raise ClosureError("graphs are captured after setup is frozen")
        self.captures += 1

    def ready(self) -> None:
        if self.state is not ClosureState.FROZEN:
            raise ClosureError("closure must be frozen before it becomes ready")
        self.state = ClosureState.READY


@dataclass(frozen=True)
class CacheKey:
    device_uuid: str
    driver: str
    binary: str

    def filename(self, model: str) -> str:
        h = hashlib.sha256(f"{self.device_uuid}|{self.driver}|{self.binary}|{model}".encode()).hexdigest()[:16]
        return f"calibration-{h}.json"


def check_runtime_dir(path: Path) -> Path:
    p = Path(path).expanduser().resolve()
    if any(part == "models" for part in p.parts):
        raise ClosureError(f"runtime directory {p} must not be inside a 'models' directory")
    return p


def kernel_library_hash() -> str:
    from ..ops import build
    files = build.kernel_sources() + sorted(build.CSRC.glob("*.cuh")) + sorted(build.CSRC.glob("*.h"))
    h = hashlib.sha256()
    for f in files:
        h.update(f.read_bytes())
    return h.hexdigest()[:16]


def cache_key(device: torch.device) -> CacheKey:
    if device.type == "cuda":
        p = torch.cuda.get_device_properties(device)
        uuid = str(getattr(p, "uuid", p.name))
        driver = str(torch.version.cuda)
    else:
        uuid, driver = "cpu", "none"
    return CacheKey(uuid, driver, kernel_library_hash())


def host_memory_limit() -> int:
    """Host RAM available to this process, honouring cgroup v2 / v1 limits
    (src/backend/cuda/calibrate.rs:583-823)."""
    import psutil
    total = psutil.virtual_memory().total
    for f in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
        try:
            v = Path(f).read_text().strip()
            if v != "max":
                total = min(total, int(v))
        except (OSError, ValueError):
            pass
    return total


def _time_cuda(fn, iters: int = 5) -> float:
    fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record(); torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e-3)
    return best


def measure_copy_rates(device: torch.device, sizes: tuple[int, ...]) -> dict:
    out = {}
    for n in sizes:
        host = torch.empty(n, dtype=torch.uint8, pin_memory=True)
        dev = torch.empty(n, dtype=torch.uint8, device=device)
        out[str(n)] = {"h2d_bytes_s": n / _time_cuda(lambda: dev.copy_(host, non_blocking=True)),
                       "d2h_bytes_s": n / _time_cuda(lambda: host.copy_(dev, non_blocking=True))}
    return out


def measure_peer_rates(device: torch.device) -> dict:
    out = {}
    if torch.cuda.device_count() < 2:
        return out
    peer = torch.device("cuda", (device.index + 1) % torch.cuda.device_count())
    for n in (4096, 8 << 20, 68 << 20):
        a = torch.empty(n, dtype=torch.uint8, device=device)
        b = torch.empty(n, dtype=torch.uint8, device=peer)
        out[str(n)] = {"bytes_s": n / _time_cuda(lambda: b.copy_(a, non_blocking=True))}
    return out


def measure_cpu_service(hidden: int, ffn: int, workers: int, rows=(1, 4, 16)) -> dict:
    from ..experts.native import ExpertPool, cpu_arm
    g = torch.Generator().manual_seed(0)
    wgu = (torch.randn(2 * ffn, hidden, generator=g) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(hidden, ffn, generator=g) * 0.02).to(torch.bfloat16)
    pool = ExpertPool(workers)
    table = {}
    for r in rows:
        x = torch.randn(r, hidden, generator=g).to(torch.bfloat16)
        jobs = [(x, wgu, wd, torch.empty(r, hidden, dtype=torch.bfloat16)) for _ in range(workers)]
        pool.run(jobs)
        t0 = time.perf_counter()
        pool.run(jobs)
        table[str(r)] = (time.perf_counter() - t0) / workers * workers / max(workers, 1)
    pool.close()
    return {"arm": cpu_arm(), "workers": workers, "seconds_per_expert_by_rows": table}


def measure_disk_rate(runtime_dir: Path, nbytes: int = 64 << 20) -> float:
    from ..experts.native import DirectReader
    p = runtime_dir / "disk-probe.bin"
    if not p.exists():
        p.write_bytes(os.urandom(1 << 20) * (nbytes >> 20))
    rd = DirectReader(2)
    fd = rd.open(str(p))
    buf = torch.empty(nbytes, dtype=torch.uint8)
    t0 = time.perf_counter()
    rd.wait(rd.submit(fd, 0, nbytes, buf), timeout_ms=60000)
    dt = time.perf_counter() - t0
    rd.close()
    p.unlink()
    return nbytes / dt


# ------------------------------------------------------------------------------------------------
# Kernel choices: decode-GEMM decompositions and the split-KV plan of decode attention, measured on the shapes of
# the model (the reference's linear-algorithm and decode-attention-plan calibration, src/backend/cuda/calibrate.rs:396-580,
# src/backend/cuda/linear_calibrate.rs). The winners go into the calibration file; ``apply_kernel_choices`` hands
# them to the kernel library when a model is loaded.
# ------------------------------------------------------------------------------------------------
def decode_linear_shapes(spec, tp: int = 1) -> list[tuple[str, int, int, int]]:
    """(name, N, K, epilogue id) of the decode projections of a dense / GQA layer on one rank of ``tp``."""
    d, h = spec.head_dim, spec.hidden
    hq, hkv = spec.heads // tp, max(1, spec.kv_heads // tp)
    f = spec.ffn // tp
    fused_rope = d == 128 and not spec.qk_norm
    return [("qkv", (hq + 2 * hkv) * d, h, 2 if fused_rope else 0), ("o", h, hq * d, 0), ("gate_up", 2 * f, h, 1),
            ("down", h, f, 0)]


def linear_candidates(epi: int) -> list[tuple[int, int]]:
    rows = (128,) if epi else (64, 96, 128)
    return [(1, 128)] + [(s, r) for s in (2, 4, 8) for r in rows]


def measure_linear_choices(spec, tp: int = 1, m: int = 64, iters: int = 12) -> dict:
    """Times every launchable decomposition of every decode projection at ``m`` rows (cold L2) and returns
    {name: {"n", "k", "epi", "s", "rows", "us", "default_us", "tried"}}. Leaves the winners installed."""
    from .. import ops
    from ..ops.lib import kernels
    from ..utils.kbench import Flusher, time_op
    import ctypes
    dev = torch.device("cuda")
    lib, flush, out = kernels(), Flusher(dev), {}
    for name, n, k, epi in decode_linear_shapes(spec, tp):
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        w = (torch.randn(n, k, device=dev) * 0.05).to(torch.bfloat16)
        # the rotary epilogue is timed through the plain epilogue with its tile constraint (128-row tiles)
        fn = (lambda: ops.linear_swiglu(x, w)) if epi == 1 and n % 256 == 0 else (lambda: ops.linear(x, w))
        lib.ff_gemm_skinny_set_choice(n, k, epi, 0, 0)
        cfg = (ctypes.c_int * 5)()
        lib.ff_gemm_skinny_config(m, n, k, epi, cfg)
        key_epi = epi if (epi == 1 and n % 256 == 0) else 0
        default_us = time_op(fn, iters, 3, flush)["us_median"]
        best, tried = (cfg[0], cfg[1], default_us), 0
        for s_, r_ in linear_candidates(epi):
            lib.ff_gemm_skinny_set_choice(n, k, key_epi, s_, r_)
            got = (ctypes.c_int * 5)()
            lib.ff_gemm_skinny_config(m, n, k, key_epi, got)
            if (got[0], got[1]) != (s_, r_):               # not launchable on this device: the plan ignored it
                continue
            tried += 1
            us = time_op(fn, iters, 3, flush)["us_median"]
            if us < best[2] * 0.97:                         # a change must win by more than the timer's noise
                best = (s_, r_, us)
        lib.ff_gemm_skinny_set_choice(n, k, key_epi, 0, 0)
        if best[2] < default_us:
            for e in {epi, key_epi}:
                lib.ff_gemm_skinny_set_choice(n, k, e, best[0], best[1])
        out[name] = {"n": n, "k": k, "epi": epi, "s": best[0], "rows": best[1], "us": best[2], "default_us": default_us,
                     "tried": tried, "calibrated": best[2] < default_us}
    return out


def measure_attention_plan(spec, tp: int = 1, cases=((64, 1100), (8, 4096), (1, 8192)), iters: int = 10) -> dict:
    """Times the split-KV decode attention for every wave target and returns the one with the least total time."""
    from ..ops.lib import kernels
    from ..utils import kbench
    lib, res = kernels(), {}
    hq, hkv = spec.heads // tp, max(1, spec.kv_heads // tp)
    for waves in (1, 2, 4, 8):
        lib.ff_attn_decode_set_waves(waves)
        tot = 0.0
        for batch, ctx in cases:
            class B: pass
            b = B(); b.batch, b.ctx, b.hq, b.hkv, b.iters, b.warmup, b.no_flush = batch, ctx, hq, hkv, iters, 2, False
            tot += kbench.bench_attn_decode(b)["us_median"]
        res[str(waves)] = tot
    best = min(res, key=lambda w: res[w])
    if res[best] > res["4"] * 0.97:
        best = "4"
    lib.ff_attn_decode_set_waves(int(best))
    return {"waves": int(best), "total_us_by_waves": res, "cases": [list(c) for c in cases]}


def apply_kernel_choices(data: dict | None) -> int:
    """Install the choices of a calibration record into the kernel library; returns how many were applied."""
    if not data or not torch.cuda.is_available():
        return 0
    from ..ops.lib import kernels
    lib, n = kernels(), 0
    for c in (data.get("linear_choices") or {}).values():
        if c.get("calibrated"):
            key_epi = c["epi"] if (c["epi"] == 1 and c["n"] % 256 == 0) else 0
            for e in {c["epi"], key_epi}:
                lib.ff_gemm_skinny_set_choice(int(c["n"]), int(c["k"]), int(e), int(c["s"]), int(c["rows"]))
            n += 1
    plan = data.get("attention_plan")
    if plan and int(plan.get("waves", 4)) != 4:
        lib.ff_attn_decode_set_waves(int(plan["waves"]))
        n += 1
    return n


def calibrate(model: str | None, settings: Settings, force: bool = False, cpu: bool = False) -> dict:
    device = torch.device("cpu") if cpu or not torch.cuda.is_available() else torch.device("cuda", settings.device)
    rt = check_runtime_dir(settings.resolved_runtime_dir())
    rt.mkdir(parents=True, exist_ok=True)
    name = Path(model).name if model else "none"
    key = cache_key(device)
    path = rt / key.filename(name)
    if path.exists() and not force:
        data = json.loads(path.read_text())
        data["cached"] = True
        return data
    closure = Closure()
    spec = None
    if model:
        spec = read_model_spec(model) if Path(model).is_dir() else named_shape(model)
    data: dict = {"key": key.__dict__, "model": name, "device": str(device), "host_memory_bytes": host_memory_limit(),
                  "capacity_buckets": list(CAPACITY_BUCKETS), "cached": False}
    closure.measure("disk")
    data["disk_bytes_s"] = measure_disk_rate(rt)
    if spec is not None and spec.moe is not None:
        closure.measure("cpu_service")
        data["cpu_service"] = measure_cpu_service(spec.hidden, spec.moe.expert_ffn, min(8, os.cpu_count() or 1))
        slot = 3 * spec.moe.expert_ffn * spec.hidden * 2
        sizes = (slot, slot * spec.moe.top_k)
    else:
        sizes = (1 << 20, 64 << 20)
    if device.type == "cuda":
        closure.measure("copies")
        data["copy_rates"] = measure_copy_rates(device, sizes)
        data["copy_engines"] = getattr(torch.cuda.get_device_properties(device), "async_engine_count", 2) or 2
        data["peer_rates"] = measure_peer_rates(device)
        from ..utils import kbench
        closure.measure("linear")
        lin = {}
        for m in (1, 16, 64, 128, 256):
            class A: pass
            a = A(); a.m, a.n, a.k, a.iters, a.warmup, a.no_flush, a.torch = m, 4096, 4096, 5, 2, False, False
            lin[str(m)] = kbench.bench_gemm(a)["us_median"]
        data["linear_us_by_rows"] = lin
        closure.measure("attention")
        att = {}
        for cap in CAPACITY_BUCKETS[:2]:
            class B: pass
            b = B(); b.batch, b.ctx, b.hq, b.hkv, b.iters, b.warmup, b.no_flush = 1, cap, 32, 8, 5, 2, False
            att[str(cap)] = kbench.bench_attn_decode(b)["us_median"]
        data["decode_attention_us_by_capacity"] = att
        if spec is not None and spec.mla is None and spec.head_dim == 128 and not spec.extra.get("v41"):
            closure.measure("linear_choices")
            data["linear_choices"] = measure_linear_choices(spec, max(settings.tp, 1))
            closure.measure("attention_plan")
            data["attention_plan"] = measure_attention_plan(spec, max(settings.tp, 1))
    closure.freeze()
    data["measurements"] = closure.measurements
    path.write_text(json.dumps(data, indent=1))
    log_json("expert_calibration", verbose_only=True, path=str(path))
    return data


def load_calibration(model: str | None, settings: Settings, device: torch.device) -> dict | None:
    rt = check_runtime_dir(settings.resolved_runtime_dir())
    name = Path(model).name if model else "none"
    p = rt / cache_key(device).filename(name)
    return json.loads(p.read_text()) if p.exists() else None
