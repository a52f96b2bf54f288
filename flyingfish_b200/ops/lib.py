"""ctypes binding of the native libraries.

``kernels()`` returns the handle of ``_ff_kernels.so`` (CUDA launchers), ``host()`` the handle of
``_ff_host.so`` (CPU expert FFN, direct-IO reader). Both are built in-tree by
:mod:`flyingfish_b200.ops.build`; if a library is missing it is compiled on first use, and if that
is impossible on a machine that has a GPU the import fails loudly -- there is no silent PyTorch
fallback for the CUDA path.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
# FLYINGFISH_TIMELINE=1 loads the tracing build of the kernels and enlarges the status buffer
# (word 8 = record count, 16-byte records from word 16 on; see utils/timeline.py).
TIMELINE = os.environ.get("FLYINGFISH_TIMELINE", "0") == "1"
TIMELINE_CAP = 1 << 18
# FLYINGFISH_DEBUG_CHECKS=1 loads the checking build: single-writer ledger (word 9 = launch epoch, word 10 = entries
# per region, word 11 = claims outside a region, ledger from word 16 on) and extra in-kernel bounds words.
DEBUG_CHECKS = os.environ.get("FLYINGFISH_DEBUG_CHECKS", "0") == "1"
DEBUG_REGIONS, DEBUG_REGION_LEN = 4, 1 << 19
_lock = threading.Lock()
_kernels: ctypes.CDLL | None = None
_host: ctypes.CDLL | None = None


class KernelError(RuntimeError):
    """A launcher refused its arguments or the CUDA runtime reported a launch error."""


_HOST_ERR = {
    -1: "bad shape", -2: "bad alignment", -3: "CUDA driver entry point unavailable",
    -4: "tensor-map encode failed", -5: "size beyond the supported maximum", -6: "unsupported configuration",
}


def kernels() -> ctypes.CDLL:
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                from . import build
                path = build.build_kernels(timeline=TIMELINE, debug_checks=DEBUG_CHECKS and not TIMELINE)
                lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
                _kernels = _EpochProxy(lib) if DEBUG_CHECKS and not TIMELINE else lib
    return _kernels


class _EpochProxy:
    """Checking build only: every launcher call first bumps the launch epoch of the current device's status buffer, so
    that the single-writer ledger tells a second write inside one launch from the write of the next launch."""

    def __init__(self, lib: ctypes.CDLL):
        self._lib = lib

    def __getattr__(self, name: str):
        fn = getattr(self._lib, name)
        if not name.startswith("ff_") or name.endswith("_plan") or name.endswith("_workspace"):
            return fn

        def call(*args):
            if torch.cuda.is_available():
                status_tensor()[9:10].add_(1)
            return fn(*args)
        return call


def host() -> ctypes.CDLL:
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                from . import build
                path = build.build_host()
                if path is None:
                    raise KernelError("native host library has no sources")
                _host = ctypes.CDLL(str(path))
    return _host


def check(rc: int, name: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise KernelError(f"{name}: {_HOST_ERR.get(rc, 'host error')} ({rc})")
    raise KernelError(f"{name}: CUDA error {rc}")


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# ------------------------------------------------------------------------------------------
# Device status word: int32[4] = (code, kernel id, detail0, detail1) per device.
# ------------------------------------------------------------------------------------------
_status: dict[int, torch.Tensor] = {}

STATUS_CODES = {0: "ok", 1: "timeout", 2: "contract", 3: "bounds", 4: "non-finite", 5: "capacity", 6: "double write"}


def debug_ledger_stats(device=None) -> dict:
    """Checking build: launch epochs so far, entries claimed at least once per region, claims that fell outside a
    region (synchronising)."""
    t = status_tensor(device)
    if not DEBUG_CHECKS or t.numel() < 16 + DEBUG_REGIONS * DEBUG_REGION_LEN:
        return {}
    led = t[16:].view(DEBUG_REGIONS, DEBUG_REGION_LEN)
    return {"epoch": int(t[9]), "claimed": [int((led[r] != 0).sum()) for r in range(DEBUG_REGIONS)], "uncovered": int(t[11])}


class DeviceStatusError(RuntimeError):
    def __init__(self, code: int, kernel: int, d0: int, d1: int):
        super().__init__(f"device status: {STATUS_CODES.get(code, code)} from kernel id {kernel} "
                         f"(detail {d0}, {d1})")
        self.code, self.kernel, self.detail = code, kernel, (d0, d1)


def status_tensor(device: torch.device | int | None = None) -> torch.Tensor:
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if dev is None:
        dev = torch.cuda.current_device()
    t = _status.get(dev)
    if t is None:
        if TIMELINE:
            n = 16 + 4 * TIMELINE_CAP
        elif DEBUG_CHECKS:
            n = 16 + DEBUG_REGIONS * DEBUG_REGION_LEN
        else:
            n = 4
        t = torch.zeros(n, dtype=torch.int32, device=f"cuda:{dev}")
        if DEBUG_CHECKS and not TIMELINE:
            t[9], t[10] = 1, DEBUG_REGION_LEN
        _status[dev] = t
    return t


def read_status(device=None, clear: bool = True) -> tuple[int, int, int, int]:
    """Synchronising read of the status word (call at an existing sync point)."""
    t = status_tensor(device)
    vals = tuple(int(v) for v in t[:4].cpu().tolist())
    if clear and vals[0] != 0:
        t[:4].zero_()
    return vals  # type: ignore[return-value]


def check_status(device=None) -> None:
    code, kid, d0, d1 = read_status(device)
    if code != 0:
        raise DeviceStatusError(code, kid, d0, d1)
