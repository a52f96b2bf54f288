"""Bindings of the native host runtime (``native/cpu_expert_ffn.cpp``): the SIMD expert FFN, the
persistent worker pool that services GPU misses, and the direct-IO reader pool of the NVMe tier."""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p

import torch

from ..ops import lib as oplib

ARMS = {0: "scalar", 1: "avx2+fma", 2: "avx512"}


def _lib():
    lib = oplib.host()
    lib.ff_pool_create.restype = c_void_p
    lib.ff_reader_create.restype = c_void_p
    return lib


def cpu_arm() -> str:
    return ARMS[_lib().ff_cpu_arm()]


def _p(t: torch.Tensor) -> c_void_p:
    return c_void_p(t.data_ptr())


def cpu_expert_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, mode: int = 0, arm: int = -1
                   ) -> torch.Tensor:
    """One SwiGLU expert on the host: BF16 [rows, h] -> BF16 [rows, h]. ``arm`` forces a SIMD arm
    (0 scalar, 1 AVX2, 2 AVX-512) for cross-checks; -1 picks the best one the CPU has."""
    assert x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16
    assert not x.is_cuda and x.stride(1) == 1 and w_gate_up.is_contiguous() and w_down.is_contiguous()
    rows, h = x.shape
    f = w_down.shape[1]
    y = torch.empty(rows, h, dtype=torch.bfloat16)
    rc = _lib().ff_cpu_expert_ffn(_p(x), x.stride(0), _p(w_gate_up), _p(w_down), _p(y), h, rows, h, f, mode, arm)
    if rc != 0:
        raise RuntimeError(f"cpu expert ffn failed ({rc})" + (" : arm not supported by this CPU" if rc == -2 else ""))
    return y


class _Job(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_longlong), ("wgu", c_void_p), ("wd", c_void_p), ("y", c_void_p),
                ("ldy", c_longlong), ("rows", c_int), ("h", c_int), ("f", c_int), ("mode", c_int)]


class ExpertPool:
    """Persistent worker threads; ``run`` executes one job per expert and returns when all are done."""

    def __init__(self, threads: int = 8):
        self.lib = _lib()
        self.handle = c_void_p(self.lib.ff_pool_create(threads))
        self.threads = threads

    def run(self, jobs: list[tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]], mode: int = 0) -> None:
        """jobs: (x [rows,h], w_gate_up [2f,h], w_down [h,f], y [rows,h] output) per expert."""
        if not jobs:
            return
        arr = (_Job * len(jobs))()
        for i, (x, wgu, wd, y) in enumerate(jobs):
            arr[i] = _Job(x.data_ptr(), x.stride(0), wgu.data_ptr(), wd.data_ptr(), y.data_ptr(), y.stride(0), x.shape[0],
                          x.shape[1], wd.shape[1], mode)
        rc = self.lib.ff_pool_run(self.handle, arr, len(jobs))
        if rc != 0:
            raise RuntimeError("expert pool failed")

    def close(self) -> None:
        if self.handle:
            self.lib.ff_pool_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DirectReader:
    """Reader threads doing aligned O_DIRECT ``pread``s into caller buffers (pinned ring slots)."""

    def __init__(self, threads: int = 4):
        self.lib = _lib()
        self.handle = c_void_p(self.lib.ff_reader_create(threads))
        self.fds: dict[str, int] = {}

    def open(self, path: str, direct: bool = True) -> int:
        if path not in self.fds:
            fd = self.lib.ff_dio_open(path.encode(), int(direct))
            if fd < 0:
                raise OSError(-fd, f"cannot open {path}")
            self.fds[path] = fd
        return self.fds[path]

    def submit(self, fd: int, offset: int, length: int, dst: torch.Tensor) -> int:
        assert dst.is_contiguous() and dst.numel() * dst.element_size() >= length
        t = self.lib.ff_reader_submit(self.handle, fd, c_longlong(offset), c_longlong(length), _p(dst))
        if t < 0:
            raise OSError(-t, "reader submit failed")
        return t

    def wait(self, ticket: int, timeout_ms: int = 10000) -> None:
        rc = self.lib.ff_reader_wait(self.handle, ticket, timeout_ms)
        if rc == 0:
            raise TimeoutError("direct-IO read did not complete in time")
        if rc < 0:
            raise OSError(-rc, "direct-IO read failed")

    def in_flight(self) -> int:
        return self.lib.ff_reader_in_flight(self.handle)

    def close(self) -> None:
        if self.handle:
            self.lib.ff_reader_destroy(self.handle)
            self.handle = None
        for fd in self.fds.values():
            self.lib.ff_dio_close(fd)
        self.fds.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
