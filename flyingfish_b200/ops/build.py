"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``_ff_kernels.so`` -- every CUDA kernel and its ``extern "C"`` launcher, compiled by nvcc for
  ``sm_100a`` only (``-gencode arch=compute_100a,code=sm_100a``). The sources have no PyTorch
  dependency, so a file compiles in seconds and nvcc can cross-compile on a machine without a GPU.
* ``_ff_host.so`` -- host-side native runtime (CPU expert FFN with AVX-512, direct-IO expert
  reader), compiled by g++.

The Python side binds the launchers with :mod:`ctypes` (see ``flyingfish_b200.ops.lib``).
A content hash of the sources is stored beside each library so an up-to-date library is
loaded without invoking the compiler. This plays the role of the reference's ``build.rs``
(per-architecture cubin compile, build.rs:147-194, 685-694) for a single target architecture.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
NATIVE = HERE.parent / "native"
BUILD = HERE / "_build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-pthread", "-fvisibility=hidden"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def _hash(files: list[Path], extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for f in sorted(files):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def kernel_sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def host_sources() -> list[Path]:
    return sorted(NATIVE.glob("*.cpp"))


def _up_to_date(lib: Path, stamp: str) -> bool:
    s = lib.with_suffix(".stamp")
    return lib.exists() and s.exists() and s.read_text().strip() == stamp


SHORT_WAIT_NS = 5_000_000      # bound of every device-side wait in the short-wait build: 5 ms instead of 2 s


def build_kernels(verbose: bool = False, force: bool = False, ptxas_info: bool = False, timeline: bool = False,
                  short_wait: bool = False, debug_checks: bool = False) -> Path:
    """Compile all ``csrc/*.cu`` into ``_ff_kernels.so`` (no-op when up to date).

    ``timeline=True`` builds the tracing variant ``_ff_kernels_tl.so`` (``-DFF_TIMELINE``): kernels
    record (time, SM, phase) stamps into the enlarged status buffer, see ``utils/timeline.py``.
    ``short_wait=True`` builds ``_ff_kernels_sw.so`` with every bounded device wait cut to 5 ms: the
    tests of the time-out paths load it, so that a wait nobody answers runs out at once.
    ``debug_checks=True`` builds ``_ff_kernels_dbg.so`` (``-DFF_DEBUG_CHECKS``): scratch with a single-writer
    contract claims its elements in a ledger and a second claim inside one launch raises a status error; extra
    in-kernel bounds words are compiled in."""
    tag = "tl" if timeline else "sw" if short_wait else "dbg" if debug_checks else ""
    lib = HERE / (f"_ff_kernels_{tag}.so" if tag else "_ff_kernels.so")
    srcs = kernel_sources()
    deps = srcs + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    base_flags = list(NVCC_FLAGS) + (["-DFF_TIMELINE"] if timeline else []) + \
        ([f"-DFF_WAIT_NS={SHORT_WAIT_NS}ull"] if short_wait else []) + (["-DFF_DEBUG_CHECKS"] if debug_checks else [])
    stamp = _hash(deps, " ".join(base_flags))
    if not force and _up_to_date(lib, stamp):
        return lib
    build_dir = BUILD / tag if tag else BUILD
    build_dir.mkdir(parents=True, exist_ok=True)
    flags = base_flags + (["-Xptxas", "-v"] if ptxas_info else [])

    def compile_one(src: Path) -> Path:
        obj = build_dir / (src.stem + ".o")
        ostamp = obj.with_suffix(".stamp")
        key = _hash([src] + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")), " ".join(flags))
        if not force and obj.exists() and ostamp.exists() and ostamp.read_text() == key:
            return obj
        cmd = [_nvcc(), *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0 or ptxas_info:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}")
        ostamp.write_text(key)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(compile_one, srcs))
    cmd = [_nvcc(), "-shared", "-o", str(lib), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
           "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link of _ff_kernels.so failed")
    lib.with_suffix(".stamp").write_text(stamp)
    return lib


def build_host(verbose: bool = False, force: bool = False) -> Path | None:
    """Compile ``native/*.cpp`` into ``_ff_host.so``."""
    srcs = host_sources()
    if not srcs:
        return None
    lib = HERE / "_ff_host.so"
    deps = srcs + sorted(NATIVE.glob("*.h"))
    stamp = _hash(deps, " ".join(CXX_FLAGS))
    if not force and _up_to_date(lib, stamp):
        return lib
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, *CXX_FLAGS, "-shared", "-o", str(lib), *map(str, srcs), "-I", str(NATIVE)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("g++ failed for native host library")
    lib.with_suffix(".stamp").write_text(stamp)
    return lib


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_kernels(verbose=verbose, force=force)
    build_kernels(verbose=verbose, force=force, short_wait=True)
    build_kernels(verbose=verbose, force=force, debug_checks=True)
    build_host(verbose=verbose, force=force)


if __name__ == "__main__":
    build_kernels(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    build_host(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built", HERE / "_ff_kernels.so")
