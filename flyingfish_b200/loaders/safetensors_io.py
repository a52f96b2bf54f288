"""Memory-mapped safetensors reader with a strict header audit, and a small writer.

Checkpoints are read in place and never converted (the reference's rule, README.md:8). The
reader maps the file, parses the JSON header itself and refuses anything irregular before a
single tensor byte is touched: data offsets must tile the data section exactly (no holes, no
overlaps, in order), sizes must match dtype x shape, names must be unique, a sharded index must not
point outside the model directory (symlink escape). Mirrors src/checkpoint.rs:115-177, 207-284.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from pathlib import Path

import torch

DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1), "F8_E4M3": (torch.float8_e4m3fn, 1),
    "F8_E5M2": (torch.float8_e5m2, 1),
}
_REV = {v[0]: k for k, v in DTYPES.items()}
MAX_HEADER = 100 * 1024 * 1024


class CheckpointError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    dtype: str
    shape: tuple[int, ...]
    begin: int
    end: int
    file: "SafetensorsFile"

    @property
    def nbytes(self) -> int:
        return self.end - self.begin


class SafetensorsFile:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise CheckpointError(f"{self.path.name}: file too short for a safetensors header")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > MAX_HEADER or 8 + hlen > size:
            raise CheckpointError(f"{self.path.name}: header length {hlen} is out of range")
        try:
            header = json.loads(self._mm[8: 8 + hlen].decode("utf-8"), object_pairs_hook=self._no_dups)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise CheckpointError(f"{self.path.name}: header is not valid JSON ({e})")
        self.metadata = header.pop("__metadata__", {}) or {}
        self.data_start = 8 + hlen
        data_len = size - self.data_start
        self.tensors: dict[str, TensorInfo] = {}
        spans = []
        for name, ent in header.items():
            if not isinstance(ent, dict) or set(ent) != {"dtype", "shape", "data_offsets"}:
                raise CheckpointError(f"{self.path.name}: malformed entry for {name!r}")
            dt = ent["dtype"]
            if dt not in DTYPES:
                raise CheckpointError(f"{self.path.name}: unsupported dtype {dt!r} for {name!r}")
            shape = tuple(int(s) for s in ent["shape"])
            if any(s < 0 for s in shape):
                raise CheckpointError(f"{self.path.name}: negative dimension in {name!r}")
            b, e = (int(x) for x in ent["data_offsets"])
            n = 1
            for s in shape:
                n *= s
            if e - b != n * DTYPES[dt][1]:
                raise CheckpointError(f"{self.path.name}: {name!r} has {e - b} bytes, dtype x shape needs {n * DTYPES[dt][1]}")
            spans.append((b, e, name))
            self.tensors[name] = TensorInfo(name, dt, shape, b, e, self)
        spans.sort()
        cursor = 0
        for b, e, name in spans:
            if b < cursor:
                raise CheckpointError(f"{self.path.name}: tensor {name!r} overlaps the previous one")
            if b > cursor:
                raise CheckpointError(f"{self.path.name}: hole of {b - cursor} bytes before {name!r}")
            cursor = e
        if cursor != data_len:
            raise CheckpointError(f"{self.path.name}: data section is {data_len} bytes, tensors cover {cursor}")

    @staticmethod
    def _no_dups(pairs):
        d = {}
        for k, v in pairs:
            if k in d:
                raise CheckpointError(f"duplicate tensor name {k!r} in header")
            d[k] = v
        return d

    def tensor(self, name: str) -> torch.Tensor:
        """Zero-copy CPU view of a tensor (backed by the mapping)."""
        info = self.tensors[name]
        dt = DTYPES[info.dtype][0]
        buf = memoryview(self._mm)[self.data_start + info.begin: self.data_start + info.end]
        if info.nbytes == 0:
            return torch.empty(info.shape, dtype=dt)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # read-only mapping: views are never written
            raw = torch.frombuffer(buf, dtype=torch.uint8)
        t = raw.view(dt) if dt != torch.bool else raw.to(torch.bool)
        return t.view(info.shape)

    def byte_range(self, name: str) -> tuple[int, int]:
        """Absolute file offsets of a tensor's bytes (for direct-IO readers)."""
        info = self.tensors[name]
        return self.data_start + info.begin, self.data_start + info.end

    def close(self) -> None:
        """Release the mapping. Tensor views handed out earlier keep it alive until they are
        garbage-collected, in which case only the file descriptor is closed here."""
        try:
            self._mm.close()
        except BufferError:
            pass
        finally:
            self._f.close()


class MappedCheckpoint:
    """A model directory: single ``model.safetensors`` or a sharded ``model.safetensors.index.json``."""

    def __init__(self, model_dir: str | Path):
        self.dir = Path(model_dir).resolve()
        self.files: dict[str, SafetensorsFile] = {}
        self.where: dict[str, SafetensorsFile] = {}
        index = self.dir / "model.safetensors.index.json"
        if index.exists():
            idx = json.loads(index.read_text())
            wm = idx.get("weight_map")
            if not isinstance(wm, dict) or not wm:
                raise CheckpointError("index has no weight_map")
            for name, fname in wm.items():
                f = self._open(fname)
                if name not in f.tensors:
                    raise CheckpointError(f"index maps {name!r} to {fname}, which does not contain it")
                self.where[name] = f
            listed = set(wm)
            for f in self.files.values():
                extra = set(f.tensors) - listed
                if extra:
                    raise CheckpointError(f"{f.path.name} holds tensors missing from the index: {sorted(extra)[:3]}")
        else:
            single = self.dir / "model.safetensors"
            if not single.exists():
                raise CheckpointError(f"no model.safetensors(.index.json) in {self.dir}")
            f = self._open("model.safetensors")
            for name in f.tensors:
                self.where[name] = f

    def _open(self, fname: str) -> SafetensorsFile:
        if fname in self.files:
            return self.files[fname]
        p = (self.dir / fname).resolve()
        if self.dir not in p.parents:
            raise CheckpointError(f"shard {fname!r} resolves outside the model directory")
        f = SafetensorsFile(p)
        self.files[fname] = f
        return f

    def names(self) -> list[str]:
        return sorted(self.where)

    def info(self, name: str) -> TensorInfo:
        return self.where[name].tensors[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)

    def has(self, name: str) -> bool:
        return name in self.where

    def close(self) -> None:
        for f in self.files.values():
            f.close()


def save_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write tensors in name order with a contiguous data section (refuses to overwrite)."""
    path = Path(path)
    if path.exists():
        raise FileExistsError(path)
    header: dict = {}
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _REV:
            raise CheckpointError(f"cannot store dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.dtype != torch.bool else t.to(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": _REV[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
