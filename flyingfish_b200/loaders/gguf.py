"""GGUF container reader (header, metadata, tensor index over a memory map) and Q4_0 blocks.

Only what the engine consumes: GGUF v2/v3 little-endian, metadata value types 0-12, tensor types
F32 / F16 / BF16 / Q4_0. A Q4_0 block is 18 bytes: one FP16 scale ``d`` and 32 4-bit codes, element
``i`` of the first half in the low nibble of byte ``i`` and element ``i+16`` in its high nibble,
value ``(code - 8) * d`` (the reference reads the same subset, src/gguf.rs:18-131, 235-470, and
dequantises with kernels/q4_0_linear.cu).
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import torch

GGUF_MAGIC = b"GGUF"
T_F32, T_F16, T_Q4_0, T_BF16 = 0, 1, 2, 30
_TYPE_BLOCK = {T_F32: (1, 4), T_F16: (1, 2), T_Q4_0: (32, 18), T_BF16: (1, 2)}
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


class GgufError(ValueError):
    pass


@dataclass
class GgufTensor:
    name: str
    shape: tuple[int, ...]      # outermost first (GGUF stores innermost first)
    ggml_type: int
    offset: int                 # absolute file offset
    nbytes: int


class GgufFile:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._pos = 0
        if self._read(4) != GGUF_MAGIC:
            raise GgufError("not a GGUF file")
        (self.version,) = self._unpack("<I")
        if self.version not in (2, 3):
            raise GgufError(f"unsupported GGUF version {self.version}")
        n_tensors, n_kv = self._unpack("<QQ")
        if n_tensors > 1 << 20 or n_kv > 1 << 20:
            raise GgufError("implausible tensor / metadata count")
        self.metadata: dict[str, object] = {}
        for _ in range(n_kv):
            key = self._string()
            (vt,) = self._unpack("<I")
            self.metadata[key] = self._value(vt)
        infos = []
        for _ in range(n_tensors):
            name = self._string()
            (nd,) = self._unpack("<I")
            if nd > 4:
                raise GgufError(f"{name}: {nd} dimensions")
            dims = self._unpack("<" + "Q" * nd)
            gt, off = self._unpack("<IQ")
            infos.append((name, tuple(reversed(dims)), gt, off))
        align = int(self.metadata.get("general.alignment", 32))
        data_start = (self._pos + align - 1) // align * align
        self.tensors: dict[str, GgufTensor] = {}
        size = len(self._mm)
        for name, shape, gt, off in infos:
            if gt not in _TYPE_BLOCK:
                raise GgufError(f"{name}: unsupported tensor type {gt}")
            n = 1
            for s in shape:
                n *= s
            be, bb = _TYPE_BLOCK[gt]
            if shape and shape[-1] % be:
                raise GgufError(f"{name}: innermost dimension {shape[-1]} is not a multiple of the block size {be}")
            nbytes = n // be * bb
            if off % align or data_start + off + nbytes > size:
                raise GgufError(f"{name}: data range outside the file or misaligned")
            if name in self.tensors:
                raise GgufError(f"duplicate tensor {name}")
            self.tensors[name] = GgufTensor(name, shape, gt, data_start + off, nbytes)

    # -- low level -----------------------------------------------------------------------------
    def _read(self, n: int) -> bytes:
        if self._pos + n > len(self._mm):
            raise GgufError("unexpected end of file")
        b = self._mm[self._pos: self._pos + n]
        self._pos += n
        return b

    def _unpack(self, fmt: str):
        return struct.unpack(fmt, self._read(struct.calcsize(fmt)))

    def _string(self) -> str:
        (n,) = self._unpack("<Q")
        if n > 1 << 24:
            raise GgufError("implausible string length")
        return self._read(n).decode("utf-8")

    def _value(self, vt: int):
        if vt in _SCALAR:
            return self._unpack(_SCALAR[vt])[0]
        if vt == 8:
            return self._string()
        if vt == 9:
            (et,) = self._unpack("<I")
            (n,) = self._unpack("<Q")
            if n > 1 << 26:
                raise GgufError("implausible array length")
            return [self._value(et) for _ in range(n)]
        raise GgufError(f"unknown metadata value type {vt}")

    # -- tensors ---------------------------------------------------------------------------------
    def raw(self, name: str) -> torch.Tensor:
        t = self.tensors[name]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)
            return torch.frombuffer(memoryview(self._mm)[t.offset: t.offset + t.nbytes], dtype=torch.uint8)

    def tensor(self, name: str, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """Dequantised tensor in ``dtype``."""
        t = self.tensors[name]
        raw = self.raw(name)
        if t.ggml_type == T_F32:
            return raw.view(torch.float32).view(t.shape).to(dtype)
        if t.ggml_type == T_F16:
            return raw.view(torch.float16).view(t.shape).to(dtype)
        if t.ggml_type == T_BF16:
            return raw.view(torch.bfloat16).view(t.shape).to(dtype)
        return q4_0_dequant(raw, t.shape, dtype)

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()


def q4_0_dequant(raw: torch.Tensor, shape: tuple[int, ...], dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    blocks = raw.view(-1, 18)
    d = blocks[:, :2].contiguous().view(torch.float16).to(torch.float32)          # [nb, 1]
    qs = blocks[:, 2:]
    lo = (qs & 0xF).to(torch.float32) - 8.0
    hi = (qs >> 4).to(torch.float32) - 8.0
    vals = torch.cat([lo, hi], dim=1) * d
    return vals.view(shape).to(dtype)


def q4_0_quant(w: torch.Tensor) -> torch.Tensor:
    """Reference Q4_0 quantiser (ggml's rule: d = max-magnitude value / -8)."""
    x = w.to(torch.float32).reshape(-1, 32)
    idx = x.abs().argmax(dim=1, keepdim=True)
    mx = x.gather(1, idx)
    d = mx / -8.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = torch.clamp((x * inv + 8.5).floor(), 0, 15).to(torch.uint8)
    packed = q[:, :16] | (q[:, 16:] << 4)
    dh = d.to(torch.float16).view(torch.uint8).view(-1, 2)
    return torch.cat([dh, packed], dim=1).reshape(-1)


def write_gguf(path: str | Path, metadata: dict[str, object], tensors: dict[str, tuple[torch.Tensor, int]],
               alignment: int = 32) -> None:
    """Minimal GGUF v3 writer (tests and export tools). ``tensors``: name -> (tensor, ggml type)."""
    path = Path(path)
    if path.exists():
        raise FileExistsError(path)

    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    def val(v) -> bytes:
        if isinstance(v, bool):
            return struct.pack("<I?", 7, v)
        if isinstance(v, int):
            return struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<II", 4, v) if v < 1 << 32 else struct.pack("<IQ", 10, v)
        if isinstance(v, float):
            return struct.pack("<If", 6, v)
        if isinstance(v, str):
            return struct.pack("<I", 8) + s(v)
        if isinstance(v, list):
            body = b"".join(val(e)[4:] for e in v)
            et = struct.unpack("<I", val(v[0])[:4])[0] if v else 4
            return struct.pack("<IIQ", 9, et, len(v)) + body
        raise GgufError(f"cannot store metadata value {v!r}")

    md = dict(metadata)
    md.setdefault("general.alignment", alignment)
    head = GGUF_MAGIC + struct.pack("<IQQ", 3, len(tensors), len(md))
    for k, v in md.items():
        head += s(k) + val(v)
    blobs, off = [], 0
    for name, (t, gt) in tensors.items():
        if gt == T_Q4_0:
            raw = q4_0_quant(t).numpy().tobytes()
        elif gt == T_F32:
            raw = t.to(torch.float32).contiguous().numpy().tobytes()
        elif gt == T_F16:
            raw = t.to(torch.float16).contiguous().view(torch.uint8).numpy().tobytes()
        else:
            raw = t.to(torch.bfloat16).contiguous().view(torch.uint8).numpy().tobytes()
        dims = tuple(reversed(t.shape))
        head += s(name) + struct.pack("<I", len(dims)) + struct.pack("<" + "Q" * len(dims), *dims) + struct.pack("<IQ", gt, off)
        pad = (alignment - len(raw) % alignment) % alignment
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    pad = (alignment - len(head) % alignment) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        for b in blobs:
            f.write(b)
