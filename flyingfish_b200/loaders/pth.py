"""Readers for PyTorch ``.pth`` checkpoints and NeMo ``.nemo`` archives without unpickling arbitrary code.

A ``.pth`` file is a ZIP of *stored* (uncompressed) members: ``<root>/data.pkl`` describes the state dict with a
pickle program, ``<root>/data/<key>`` hold the raw storages. ``read_pth`` runs a restricted pickle machine that
understands only the opcodes ``torch.save`` emits and only an allow-list of globals (tensor rebuild helpers,
storage classes, ``OrderedDict``); anything else is refused. Tensors are views over a memory map of the file, so
loading is zero-copy. A ``.nemo`` file is a tar: ``read_nemo`` finds ``model_config.yaml`` and the weights member
(``model_weights.ckpt``, itself a ``.pth``) by offset without extracting.
Plays the role of the reference's stored-ZIP pickle parser and tar member reader (src/checkpoint.rs:207-284,
:311-339)."""
from __future__ import annotations

import io
import mmap
import struct
import tarfile
import zipfile
from dataclasses import dataclass
from pathlib import Path

import torch

_DTYPES = {"FloatStorage": torch.float32, "HalfStorage": torch.float16, "BFloat16Storage": torch.bfloat16,
           "DoubleStorage": torch.float64, "LongStorage": torch.int64, "IntStorage": torch.int32,
           "ShortStorage": torch.int16, "CharStorage": torch.int8, "ByteStorage": torch.uint8, "BoolStorage": torch.bool}


class UnsafePickle(ValueError):
    pass


@dataclass
class _StorageRef:
    dtype: torch.dtype
    key: str
    numel: int


@dataclass
class TensorRecord:
    dtype: torch.dtype
    shape: tuple[int, ...]
    stride: tuple[int, ...]
    storage: _StorageRef
    offset: int                     # elements


class _Global:
    def __init__(self, module: str, name: str):
        self.module, self.name = module, name


_ALLOWED = {("collections", "OrderedDict"), ("torch._utils", "_rebuild_tensor_v2"), ("torch._utils", "_rebuild_parameter"),
            ("torch", "Size")} | {("torch", n) for n in _DTYPES}


def _run_pickle(data: bytes):
    """Restricted pickle machine (protocol 2-4 subset)."""
    stack: list = []
    marks: list[int] = []
    memo: dict[int, object] = {}
    pos = 0

    def pop_mark():
        m = marks.pop()
        items = stack[m:]
        del stack[m:]
        return items

    while True:
        op = data[pos]; pos += 1
        if op == 0x80:                                   # PROTO
            pos += 1
        elif op == 0x95:                                 # FRAME
            pos += 8
        elif op == ord("."):
            return stack.pop()
        elif op == ord("("):
            marks.append(len(stack))
        elif op == ord("}"):
            stack.append({})
        elif op == ord("]"):
            stack.append([])
        elif op == ord(")"):
            stack.append(())
        elif op == ord("N"):
            stack.append(None)
        elif op == 0x88:
            stack.append(True)
        elif op == 0x89:
            stack.append(False)
        elif op in (ord("K"), ord("M"), ord("J")):
            n = {ord("K"): 1, ord("M"): 2, ord("J"): 4}[op]
            v = int.from_bytes(data[pos: pos + n], "little", signed=(op == ord("J"))); pos += n
            stack.append(v)
        elif op == 0x8a:                                 # LONG1
            n = data[pos]; pos += 1
            stack.append(int.from_bytes(data[pos: pos + n], "little", signed=True)); pos += n
        elif op == ord("G"):
            stack.append(struct.unpack(">d", data[pos: pos + 8])[0]); pos += 8
        elif op in (ord("X"), 0x8c, 0x8d):               # BINUNICODE, SHORT_BINUNICODE, BINUNICODE8
            n = {ord("X"): 4, 0x8c: 1, 0x8d: 8}[op]
            ln = int.from_bytes(data[pos: pos + n], "little"); pos += n
            stack.append(data[pos: pos + ln].decode("utf-8")); pos += ln
        elif op == ord("c"):                             # GLOBAL
            e1 = data.index(b"\n", pos); module = data[pos:e1].decode(); e2 = data.index(b"\n", e1 + 1)
            name = data[e1 + 1:e2].decode(); pos = e2 + 1
            if (module, name) not in _ALLOWED:
                raise UnsafePickle(f"global {module}.{name} is not allowed in a checkpoint")
            stack.append(_Global(module, name))
        elif op == 0x93:                                 # STACK_GLOBAL
            name = stack.pop(); module = stack.pop()
            if (module, name) not in _ALLOWED:
                raise UnsafePickle(f"global {module}.{name} is not allowed in a checkpoint")
            stack.append(_Global(module, name))
        elif op in (ord("q"), ord("r"), 0x94):           # BINPUT, LONG_BINPUT, MEMOIZE
            if op == ord("q"):
                memo[data[pos]] = stack[-1]; pos += 1
            elif op == ord("r"):
                memo[int.from_bytes(data[pos: pos + 4], "little")] = stack[-1]; pos += 4
            else:
                memo[len(memo)] = stack[-1]
        elif op in (ord("h"), ord("j")):                 # BINGET, LONG_BINGET
            n = 1 if op == ord("h") else 4
            stack.append(memo[int.from_bytes(data[pos: pos + n], "little")]); pos += n
        elif op == ord("t"):
            stack.append(tuple(pop_mark()))
        elif op == 0x85:
            stack.append((stack.pop(),))
        elif op == 0x86:
            b = stack.pop(); a = stack.pop(); stack.append((a, b))
        elif op == 0x87:
            c = stack.pop(); b = stack.pop(); a = stack.pop(); stack.append((a, b, c))
        elif op == ord("Q"):                             # BINPERSID: ('storage', class, key, location, numel)
            pid = stack.pop()
            if not (isinstance(pid, tuple) and len(pid) >= 5 and pid[0] == "storage" and isinstance(pid[1], _Global)):
                raise UnsafePickle("unexpected persistent id")
            stack.append(_StorageRef(_DTYPES[pid[1].name], str(pid[2]), int(pid[4])))
        elif op == ord("R"):                             # REDUCE
            args = stack.pop(); fn = stack.pop()
            if not isinstance(fn, _Global):
                raise UnsafePickle("call of a non-global")
            if fn.name == "OrderedDict":
                stack.append({})
            elif fn.name == "_rebuild_tensor_v2":
                st, off, shape, stride = args[0], args[1], args[2], args[3]
                stack.append(TensorRecord(st.dtype, tuple(shape), tuple(stride), st, int(off)))
            elif fn.name == "_rebuild_parameter":
                stack.append(args[0])
            elif fn.name == "Size":
                stack.append(tuple(args[0]))
            else:
                raise UnsafePickle(f"call of {fn.module}.{fn.name}")
        elif op == ord("s"):                             # SETITEM
            v = stack.pop(); k = stack.pop(); stack[-1][k] = v
        elif op == ord("u"):                             # SETITEMS
            items = pop_mark()
            for i in range(0, len(items), 2):
                stack[-1][items[i]] = items[i + 1]
        elif op == ord("a"):
            v = stack.pop(); stack[-1].append(v)
        elif op == ord("e"):
            items = pop_mark(); stack[-1].extend(items)
        elif op == ord("b"):                             # BUILD (OrderedDict state etc.): keep the object, drop the state
            stack.pop()
        else:
            raise UnsafePickle(f"pickle opcode 0x{op:02x} is not supported")


def _flatten(obj, prefix: str, out: dict[str, TensorRecord]) -> None:
    if isinstance(obj, TensorRecord):
        out[prefix] = obj
    elif isinstance(obj, dict):
        for k, v in obj.items():
            _flatten(v, f"{prefix}.{k}" if prefix else str(k), out)


class PthFile:
    """Memory-mapped ``.pth``: ``tensors()`` yields zero-copy views."""

    def __init__(self, path: str | Path, base_offset: int = 0, length: int | None = None):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._base = base_offset
        window = self._mm[base_offset: base_offset + length] if length is not None else self._mm
        with zipfile.ZipFile(io.BytesIO(window) if length is not None else self._f) as z:
            infos = {i.filename: i for i in z.infolist()}
            pkl = [n for n in infos if n.endswith("data.pkl")]
            if len(pkl) != 1:
                raise ValueError("not a torch zip checkpoint")
            self.root = pkl[0][: -len("data.pkl")]
            for i in infos.values():
                if i.compress_type != zipfile.ZIP_STORED:
                    raise ValueError(f"member {i.filename} is compressed; storages must be stored")
            obj = _run_pickle(z.read(pkl[0]))
            self._offsets = {}
            for name, i in infos.items():
                # local header: 30 bytes + name + extra
                hdr = window[i.header_offset: i.header_offset + 30]
                nlen, elen = struct.unpack("<HH", hdr[26:30])
                self._offsets[name] = (self._base + i.header_offset + 30 + nlen + elen, i.file_size)
        self.records: dict[str, TensorRecord] = {}
        _flatten(obj, "", self.records)

    def tensor(self, name: str) -> torch.Tensor:
        r = self.records[name]
        off, size = self._offsets[f"{self.root}data/{r.storage.key}"]
        item = torch.empty(0, dtype=r.dtype).element_size()
        if r.storage.numel * item > size:
            raise ValueError(f"storage {r.storage.key} is shorter than the pickle says")
        t = torch.frombuffer(self._mm, dtype=r.dtype if r.dtype != torch.bool else torch.uint8, count=r.storage.numel,
                             offset=off)
        if r.dtype == torch.bool:
            t = t.view(torch.bool)
        return torch.as_strided(t, r.shape, r.stride, r.offset)

    def tensors(self) -> dict[str, torch.Tensor]:
        return {n: self.tensor(n) for n in self.records}

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()


def read_pth(path: str | Path) -> PthFile:
    return PthFile(path)


def read_nemo(path: str | Path) -> tuple[str, PthFile]:
    """-> (text of ``model_config.yaml``, weights reader). The tar must store members uncompressed."""
    path = Path(path)
    cfg, weights = None, None
    with tarfile.open(path, "r:") as tar:
        for m in tar:
            base = m.name.rsplit("/", 1)[-1]
            if ".." in m.name.split("/") or m.name.startswith("/"):
                raise ValueError(f"tar member {m.name} escapes the archive")
            if base == "model_config.yaml" and m.isfile():
                cfg = tar.extractfile(m).read().decode("utf-8")
            elif base == "model_weights.ckpt" and m.isfile():
                weights = (m.offset_data, m.size)
    if cfg is None or weights is None:
        raise ValueError("not a .nemo archive (model_config.yaml / model_weights.ckpt missing)")
    return cfg, PthFile(path, weights[0], weights[1])


def read_nemo_member(path: str | Path, suffix: str) -> bytes:
    """Bytes of the one archive member whose name ends in ``suffix`` (tokenizer vocabularies carry a hash prefix)."""
    hits = []
    with tarfile.open(Path(path), "r:") as tar:
        for m in tar:
            if ".." in m.name.split("/") or m.name.startswith("/"):
                raise ValueError(f"tar member {m.name} escapes the archive")
            if m.isfile() and m.name.endswith(suffix):
                hits.append(tar.extractfile(m).read())
    if len(hits) != 1:
        raise ValueError(f"{len(hits)} archive members end in {suffix!r}; one is expected")
    return hits[0]
