"""Engram: n-gram hash tables (DeepSeek-style memory rows addressed by hashes of the last tokens).

* ``EngramHashSetup``: per layer, one odd multiplier per n-gram position and one prime table size per (n-gram
  size, head); tokens are first mapped to a compressed vocabulary.
* ``NgramHistory.prepare``: for every new position and layer, the row ids of all (n-gram size >= 2, head) tables:
  ``rolling = tok[0] * m[0]``, then for each further token ``rolling ^= tok[i] * m[i]`` and
  ``row = offset(size, head) + rolling % prime(size, head)``; an n-gram that reaches before the start of the
  sequence or over a non-text token is padded from that token on.
* ``RowService``: rows live in a file (row = 256 one-byte codes + 8 one-byte power-of-two scales, one per 32 codes);
  a least-frequently-used cache keeps hot rows in memory, misses are read through the direct-IO reader of the
  native host library when present, else ``os.pread``.
Mirrors src/engram.rs:13-36 (row geometry, setup record) and :497-612 (history and hashing) of the reference; its
native row service (:640-1009) is the model for ``RowService``.
"""
from __future__ import annotations

import hashlib
import os
from dataclasses import dataclass, field

import numpy as np

HEAD_DIM, SCALES = 256, 8
ROW_BYTES = HEAD_DIM + SCALES
DEAD_TOKEN = -1


def _is_prime(n: int) -> bool:
    if n < 2:
        return False
    if n % 2 == 0:
        return n == 2
    i = 3
    while i * i <= n:
        if n % i == 0:
            return False
        i += 2
    return True


def _next_prime(n: int, taken: set[int]) -> int:
    while not _is_prime(n) or n in taken:
        n += 1
    return n


@dataclass
class EngramHashSetup:
    layer_ids: list[int]
    tokenizer_vocab: int
    compressed_vocab: int
    pad_id: int
    token_map: list[int]                       # tokenizer id -> compressed id
    multipliers: list[list[int]]               # [layer][ngram position]
    primes: list[list[list[int]]]              # [layer][ngram size - 2][head]
    schema: int = 1

    @classmethod
    def build(cls, layer_ids: list[int], tokenizer_vocab: int, compressed_vocab: int, ngram: int, heads: int,
              table_rows: int, seed: int = 0) -> "EngramHashSetup":
        """Deterministic setup: the token map folds the tokenizer vocabulary onto the compressed one, multipliers are
        odd and bounded so that products never overflow 63 bits, table sizes are distinct primes >= ``table_rows``."""
        rng = np.random.default_rng(seed)
        token_map = [int(t % (compressed_vocab - 1)) + 1 for t in range(tokenizer_vocab)]       # 0 is the pad id
        bound = max(((1 << 63) - 1) // compressed_vocab // 2, 1)
        mult = [[int(rng.integers(1, bound) | 1) for _ in range(ngram)] for _ in layer_ids]
        taken: set[int] = set()
        primes = []
        for _ in layer_ids:
            sizes = []
            for _ in range(ngram - 1):
                row = []
                for _ in range(heads):
                    p = _next_prime(table_rows, taken)
                    taken.add(p)
                    row.append(p)
                sizes.append(row)
            primes.append(sizes)
        s = cls(list(layer_ids), tokenizer_vocab, compressed_vocab, 0, token_map, mult, primes)
        s.validate()
        return s

    def validate(self) -> None:
        layers = len(self.primes)
        if not (layers == len(self.layer_ids) == len(self.multipliers) and layers > 0):
            raise ValueError("engram setup: layer extents differ")
        if not (self.tokenizer_vocab > self.compressed_vocab > 1 and self.pad_id < self.compressed_vocab):
            raise ValueError("engram tokenizer/compressed vocab or pad id is invalid")
        if len(self.token_map) != self.tokenizer_vocab or any(not 0 <= t < self.compressed_vocab for t in self.token_map):
            raise ValueError("engram token map is invalid")
        seen: set[int] = set()
        for layer in self.primes:
            for sizes in layer:
                for p in sizes:
                    if not _is_prime(p) or p in seen:
                        raise ValueError("engram table sizes must be distinct primes")
                    seen.add(p)
        limit = ((1 << 63) - 1) // self.compressed_vocab
        if any(not 0 < m <= limit for layer in self.multipliers for m in layer):
            raise ValueError("engram multiplier would overflow")

    @property
    def ngram(self) -> int:
        return len(self.multipliers[0])

    @property
    def heads(self) -> int:
        return len(self.primes[0][0])

    @property
    def hash_width(self) -> int:
        return (self.ngram - 1) * self.heads

    def offsets(self) -> list[list[int]]:
        out = []
        for layer in self.primes:
            offs, total = [], 0
            for sizes in layer:
                for p in sizes:
                    offs.append(total)
                    total += p
            out.append(offs)
        return out

    def table_rows(self, layer: int) -> int:
        return sum(p for sizes in self.primes[layer] for p in sizes)

    def digest(self) -> str:
        h = hashlib.sha256()
        h.update(repr((self.schema, self.layer_ids, self.compressed_vocab, self.pad_id, self.multipliers, self.primes)).encode())
        h.update(np.asarray(self.token_map, dtype=np.uint32).tobytes())
        return h.hexdigest()


class NgramHistory:
    def __init__(self, setup: EngramHashSetup, capacity: int):
        if capacity <= 0:
            raise ValueError("engram history capacity is zero")
        self.setup, self.capacity = setup, capacity
        self.compressed = np.zeros(capacity, dtype=np.int64)
        self.initialized = np.zeros(capacity, dtype=bool)
        self._offsets = setup.offsets()

    def reset(self) -> None:
        self.compressed[:] = 0
        self.initialized[:] = False

    def prepare(self, input_ids: list[int], start_position: int, text_mask: list[bool] | None = None) -> list[list[int]]:
        """-> per layer, ``len(input_ids) * hash_width`` row ids (position-major)."""
        s = self.setup
        if not input_ids:
            raise ValueError("engram request has no tokens")
        if text_mask is not None and len(text_mask) != len(input_ids):
            raise ValueError("engram text mask extent differs")
        end = start_position + len(input_ids)
        if end > self.capacity:
            raise ValueError(f"engram request {start_position}..{end} exceeds capacity {self.capacity}")
        for off, tid in enumerate(input_ids):
            if not 0 <= tid < len(s.token_map):
                raise ValueError(f"engram token id {tid} at position {start_position + off} is outside the token map")
            dead = text_mask is not None and not text_mask[off]
            self.compressed[start_position + off] = DEAD_TOKEN if dead else s.token_map[tid]
            self.initialized[start_position + off] = True
        result: list[list[int]] = [[] for _ in s.primes]
        for pos in range(start_position, end):
            tokens, blocked = [], False
            for shift in range(s.ngram):
                if shift > pos:
                    blocked = True
                else:
                    if not self.initialized[pos - shift]:
                        raise ValueError(f"engram history position {pos - shift} is missing")
                    if self.compressed[pos - shift] == DEAD_TOKEN:
                        blocked = True
                tokens.append(s.pad_id if blocked else int(self.compressed[pos - shift]))
            for layer in range(len(s.primes)):
                rolling = tokens[0] * s.multipliers[layer][0]
                for n in range(1, s.ngram):
                    rolling ^= tokens[n] * s.multipliers[layer][n]
                    for head in range(s.heads):
                        result[layer].append(self._offsets[layer][(n - 1) * s.heads + head] + rolling % s.primes[layer][n - 1][head])
        return result


def decode_rows(rows: np.ndarray) -> np.ndarray:
    """uint8 [n, 264] -> float32 [n, 256]: signed one-byte codes times 2^(scale - 127), one scale per 32 codes."""
    codes = rows[:, :HEAD_DIM].view(np.int8).astype(np.float32).reshape(-1, SCALES, HEAD_DIM // SCALES)
    scale = np.ldexp(1.0, rows[:, HEAD_DIM:].astype(np.int32) - 127).astype(np.float32)
    return (codes * scale[:, :, None]).reshape(-1, HEAD_DIM)


@dataclass
class _Entry:
    data: np.ndarray
    freq: int = 0
    tick: int = 0


class RowService:
    """File-backed table rows with a least-frequently-used cache (ties: least recently used)."""

    def __init__(self, path: str, rows: int, cache_rows: int):
        if os.path.getsize(path) < rows * ROW_BYTES:
            raise ValueError("engram table file is shorter than its row count")
        self.rows, self.cache_rows = rows, max(cache_rows, 1)
        self.fd = os.open(path, os.O_RDONLY)
        self.cache: dict[int, _Entry] = {}
        self.tick = 0
        self.stats = {"hits": 0, "misses": 0, "evictions": 0, "bytes_read": 0}

    def close(self) -> None:
        if self.fd >= 0:
            os.close(self.fd)
            self.fd = -1

    def _read(self, row: int) -> np.ndarray:
        buf = os.pread(self.fd, ROW_BYTES, row * ROW_BYTES)
        if len(buf) != ROW_BYTES:
            raise IOError(f"short read of engram row {row}")
        self.stats["bytes_read"] += ROW_BYTES
        return np.frombuffer(buf, dtype=np.uint8).copy()

    def gather(self, row_ids: list[int]) -> np.ndarray:
        out = np.empty((len(row_ids), ROW_BYTES), dtype=np.uint8)
        for i, r in enumerate(row_ids):
            if not 0 <= r < self.rows:
                raise IndexError(f"engram row {r} outside the table")
            self.tick += 1
            e = self.cache.get(r)
            if e is None:
                self.stats["misses"] += 1
                if len(self.cache) >= self.cache_rows:
                    victim = min(self.cache, key=lambda k: (self.cache[k].freq, self.cache[k].tick))
                    del self.cache[victim]
                    self.stats["evictions"] += 1
                e = _Entry(self._read(r))
                self.cache[r] = e
            else:
                self.stats["hits"] += 1
            e.freq += 1
            e.tick = self.tick
            out[i] = e.data
        return out
