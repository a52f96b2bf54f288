"""Prefix cache: save / restore the committed KV blocks of a token prefix as a hashed package.

A ``PrefixSnapshot`` is a directory with a manifest (identity + geometry + token ids) and one
safetensors file holding, per layer, the K and V rows of the prefix. The identity hash covers the
model name, the tokenizer fingerprint, the RoPE context (theta, head dim, scaling) and the KV
format tag, so a snapshot can only be restored into an engine that would have produced the same
cache (the reference's src/prefix_state.rs:39-130, 247-330, 609-1025; engine side
src/backend/cuda/engine.rs:3543-4007). Restoring allocates blocks, copies the rows in and commits
the length, after which generation continues as if the prefix had just been prefilled.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from pathlib import Path

import torch

from ..loaders.safetensors_io import SafetensorsFile, save_safetensors

FORMAT = "flyingfish-prefix-1"


class PrefixError(RuntimeError):
    pass


@dataclass(frozen=True)
class PrefixIdentity:
    model: str
    tokenizer: str
    rope: str
    kv_format: str

    def digest(self) -> str:
        return hashlib.sha256("|".join((self.model, self.tokenizer, self.rope, self.kv_format)).encode()).hexdigest()


def identity_for(model) -> PrefixIdentity:
    spec = model.spec
    tk = model.tokenizer
    tk_id = f"{type(tk).__name__}:{getattr(tk, 'vocab_size', spec.vocab)}"
    rope = hashlib.sha256(json.dumps([spec.rope_theta, spec.head_dim, spec.extra.get("rope_scaling")],
                                     sort_keys=True).encode()).hexdigest()[:16]
    return PrefixIdentity(model.name, tk_id, rope, model.settings.kv_format)


def token_hash(ids: list[int]) -> str:
    return hashlib.sha256(",".join(map(str, ids)).encode()).hexdigest()


def save_prefix(model, seq, directory: str | Path) -> Path:
    """Write the committed prefix of ``seq`` (its first ``kv length`` tokens)."""
    eng = model.engine
    kvs = eng.kv.seqs[seq.seq_id]
    n = kvs.length
    if n == 0:
        raise PrefixError("sequence has no committed tokens")
    d = Path(directory)
    if d.exists():
        raise PrefixError(f"refusing to overwrite {d}")
    d.mkdir(parents=True)
    bs = eng.kv.block_size
    blocks = torch.tensor(kvs.blocks[: (n + bs - 1) // bs], device=eng.device)
    tensors = {}
    for l in range(eng.kv.layers):
        for tag, cache in (("k", eng.kv.k[l]), ("v", eng.kv.v[l])):
            if cache is None:
                continue
            rows = cache[blocks].permute(1, 0, 2, 3).reshape(cache.shape[1], -1, cache.shape[3])[:, :n]
            tensors[f"layer.{l}.{tag}"] = rows.contiguous().cpu()
    save_safetensors(d / "kv.safetensors", tensors)
    tokens = seq.all_tokens[:n]
    ident = identity_for(model)
    manifest = {"format": FORMAT, "identity": ident.__dict__, "identity_digest": ident.digest(), "tokens": tokens,
                "token_hash": token_hash(tokens), "length": n, "layers": eng.kv.layers, "kv_heads": eng.kv.kv_heads,
                "head_dim": eng.kv.head_dim}
    (d / "manifest.json").write_text(json.dumps(manifest))
    return d


def restore_prefix(model, directory: str | Path, limit: int | None = None):
    """Create a sequence whose cache holds the snapshot's prefix (its first ``limit`` tokens when given). Returns the
    sequence; its ``prefilled`` equals the restored length, so a longer prompt continues from there."""
    d = Path(directory)
    try:
        man = json.loads((d / "manifest.json").read_text())
    except (OSError, json.JSONDecodeError) as e:
        raise PrefixError(f"unreadable prefix manifest: {e}")
    if man.get("format") != FORMAT:
        raise PrefixError("unknown prefix package format")
    ident = identity_for(model)
    if man.get("identity_digest") != ident.digest():
        raise PrefixError("prefix package was written for a different model / tokenizer / rope / KV format")
    if token_hash(man["tokens"]) != man.get("token_hash") or len(man["tokens"]) != man["length"]:
        raise PrefixError("prefix package token list is corrupt")
    eng = model.engine
    if (man["layers"], man["kv_heads"], man["head_dim"]) != (eng.kv.layers, eng.kv.kv_heads, eng.kv.head_dim):
        raise PrefixError("prefix package geometry differs from the engine's cache")
    n = man["length"] if limit is None else min(man["length"], limit)
    if n <= 0:
        raise PrefixError("nothing to restore")
    seq = eng.add_sequence(list(man["tokens"][:n]) + [0])   # placeholder next token; caller replaces the prompt
    seq.prompt = list(man["tokens"][:n])
    eng.kv.reserve(seq.seq_id, n)
    kvs = eng.kv.seqs[seq.seq_id]
    bs = eng.kv.block_size
    f = SafetensorsFile(d / "kv.safetensors")
    try:
        pos = torch.arange(n)
        blk = torch.tensor([kvs.blocks[p // bs] for p in range(n)], device=eng.device)
        off = (pos % bs).to(eng.device)
        for l in range(eng.kv.layers):
            for tag, cache in (("k", eng.kv.k[l]), ("v", eng.kv.v[l])):
                if cache is None:
                    continue
                rows = f.tensor(f"layer.{l}.{tag}")[:, :n].to(eng.device)   # [heads, n, dim]
                cache[blk, :, off, :] = rows.permute(1, 0, 2).to(cache.dtype)
    finally:
        f.close()
    eng.kv.commit(seq.seq_id, n)
    seq.prefilled = n
    return seq


class PrefixStore:
    """Directory of prefix packages with an index, behind ``--prefix-cache true``: before a prompt is prefilled the
    longest stored prefix of it is restored (only the rest is computed), afterwards the prompt's own cache is stored
    (the reference wires its prefix state the same way around prefill, src/backend/cuda/engine.rs:3543-4007)."""

    def __init__(self, root: str | Path):
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)
        self.hits = 0
        self.stored = 0

    def _index(self) -> list[dict]:
        p = self.root / "index.json"
        try:
            return json.loads(p.read_text())
        except (OSError, json.JSONDecodeError):
            return []

    def lookup(self, model, ids: list[int]) -> tuple[Path, int] | None:
        """Longest stored package whose tokens are a prefix of ``ids`` (at most ``len(ids) - 1`` tokens are used: the
        last prompt token is always computed, it produces the first output)."""
        digest = identity_for(model).digest()
        best = None
        for ent in self._index():
            n = min(ent["length"], len(ids) - 1)
            if ent["identity"] != digest or n <= 0:
                continue
            if ent["length"] <= len(ids) and token_hash(ids[: ent["length"]]) == ent["token_hash"]:
                if best is None or n > best[1]:
                    best = (self.root / ent["dir"], n)
        return best

    def restore(self, model, ids: list[int]):
        """A sequence for ``ids`` whose first tokens come from the store, or None on a miss. The caller prefills it."""
        hit = self.lookup(model, ids)
        if hit is None:
            return None
        seq = restore_prefix(model, hit[0], limit=hit[1])
        seq.prompt = list(ids)
        self.hits += 1
        return seq

    def store(self, model, seq) -> Path | None:
        """Store the committed prompt of ``seq`` unless an identical package exists."""
        n = min(model.engine.kv.seqs[seq.seq_id].length, len(seq.prompt))
        tokens = seq.prompt[:n]
        th = token_hash(tokens)
        index = self._index()
        digest = identity_for(model).digest()
        if n == 0 or any(e["token_hash"] == th and e["identity"] == digest for e in index):
            return None
        name = f"{th[:16]}-{n}"
        d = save_prefix(model, seq, self.root / name)
        index.append({"dir": name, "length": n, "token_hash": th, "identity": digest})
        (self.root / "index.json").write_text(json.dumps(index))
        self.stored += 1
        return d
