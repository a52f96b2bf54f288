"""Tokenizer loading and the streaming detokeniser.

``load_tokenizer`` reads ``tokenizer.json`` with the Hugging Face ``tokenizers`` library
(the reference binds the same Rust crate, src/tokenizer.rs:11-24). ``ByteTokenizer`` is a
dependency-free byte-level tokenizer used by tests and by random-init benchmark models that have no
vocabulary file.

``Detok`` turns a growing list of token ids into text deltas. A multi-byte UTF-8 character can be
split over several byte-fallback tokens, so text ending in an incomplete sequence (it decodes to
U+FFFD) is held back until the following tokens complete it (src/serve/detok.rs:93-205).
"""
from __future__ import annotations

import json
from pathlib import Path


class ByteTokenizer:
    """ids 0..255 are bytes; 256 = BOS, 257 = EOS. Any vocabulary size >= 258 works."""
    bos_token_id, eos_token_id = 256, 257
    bos_token = "<s>"

    def __init__(self, vocab_size: int = 258):
        self.vocab_size = max(vocab_size, 258)

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids: list[int], skip_special_tokens: bool = True) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")


class HFTokenizer:
    def __init__(self, path: Path):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(str(path / "tokenizer.json"))
        self.vocab_size = self.tk.get_vocab_size()
        cfg = {}
        p = path / "tokenizer_config.json"
        if p.exists():
            cfg = json.loads(p.read_text())
        def tok(name):
            v = cfg.get(name)
            if isinstance(v, dict):
                v = v.get("content")
            return v
        self.bos_token = tok("bos_token") or ""
        self.eos_token = tok("eos_token")
        self.bos_token_id = self.tk.token_to_id(self.bos_token) if self.bos_token else None
        self.eos_token_id = self.tk.token_to_id(self.eos_token) if self.eos_token else None
        self.chat_template = cfg.get("chat_template")

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        return self.tk.encode(text, add_special_tokens=add_special_tokens).ids

    def decode(self, ids: list[int], skip_special_tokens: bool = True) -> str:
        return self.tk.decode(ids, skip_special_tokens=skip_special_tokens)


def load_tokenizer(model_dir: str | Path):
    p = Path(model_dir)
    if (p / "tokenizer.json").exists():
        return HFTokenizer(p)
    return None


def read_chat_template(model_dir: str | Path) -> str | None:
    """``chat_template.jinja`` in the model directory, else the template embedded in
    ``tokenizer_config.json``."""
    p = Path(model_dir)
    f = p / "chat_template.jinja"
    if f.exists():
        return f.read_text()
    c = p / "tokenizer_config.json"
    if c.exists():
        return json.loads(c.read_text()).get("chat_template")
    return None


class Detok:
    """Incremental detokeniser with hold-back of incomplete UTF-8."""

    def __init__(self, tokenizer, window: int = 8):
        self.tk = tokenizer
        self.ids: list[int] = []
        self.prefix_off = 0          # start of the decoding window
        self.read_off = 0            # ids before this index are already emitted as text
        self.window = window

    def push(self, new_ids: list[int]) -> str:
        """Append tokens and return the newly printable text (possibly empty)."""
        self.ids.extend(new_ids)
        prefix = self.tk.decode(self.ids[self.prefix_off: self.read_off])
        full = self.tk.decode(self.ids[self.prefix_off:])
        if full.endswith("�"):
            return ""                # incomplete character: wait for more tokens
        delta = full[len(prefix):]
        self.prefix_off = max(self.read_off - self.window, self.prefix_off) if self.read_off > self.window else self.prefix_off
        self.read_off = len(self.ids)
        self.prefix_off = max(self.prefix_off, self.read_off - self.window)
        return delta

    def flush(self) -> str:
        """Emit whatever is still held back (replacement characters included)."""
        prefix = self.tk.decode(self.ids[self.prefix_off: self.read_off])
        full = self.tk.decode(self.ids[self.prefix_off:])
        self.read_off = len(self.ids)
        return full[len(prefix):]
