"""Prompt assembly of the text-to-music family: caption clean-up, lyric normalisation, and the paired conditional /
unconditional token layout (src/music3.rs:14-228 of the reference).

Captions arrive as light markdown with ``<|key value|>`` tags; lyrics as lines with ``[Section]`` tags. The cleaned
caption and the normalised lyrics are framed by the family's marker tokens; the unconditional twin of a prompt keeps its
first token and its last two and replaces everything between by the padding token."""
from __future__ import annotations

import re
from typing import Callable, Sequence

UNCONDITIONAL_FILL = 151654
MAX_PROMPT_TOKENS = 5000


def _rewrite_tags(text: str) -> str:
    """``<|bpm 92|>`` -> ``bpm is 92`` (further words follow after a space); a tag of one word keeps the word."""
    def repl(m: re.Match) -> str:
        words = m.group(1).split()
        if len(words) >= 2:
            return " ".join([words[0], "is", words[1]] + words[2:])
        return m.group(1).strip()
    return re.sub(r"<\|(.*?)\|>", repl, text, flags=re.S)


_HEADING = re.compile(r"^[ \t]{0,3}#{1,6}(?=\s)\s*")
_BULLET = re.compile(r"^\s*[*+-]\s+")
_BOLD = re.compile(r"\*\*(.+?)\*\*", re.S)
_ITALIC = re.compile(r"(?<!\*)\*(?!\*)(.+?)(?<!\*)\*(?!\*)")


def clean_caption(caption: str) -> str:
    lines = []
    for line in _rewrite_tags(caption).splitlines():
        line = _HEADING.sub("", line, count=1)
        for _ in range(2):
            line = _BULLET.sub("", line, count=1)
        line = _BOLD.sub(r"\1", line)
        line = _ITALIC.sub(r"\1", line)
        lines.append(line.rstrip())
    kept = [ln for ln in lines if len(ln.strip()) < 3 or any(c not in "-*_ \t" for c in ln.strip())]   # drops rules like "----"
    text = "\n".join(kept).replace("• ", "").replace("    ", "")
    while "\n\n" in text:
        text = text.replace("\n\n", "\n")
    return text


_LEADING_TAGS = re.compile(r"^[ \t]*((?:\[[^\]]+\][ \t]*)+)")


def normalize_lyrics(lyrics: str) -> str:
    """A line that opens with section tags keeps only the tags; tags go on lines of their own in lower case; `` ^ ``
    breaks a line; the text opens with ``[start]``."""
    lines = []
    for line in lyrics.split("\n"):
        m = _LEADING_TAGS.match(line)
        lines.append(m.group(1).strip() if m else line)
    text = "\n".join(lines).replace("] ", "]\n").replace(" [", "\n[").replace(" ^ ", "\n")
    text = re.sub(r"\[([^\[\]]+)\]", lambda m: "[" + m.group(1).lower() + "]", text)
    return "[start]\n" + text


def assemble_prompt(prompt: str, lyrics: str) -> str:
    if not prompt.strip():
        raise ValueError("empty music prompt")
    if not lyrics.strip():
        raise ValueError("empty music lyrics")
    return ("<|im_start|><|caption_start|>" + clean_caption(prompt) + "<|caption_end|><|lyrics_start|>" + normalize_lyrics(lyrics)
            + "<|lyrics_end|><|im_end|><|audio_start|>")


def paired_prompt_ids(prompt: str, lyrics: str, encode: Callable[[str], Sequence[int]]) -> list[int]:
    """Conditional ids followed by their unconditional twin (same length: first token and last two kept, the rest
    replaced by the padding id), the layout the generator's guidance reads as two rows."""
    cond = [int(t) for t in encode(assemble_prompt(prompt, lyrics))]
    if len(cond) < 3:
        raise ValueError("music prompt encodes to fewer than three tokens")
    if len(cond) > MAX_PROMPT_TOKENS:
        raise ValueError(f"music prompt has {len(cond)} tokens")
    uncond = [cond[0]] + [UNCONDITIONAL_FILL] * (len(cond) - 3) + cond[-2:]
    return cond + uncond


def interleave_stereo(pcm: Sequence[float]) -> list[float]:
    """Planar stereo [left..., right...] -> interleaved [l0, r0, l1, r1, ...]."""
    if len(pcm) % 2:
        raise ValueError("planar stereo needs an even number of samples")
    half = len(pcm) // 2
    out = [0.0] * len(pcm)
    out[0::2], out[1::2] = list(pcm[:half]), list(pcm[half:])
    return out
