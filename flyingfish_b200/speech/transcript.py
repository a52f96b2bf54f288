"""Transcription results: text with word and sentence time stamps, built from a token / duration trajectory.

Rules (src/parakeet.rs:590-704 of the reference): a token's cue spans ``[frame, frame + duration) * frame_seconds``;
a lone punctuation piece that does not open a word takes the end time of the previous cue as both its start and end;
a cue opens a new word when it is marked as a boundary by the vocabulary (the piece starts with the word marker) or
starts with white space and is not punctuation; sentences close on ``.``, ``?`` or ``!``."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Callable, Sequence

PUNCTUATION = ("?", "'", "¡", "¿", "-", ":", ",", "%", "/", ".", "!")
WORD_MARKER = "▁"


@dataclass
class TextSegment:
    start: float
    end: float
    text: str


@dataclass
class Transcription:
    text: str
    segments: list[TextSegment] = field(default_factory=list)
    words: list[TextSegment] = field(default_factory=list)

    @classmethod
    def whole_clip(cls, text: str, seconds: float) -> "Transcription":
        if not (seconds >= 0.0):
            raise ValueError("clip length must be a non-negative number of seconds")
        return cls(text=text, segments=[TextSegment(0.0, seconds, text)] if text else [], words=[])

    def to_json(self) -> str:
        return json.dumps(asdict(self), ensure_ascii=False)

    def to_srt(self) -> str:
        out = []
        for i, s in enumerate(self.segments, 1):
            out.append(f"{i}\n{_stamp(s.start, ',')} --> {_stamp(s.end, ',')}\n{s.text}\n")
        return "\n".join(out)

    def to_vtt(self) -> str:
        out = ["WEBVTT\n"]
        for s in self.segments:
            out.append(f"{_stamp(s.start, '.')} --> {_stamp(s.end, '.')}\n{s.text}\n")
        return "\n".join(out)


def _stamp(seconds: float, sep: str) -> str:
    ms = int(round(seconds * 1000.0))
    h, ms = divmod(ms, 3600000)
    m, ms = divmod(ms, 60000)
    s, ms = divmod(ms, 1000)
    return f"{h:02d}:{m:02d}:{s:02d}{sep}{ms:03d}"


def word_segments(cues: Sequence[tuple[bool, TextSegment]]) -> tuple[list[TextSegment], list[TextSegment]]:
    """(marked, cue) pairs -> (words, sentence segments)."""
    words: list[TextSegment] = []
    pending = False
    for marked, cue in cues:
        text = cue.text.strip()
        boundary = cue.text[:1].isspace() or cue.text.startswith(WORD_MARKER)
        if not text:
            pending = pending or marked or boundary
            continue
        marked = marked or pending
        boundary = boundary or pending
        pending = False
        punctuation = text in PUNCTUATION
        if not words or marked or (not punctuation and boundary):
            words.append(TextSegment(cue.start, cue.end, text))
        else:
            words[-1].end = cue.end
            words[-1].text += text
    segments: list[TextSegment] = []
    current: TextSegment | None = None
    for word in words:
        if current is None:
            current = TextSegment(word.start, word.end, word.text)
        else:
            current.end = word.end
            current.text += " " + word.text
        if current.text.endswith((".", "?", "!")):
            segments.append(current)
            current = None
    if current is not None:
        segments.append(current)
    return words, segments


def tdt_cues(tokens: Sequence[int], durations: Sequence[int], blank: int, decode: Callable[[Sequence[int]], str],
             boundary: Callable[[int], bool], frame_seconds: float = 0.08, pad_token: int = 2) -> Transcription:
    """Token / duration trajectory of a transducer decode -> text, words and sentences with time stamps."""
    if len(tokens) != len(durations):
        raise ValueError("token and duration trajectories differ in length")
    full_text = decode(list(tokens))
    cues: list[tuple[bool, TextSegment]] = []
    frame = 0
    for token, duration in zip(tokens, durations):
        if token == blank or token == pad_token:
            frame += duration
            continue
        chunk = decode([token])
        if not chunk:
            frame += duration
            continue
        start, end = frame * frame_seconds, (frame + duration) * frame_seconds
        opens = boundary(token)
        if chunk in PUNCTUATION and not opens and cues:
            prev_end = cues[-1][1].end
            cues.append((opens, TextSegment(prev_end, prev_end, chunk)))
        else:
            cues.append((opens, TextSegment(start, end, chunk)))
        frame += duration
    words, segments = word_segments(cues)
    return Transcription(text=full_text, segments=segments, words=words)


def speaker_segments(logits, speakers: int, attention_mask=None, threshold: float = 0.5, frame_seconds: float = 0.08) -> list[TextSegment]:
    """Frame-level speaker activity logits ``[frames, speakers]`` (row-major sequence or tensor) -> one segment per run
    of frames whose sigmoid exceeds ``threshold`` (masked frames are inactive), labelled ``speaker_<n>``, times rounded to
    hundredths (ties to even), sorted by start then speaker (src/diarization.rs:54-112 of the reference)."""
    import math
    flat = [float(v) for v in (logits.reshape(-1).tolist() if hasattr(logits, "reshape") else logits)]
    if speakers <= 0:
        raise ValueError("speaker count must be positive")
    if not flat or len(flat) % speakers:
        raise ValueError("diarization logits extent")
    if not all(math.isfinite(v) for v in flat):
        raise ValueError("non-finite logit")
    if not (math.isfinite(threshold) and 0.0 <= threshold <= 1.0):
        raise ValueError("invalid diarization threshold")
    if not (math.isfinite(frame_seconds) and frame_seconds > 0.0):
        raise ValueError("invalid frame duration")
    frames = len(flat) // speakers
    mask = None if attention_mask is None else [bool(m) for m in attention_mask]
    if mask is not None and len(mask) != frames:
        raise ValueError("diarization mask extent")

    def stamp(frame: int) -> float:
        return round(frame * frame_seconds * 100.0) / 100.0          # Python rounds ties to even

    found = []
    for spk in range(speakers):
        start = None
        for idx in range(frames + 1):
            active = idx < frames and (mask is None or mask[idx]) and 1.0 / (1.0 + math.exp(-flat[idx * speakers + spk])) > threshold
            if start is None and active:
                start = idx
            elif start is not None and not active:
                found.append((stamp(start), spk, stamp(idx)))
                start = None
    found.sort(key=lambda t: (t[0], t[1]))
    return [TextSegment(a, b, f"speaker_{spk}") for a, spk, b in found]


def to_rttm(file_id: str, segments: Sequence[TextSegment]) -> str:
    """Speaker segments as RTTM lines (``SPEAKER <file> 1 <start> <duration> <NA> <NA> <label> <NA> <NA>``)."""
    if not file_id or any(c.isspace() for c in file_id):
        raise ValueError("RTTM file id must be one token")
    out = []
    for seg in segments:
        if not (seg.start >= 0.0 and seg.end >= seg.start):
            raise ValueError("segment times are not ordered")
        if not seg.text or any(c.isspace() for c in seg.text):
            raise ValueError("RTTM speaker label must be one token")
        out.append(f"SPEAKER {file_id} 1 {seg.start:.3f} {seg.end - seg.start:.3f} <NA> <NA> {seg.text} <NA> <NA>\n")
    return "".join(out)
