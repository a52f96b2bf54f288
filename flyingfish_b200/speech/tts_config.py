"""Host-side contract of the text-to-speech family: the speaker-prefixed prompt and the sampling settings read from a
checkpoint's ``generation_config.json`` (src/breeze.rs:23-92 of the reference). The language-model stack and the audio
codec of that family are not part of this build; these pieces pin what a `speak` request means."""
from __future__ import annotations

from dataclasses import dataclass

ALLOWED_KEYS = ("bos_token_id", "depth_decoder_do_sample", "depth_decoder_temperature", "do_sample", "eos_token_id", "max_new_tokens",
                "pad_token_id", "repetition_penalty", "temperature", "top_k", "top_p", "transformers_version")
MAX_FRAMES = 750                       # 12.5 codec frames per second: one minute of speech
SAMPLES_PER_FRAME = 1920               # at 24 kHz
SAMPLING_RATE = 24000
CODEBOOKS = 16


def plain_prompt(text: str) -> str:
    """Text as the model reads it: the first speaker's tag in front."""
    return "[S0]" + text


@dataclass(frozen=True)
class SpeakConfig:
    temperature: float
    top_k: int
    top_p: float
    repetition_penalty: float
    max_new_tokens: int

    @property
    def max_seconds(self) -> float:
        return self.max_new_tokens * SAMPLES_PER_FRAME / SAMPLING_RATE


def speak_config(root: dict) -> SpeakConfig:
    """Validates a ``generation_config.json``: sampling on for backbone and depth decoder with one shared temperature,
    the family's special token ids, defaults top-k 50, top-p 1, repetition penalty 1.1, at most 750 frames."""
    if not isinstance(root, dict):
        raise ValueError("generation config must be an object")
    for key in root:
        if key not in ALLOWED_KEYS:
            raise ValueError(f"unknown generation key {key}")
    for key, want in (("do_sample", True), ("depth_decoder_do_sample", True), ("bos_token_id", 2), ("eos_token_id", [1]), ("pad_token_id", 0)):
        if root.get(key) != want:
            raise ValueError(f"generation config: {key} must be {want!r}")
    try:
        temperature, depth = float(root["temperature"]), float(root["depth_decoder_temperature"])
        max_new = int(root["max_new_tokens"])
    except (KeyError, TypeError, ValueError):
        raise ValueError("generation config lacks temperature / depth_decoder_temperature / max_new_tokens") from None
    if temperature != depth:
        raise ValueError("backbone and depth-decoder temperatures differ")
    top_k, top_p, penalty = int(root.get("top_k", 50)), float(root.get("top_p", 1.0)), float(root.get("repetition_penalty", 1.1))
    if not (temperature > 0 and top_k > 0 and 0 < top_p <= 1 and penalty > 0):
        raise ValueError("invalid sampling settings")
    if not (0 < max_new <= MAX_FRAMES):
        raise ValueError(f"generation limit {max_new} outside 1..{MAX_FRAMES}")
    return SpeakConfig(temperature, top_k, top_p, penalty, max_new)
