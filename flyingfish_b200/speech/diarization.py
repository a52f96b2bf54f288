"""Streaming speaker diarization (frame classification over eight speaker slots in arrival order).

The model (published layout ``Nemotron3DiarizationForAudioFrameClassification``; src/diarization.rs and
src/backend/cuda/engine_diarization.rs of the reference): ``factor`` log-mel frames are stacked into one row and
projected, a pre-norm transformer encoder with rotary positions runs bidirectionally over a *window* of rows, a small
head brings the rows back to the spectrogram frame grid (projection, a width-3 convolution whose ``factor * c`` output
channels are read as ``factor`` consecutive frames, two dense layers) and emits one logit per frame and speaker.

Long audio goes through the window in chunks. The window is ``[speaker cache | FIFO | chunk | right context]``: rows that
leave the FIFO enter the speaker cache, and once the cache is over its capacity it is compressed to the rows that score
best per speaker (``select_cache_rows``), which is what keeps a speaker in the same output slot for the whole recording.

B200 mapping: the encoder is the vision tower's recipe -- every projection is the tcgen05 GEMM followed by a fused bias +
activation pass, heads (64 wide in the published model) are widened to the 128 lanes of the tcgen05 prefill attention
kernel, which runs bidirectionally over a scratch page cache with the number of valid keys as the context length; rotary
and the K / V page writes are one kernel. The reference runs the same network in FP32 on cuBLAS with host-side cache
policy; the cache policy stays on the host here too (it looks at a few hundred probabilities once per chunk), the rows it
selects are gathered on the device."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path

import torch
import torch.nn.functional as F

from .. import ops
from ..ops import vision_ops as vo
from .audio import LogMel, LogMelConfig, StreamingLogMel
from .transcript import TextSegment, speaker_segments

BF16 = torch.bfloat16
PAGE = 64
LANES = 128
DEFAULT_THRESHOLD = 0.5
ARCHITECTURE = "Nemotron3DiarizationForAudioFrameClassification"


@dataclass(frozen=True)
class ChunkConfig:
    frames: int          # rows of a chunk whose logits are emitted
    right: int           # look-ahead rows behind the chunk
    fifo: int            # rows the FIFO may hold
    update: int          # rows popped from the FIFO at least, once it overflows


@dataclass(frozen=True)
class SpeakerCacheConfig:
    frames: int = 264
    silence: int = 1
    fifo: int = 264
    update: int = 222
    threshold: float = 0.25
    latest_boost: float = 0.05
    positive_rate: float = 0.5
    strong_rate: float = 0.75
    weak_rate: float = 1.5

    def budget(self, speakers: int) -> int:
        return self.frames // speakers - self.silence

    def counts(self, speakers: int) -> tuple[int, int, int]:
        """(minimum positive scores, strongly boosted rows, weakly boosted rows) per speaker."""
        b = self.budget(speakers)
        return int(math.floor(b * self.positive_rate)), int(math.floor(b * self.strong_rate)), int(math.floor(b * self.weak_rate))


@dataclass
class DiarizationSpec:
    hidden: int = 512
    intermediate: int = 2048
    layers: int = 31
    heads: int = 8
    head_hidden: int = 192
    speakers: int = 8
    factor: int = 8
    max_positions: int = 5000
    rope_theta: float = 10000.0
    eps: float = 1e-5
    mel: LogMelConfig = field(default_factory=lambda: LogMelConfig(normalize=False))
    offline: ChunkConfig = ChunkConfig(340, 40, 40, 300)
    cache: SpeakerCacheConfig = SpeakerCacheConfig()
    modes: dict[str, tuple[int, int]] = field(default_factory=lambda: {"low_latency": (9, 4), "very_low_latency": (6, 2),
                                                                        "ultra_low_latency": (3, 1)})
    default_mode: str = "low_latency"

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def frame_seconds(self) -> float:
        return self.mel.hop_length / self.mel.sampling_rate

    def stream_config(self, mode: str | None = None) -> ChunkConfig:
        name = mode or self.default_mode
        if name not in self.modes:
            raise ValueError(f"unknown streaming mode {name!r} (have {sorted(self.modes)})")
        frames, right = self.modes[name]
        return ChunkConfig(frames, right, self.cache.fifo, self.cache.update)

    def max_encoder_rows(self) -> int:
        rows = self.cache.frames + self.offline.fifo + self.offline.frames + self.offline.right
        for frames, right in self.modes.values():
            rows = max(rows, self.cache.frames + self.cache.fifo + frames + right)
        return rows

    def check(self) -> None:
        if min(self.hidden, self.intermediate, self.layers, self.heads, self.head_hidden, self.speakers, self.factor) <= 0:
            raise ValueError("diarization geometry must be positive")
        if self.hidden % self.heads or self.head_dim % 2 or self.head_dim > LANES:
            raise ValueError("unsupported head geometry")
        if (self.factor * self.mel.mel_bins) % 8 or self.hidden % 8 or self.head_hidden % 8 or self.intermediate % 8:
            raise ValueError("row widths must be multiples of 8")
        if self.cache.frames % self.speakers or self.cache.budget(self.speakers) <= 0:
            raise ValueError("speaker cache length must leave every speaker a positive budget")
        if not (0.0 < self.cache.threshold < 0.5):
            raise ValueError("cache score threshold must lie in (0, 0.5)")
        for cfg in [self.offline] + [self.stream_config(m) for m in self.modes]:
            if min(cfg.frames, cfg.fifo, cfg.update) <= 0 or cfg.right < 0:
                raise ValueError("chunk geometry must be positive")
        if self.max_encoder_rows() > self.max_positions:
            raise ValueError("diarization window exceeds rotary positions")
        self.mel.check()

    # -- published configuration files ---------------------------------------------------------------
    @classmethod
    def from_json(cls, root: dict, processor: dict) -> "DiarizationSpec":
        """``config.json`` and ``processor_config.json`` of a published checkpoint."""
        if root.get("architectures") != [ARCHITECTURE] or root.get("model_type") != "nemotron3_diarization":
            raise ValueError("not a diarization configuration")
        audio, head, cache = root.get("audio_config"), root.get("head_config"), root.get("streaming_config")
        if not all(isinstance(x, dict) for x in (audio, head, cache)):
            raise ValueError("audio_config / head_config / streaming_config missing")
        rope = audio.get("rope_parameters", {})
        if audio.get("hidden_act") != "gelu" or float(audio.get("partial_rotary_factor", 1.0)) != 1.0 or \
                rope.get("rope_type", "default") != "default" or float(rope.get("partial_rotary_factor", 1.0)) != 1.0:
            raise ValueError("unsupported encoder activation or rotary scheme")
        if audio.get("num_key_value_heads", audio["num_attention_heads"]) != audio["num_attention_heads"]:
            raise ValueError("grouped-query encoders are not supported")
        factor = int(audio["subsampling_factor"])
        for part, name in ((head, "head_config"), (cache, "streaming_config"), (processor, "processor_config")):
            if int(part.get("subsampling_factor", factor)) != factor:
                raise ValueError(f"{name}: subsampling factor differs from the encoder's")
        if int(head.get("audio_hidden_size", audio["hidden_size"])) != int(audio["hidden_size"]):
            raise ValueError("head input width differs from the encoder's")
        if int(cache.get("num_speakers", head["num_speakers"])) != int(head["num_speakers"]):
            raise ValueError("speaker counts of head and cache differ")
        feats = processor.get("feature_extractor")
        if not isinstance(feats, dict):
            raise ValueError("feature_extractor missing")
        if feats.get("padding_side", "right") != "right" or float(feats.get("padding_value", 0.0)) != 0.0:
            raise ValueError("unsupported feature padding")
        mel = LogMelConfig(sampling_rate=int(feats["sampling_rate"]), n_fft=int(feats["n_fft"]), win_length=int(feats["win_length"]),
                           hop_length=int(feats["hop_length"]), mel_bins=int(feats["feature_size"]),
                           preemphasis=float(feats["preemphasis"]), normalize=False)
        if mel.mel_bins != int(audio["num_mel_bins"]):
            raise ValueError("feature size and encoder mel bins differ")
        modes = {str(k): (int(v[0]), int(v[1])) for k, v in processor.get("streaming_modes", {}).items()}
        default_mode = str(processor.get("streaming_mode", "low_latency"))
        if default_mode not in modes:
            raise ValueError("default streaming mode is not among streaming_modes")
        spec = cls(hidden=int(audio["hidden_size"]), intermediate=int(audio["intermediate_size"]), layers=int(audio["num_hidden_layers"]),
                   heads=int(audio["num_attention_heads"]), head_hidden=int(head["hidden_size"]), speakers=int(head["num_speakers"]),
                   factor=factor, max_positions=int(audio["max_position_embeddings"]), rope_theta=float(rope.get("rope_theta", 10000.0)),
                   mel=mel,
                   offline=ChunkConfig(int(root["chunk_length"]), int(root["chunk_right_context"]), int(root["fifo_length"]),
                                       int(root["speaker_cache_update_period"])),
                   cache=SpeakerCacheConfig(frames=int(cache["speaker_cache_length"]),
                                            silence=int(cache["speaker_cache_silence_frames_per_speaker"]),
                                            fifo=int(cache["fifo_length"]), update=int(cache["speaker_cache_update_period"]),
                                            threshold=float(cache["prediction_score_threshold"]),
                                            latest_boost=float(cache["latest_frames_score_boost"]),
                                            positive_rate=float(cache["min_positive_scores_rate"]),
                                            strong_rate=float(cache["strong_boost_rate"]), weak_rate=float(cache["weak_boost_rate"])),
                   modes=modes, default_mode=default_mode)
        spec.check()
        return spec

    def to_json(self) -> tuple[dict, dict]:
        m, c = self.mel, self.cache
        root = {"architectures": [ARCHITECTURE], "model_type": "nemotron3_diarization", "dtype": "float32",
                "audio_config": {"attention_dropout": 0.0, "hidden_act": "gelu", "hidden_size": self.hidden,
                                 "intermediate_size": self.intermediate, "max_position_embeddings": self.max_positions,
                                 "model_type": "nemotron3_diarization_audio", "num_attention_heads": self.heads,
                                 "num_hidden_layers": self.layers, "num_key_value_heads": self.heads, "num_mel_bins": m.mel_bins,
                                 "partial_rotary_factor": 1.0,
                                 "rope_parameters": {"partial_rotary_factor": 1.0, "rope_theta": self.rope_theta, "rope_type": "default"},
                                 "subsampling_factor": self.factor},
                "chunk_length": self.offline.frames, "chunk_right_context": self.offline.right, "fifo_length": self.offline.fifo,
                "speaker_cache_update_period": self.offline.update,
                "head_config": {"audio_hidden_size": self.hidden, "hidden_size": self.head_hidden, "model_type": "",
                                "num_speakers": self.speakers, "subsampling_factor": self.factor},
                "streaming_config": {"fifo_length": c.fifo, "latest_frames_score_boost": c.latest_boost,
                                     "min_positive_scores_rate": c.positive_rate, "model_type": "", "num_speakers": self.speakers,
                                     "prediction_score_threshold": c.threshold, "speaker_cache_length": c.frames,
                                     "speaker_cache_silence_frames_per_speaker": c.silence, "speaker_cache_update_period": c.update,
                                     "strong_boost_rate": c.strong_rate, "subsampling_factor": self.factor, "weak_boost_rate": c.weak_rate}}
        processor = {"processor_class": "Nemotron3DiarizationProcessor", "streaming_mode": self.default_mode,
                     "streaming_modes": {k: list(v) for k, v in self.modes.items()}, "subsampling_factor": self.factor,
                     "feature_extractor": {"feature_extractor_type": "NemotronAsrStreamingFeatureExtractor", "feature_size": m.mel_bins,
                                           "hop_length": m.hop_length, "n_fft": m.n_fft, "padding_side": "right", "padding_value": 0.0,
                                           "preemphasis": m.preemphasis, "return_attention_mask": True,
                                           "sampling_rate": m.sampling_rate, "win_length": m.win_length}}
        return root, processor

    def expected_tensors(self) -> dict[str, tuple[str, tuple[int, ...]]]:
        h, i, c, r = self.hidden, self.intermediate, self.head_hidden, self.factor
        out: dict[str, tuple[str, tuple[int, ...]]] = {}
        for layer in range(self.layers):
            p = f"model.audio_tower.layers.{layer}."
            for norm in ("layer_norm1", "layer_norm2"):
                out[p + norm + ".weight"] = ("F32", (h,))
                out[p + norm + ".bias"] = ("F32", (h,))
            for proj in ("q_proj", "k_proj", "v_proj", "o_proj"):
                out[p + f"self_attn.{proj}.weight"] = ("F32", (h, h))
            out[p + "self_attn.o_proj.bias"] = ("F32", (h,))
            out[p + "mlp.fc1.weight"], out[p + "mlp.fc1.bias"] = ("F32", (i, h)), ("F32", (i,))
            out[p + "mlp.fc2.weight"], out[p + "mlp.fc2.bias"] = ("F32", (h, i)), ("F32", (h,))
        out["model.audio_tower.embedder.projection.weight"] = ("F32", (h, r * self.mel.mel_bins))
        for norm in ("input_layer_norm", "layer_norm"):
            out[f"model.audio_tower.{norm}.weight"] = ("F32", (h,))
            out[f"model.audio_tower.{norm}.bias"] = ("F32", (h,))
        out["model.proj.weight"], out["model.proj.bias"] = ("F32", (c, h)), ("F32", (c,))
        out["model.upsampler.conv.weight"], out["model.upsampler.conv.bias"] = ("F32", (r * c, c, 3)), ("F32", (r * c,))
        out["classifier.dense.weight"], out["classifier.dense.bias"] = ("F32", (c, c)), ("F32", (c,))
        out["classifier.out_proj.weight"], out["classifier.out_proj.bias"] = ("F32", (self.speakers, c)), ("F32", (self.speakers,))
        out["silence_embeds"] = ("F32", (h,))
        return out

    def validate(self, tensors: dict[str, torch.Tensor]) -> int:
        want = self.expected_tensors()
        missing = sorted(set(want) - set(tensors))
        extra = sorted(set(tensors) - set(want))
        if missing or extra:
            raise ValueError(f"diarization checkpoint: missing {missing[:3]}, unexpected {extra[:3]}")
        for name, (_, shape) in want.items():
            if tuple(tensors[name].shape) != shape:
                raise ValueError(f"diarization checkpoint: {name} has shape {tuple(tensors[name].shape)}, expected {shape}")
        return len(want)


def diarization_tiny() -> DiarizationSpec:
    """A small geometry with every mechanism of the published one (for tests): 4 speakers, a cache of 16 rows."""
    spec = DiarizationSpec(hidden=64, intermediate=128, layers=2, heads=2, head_hidden=32, speakers=4, factor=4, max_positions=128,
                           mel=LogMelConfig(sampling_rate=16000, n_fft=64, win_length=48, hop_length=32, mel_bins=16, normalize=False),
                           offline=ChunkConfig(12, 3, 6, 8),
                           cache=SpeakerCacheConfig(frames=16, silence=1, fifo=10, update=6, threshold=0.25, latest_boost=0.05),
                           modes={"low_latency": (5, 2), "ultra_low_latency": (2, 1)}, default_mode="low_latency")
    spec.check()
    return spec


def random_tensors(spec: DiarizationSpec, seed: int = 0, std: float = 0.08) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (_, shape) in spec.expected_tensors().items():
        t = torch.randn(*shape, generator=g) * std
        if name.endswith("norm.weight") or "layer_norm1.weight" in name or "layer_norm2.weight" in name:
            t = t + 1.0
        out[name] = t
    return out


# ------------------------------------------------------------------------------------------------
# speaker cache policy (host)
# ------------------------------------------------------------------------------------------------
def _boost_top(scores: torch.Tensor, count: int, boost: float) -> None:
    """Adds ``boost`` to the ``count`` best rows of every speaker column (ties: the earlier row)."""
    if count <= 0:
        return
    frames = scores.shape[0]
    k = min(count, frames)
    order = torch.sort(scores, dim=0, descending=True, stable=True).indices[:k]
    scores.scatter_add_(0, order, torch.full_like(order, boost, dtype=scores.dtype))


def cache_scores(spec: DiarizationSpec, probs: torch.Tensor, boosts: bool = True) -> torch.Tensor:
    """Score of row t for speaker s, [frames, speakers] (src/backend/cuda/engine_diarization.rs:238-300 of the
    reference): ``log max(p_ts, th) - log max(1 - p_ts, th) + sum_s' log max(1 - p_ts', th) - log 0.5`` for rows where s
    speaks (p > 0.5), minus infinity elsewhere: high when s speaks alone. Speakers with enough positive scores drop
    their non-positive rows. With ``boosts``: rows newer than the old cache get a small bonus, the best ``strong`` rows
    of a speaker get 2 log 2 and the best ``weak`` rows log 2 on top, so that every speaker keeps a share of the cache."""
    frames, speakers = probs.shape
    cfg = spec.cache
    positive, strong, weak = cfg.counts(speakers)
    p = probs.detach().float().cpu()
    th = torch.tensor(cfg.threshold, dtype=torch.float32)
    log_one_minus = torch.log(torch.maximum(1.0 - p, th))
    scores = torch.log(torch.maximum(p, th)) - log_one_minus + log_one_minus.sum(dim=1, keepdim=True) - math.log(0.5)
    speech = p > 0.5
    neg_inf = torch.tensor(float("-inf"))
    scores = torch.where(speech, scores, neg_inf)
    enough = (scores > 0.0).sum(dim=0) >= positive
    scores = torch.where(enough[None, :] & speech & (scores <= 0.0), neg_inf, scores)
    if boosts:
        scores[cfg.frames:] += cfg.latest_boost
        _boost_top(scores, strong, 2.0 * math.log(2.0))
        _boost_top(scores, weak, math.log(2.0))
    return scores


def select_cache_rows(spec: DiarizationSpec, probs: torch.Tensor) -> list[int]:
    """Which rows survive a compression of the speaker cache. ``probs`` [frames, speakers] are the pooled speaker
    probabilities of the cache rows followed by the rows just popped from the FIFO (``frames`` > capacity). Returns
    ``capacity`` row indices, grouped by the speaker that claimed them and in time order inside a group; the index
    ``frames`` stands for the silence row (one per speaker always, and one for every slot no row qualified for):
    the ``capacity`` best entries of ``cache_scores`` over all (speaker, row) pairs, each speaker's silence row counting
    as plus infinity (src/backend/cuda/engine_diarization.rs:301-323 of the reference)."""
    frames, speakers = probs.shape
    cfg = spec.cache
    capacity = cfg.frames
    if speakers != spec.speakers or frames <= capacity:
        raise ValueError("diarization compression extent")
    scores = cache_scores(spec, probs)
    scored = frames + cfg.silence
    flat = torch.full((speakers, scored), float("-inf"))
    flat[:, :frames] = scores.t()
    flat[:, frames] = float("inf")
    order = torch.sort(flat.reshape(-1), descending=True, stable=True).indices[:capacity]
    values = flat.reshape(-1)[order]
    sentinel = speakers * scored
    picked = sorted(int(i) if v > float("-inf") else sentinel for i, v in zip(order.tolist(), values.tolist()))
    return [frames if i == sentinel else min(i % scored, frames) for i in picked]


@dataclass
class SpeakerState:
    """Arrival-order speaker memory of one stream: cache rows (embeddings entering the encoder, with the probabilities
    they were selected by) and the FIFO of recent rows."""
    config: ChunkConfig
    cache: torch.Tensor                 # [cache_len, hidden]
    fifo: torch.Tensor                  # [fifo_len, hidden]
    probs: torch.Tensor                 # [cache_len, speakers] FP32 on the host
    compressed: bool = False
    updates: int = 0                    # compressions so far

    @property
    def cached_rows(self) -> int:
        return self.cache.shape[0] + self.fifo.shape[0]


# ------------------------------------------------------------------------------------------------
# the model
# ------------------------------------------------------------------------------------------------
def _widen_rows(w: torch.Tensor, heads: int, d: int) -> torch.Tensor:
    """[heads * d, k] -> [heads * 128, k]: each rotary half of a head (d / 2 rows) opens a 64-row half."""
    if d == LANES:
        return w
    k = w.shape[1]
    out = torch.zeros(heads, 2, LANES // 2, k, dtype=w.dtype)
    out[:, :, : d // 2] = w.reshape(heads, 2, d // 2, k)
    return out.reshape(heads * LANES, k)


def _pad_rows(w: torch.Tensor, multiple: int) -> torch.Tensor:
    n = (w.shape[0] + multiple - 1) // multiple * multiple
    if n == w.shape[0]:
        return w
    return torch.cat([w, torch.zeros(n - w.shape[0], *w.shape[1:], dtype=w.dtype)], 0)


@dataclass
class _Layer:
    ln1_w: torch.Tensor
    ln1_b: torch.Tensor
    wqkv: torch.Tensor                  # [3 * heads * 128, hidden]
    wo: torch.Tensor                    # [hidden, heads * 128]
    bo: torch.Tensor
    ln2_w: torch.Tensor
    ln2_b: torch.Tensor
    w1: torch.Tensor
    b1: torch.Tensor
    w2: torch.Tensor
    b2: torch.Tensor


class DiarizationModel:
    def __init__(self, spec: DiarizationSpec, tensors: dict[str, torch.Tensor], device: torch.device | str = "cpu"):
        spec.check()
        spec.validate(tensors)
        self.spec, self.device = spec, torch.device(device)
        s, h, d = spec, spec.heads, spec.head_dim

        def dev(t: torch.Tensor) -> torch.Tensor:
            return t.to(BF16).contiguous().to(self.device)

        t = {k: v.float() for k, v in tensors.items()}
        self.embed_w = dev(t["model.audio_tower.embedder.projection.weight"])
        self.in_ln = (dev(t["model.audio_tower.input_layer_norm.weight"]), dev(t["model.audio_tower.input_layer_norm.bias"]))
        self.out_ln = (dev(t["model.audio_tower.layer_norm.weight"]), dev(t["model.audio_tower.layer_norm.bias"]))
        self.layers: list[_Layer] = []
        for i in range(s.layers):
            p = f"model.audio_tower.layers.{i}."
            wqkv = torch.cat([_widen_rows(t[p + f"self_attn.{n}.weight"], h, d) for n in ("q_proj", "k_proj", "v_proj")], 0)
            wo = _widen_rows(t[p + "self_attn.o_proj.weight"].t().contiguous(), h, d).t().contiguous()
            self.layers.append(_Layer(dev(t[p + "layer_norm1.weight"]), dev(t[p + "layer_norm1.bias"]), dev(wqkv), dev(wo),
                                      dev(t[p + "self_attn.o_proj.bias"]), dev(t[p + "layer_norm2.weight"]),
                                      dev(t[p + "layer_norm2.bias"]), dev(t[p + "mlp.fc1.weight"]), dev(t[p + "mlp.fc1.bias"]),
                                      dev(t[p + "mlp.fc2.weight"]), dev(t[p + "mlp.fc2.bias"])))
        self.proj = (dev(t["model.proj.weight"]), dev(t["model.proj.bias"]))
        # the width-3 convolution as one GEMM over [previous | this | next] row: weight [r c, c, 3] -> [r c, 3 c], tap major
        conv = t["model.upsampler.conv.weight"]
        self.conv = (dev(conv.permute(0, 2, 1).reshape(conv.shape[0], -1)), dev(t["model.upsampler.conv.bias"]))
        self.dense = (dev(t["classifier.dense.weight"]), dev(t["classifier.dense.bias"]))
        self.out = (dev(_pad_rows(t["classifier.out_proj.weight"], 64)), dev(_pad_rows(t["classifier.out_proj.bias"], 64)))
        self.silence = dev(t["silence_embeds"])[None, :]
        self.scale = d ** -0.5
        # rotary table of the window positions ("rotate half" pairs), values rounded like the activations
        inv = 1.0 / torch.pow(torch.tensor(s.rope_theta, dtype=torch.float32), torch.arange(d // 2, dtype=torch.float32) * 2 / d)
        ang = torch.arange(s.max_encoder_rows(), dtype=torch.float32)[:, None] * inv[None, :]
        self.rope = torch.stack([torch.cos(ang).to(BF16).float(), torch.sin(ang).to(BF16).float()], dim=-1).contiguous().to(self.device)
        self.mel = LogMel(spec.mel, self.device)
        self.encoder_calls = 0

    @classmethod
    def random(cls, spec: DiarizationSpec, device="cpu", seed: int = 0) -> "DiarizationModel":
        return cls(spec, random_tensors(spec, seed), device)

    # -- pieces --------------------------------------------------------------------------------------
    def embed(self, features: torch.Tensor) -> torch.Tensor:
        """Log-mel frames [frames, mel] -> rows [ceil(frames / factor), hidden] (the last stack is zero padded)."""
        s = self.spec
        frames = features.shape[0]
        rows = (frames + s.factor - 1) // s.factor
        x = features.to(self.device, torch.float32)
        if rows * s.factor != frames:
            x = F.pad(x, (0, 0, 0, rows * s.factor - frames))
        return ops.linear(x.reshape(rows, s.factor * s.mel.mel_bins).to(BF16), self.embed_w)

    def encode(self, embeds: torch.Tensor, valid: int) -> torch.Tensor:
        """Window rows [rows, hidden] -> encoder output; keys beyond ``valid`` rows are masked for every query."""
        s, dev, h = self.spec, self.device, self.spec.heads
        rows = embeds.shape[0]
        if not (0 < valid <= rows <= s.max_encoder_rows()):
            raise ValueError(f"diarization window of {rows} rows ({valid} valid) outside 1..{s.max_encoder_rows()}")
        self.encoder_calls += 1
        blocks = (rows + PAGE - 1) // PAGE
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        slots = torch.arange(rows, dtype=torch.int32, device=dev)
        bt = torch.arange(blocks, dtype=torch.int32, device=dev)[None, :].contiguous()
        q_start, q_lens, ctx = i32([0]), i32([rows]), i32([valid])
        kc = torch.zeros(blocks, h, PAGE, LANES, dtype=BF16, device=dev)
        vc = torch.zeros_like(kc)
        table = self.rope[:rows].contiguous()
        x = vo.layernorm(embeds, *self.in_ln, s.eps)
        for ly in self.layers:
            n1 = vo.layernorm(x, ly.ln1_w, ly.ln1_b, s.eps)
            qkv = ops.linear(n1, ly.wqkv)
            vo.rope_table_apply_(qkv, table, h, LANES, rot_dim=s.head_dim, slots=slots, kcache=kc, vcache=vc, kv_heads=h)
            a = ops.attn_prefill(qkv, kc, vc, bt, q_start, q_lens, ctx, rows, h, h, LANES, self.scale, window=-1)
            x = x + vo.linear_bias_act(a, ly.wo, ly.bo)
            n2 = vo.layernorm(x, ly.ln2_w, ly.ln2_b, s.eps)
            f = vo.linear_bias_act(n2, ly.w1, ly.b1, "gelu")
            x = x + vo.linear_bias_act(f, ly.w2, ly.b2)
        return vo.layernorm(x, *self.out_ln, s.eps)

    def classify(self, encoded: torch.Tensor) -> torch.Tensor:
        """Encoder rows [rows, hidden] -> logits [rows * factor, speakers] FP32 at the spectrogram frame grid."""
        s = self.spec
        rows, c = encoded.shape[0], s.head_hidden
        p = vo.linear_bias_act(encoded, *self.proj)
        zero = torch.zeros(1, c, dtype=p.dtype, device=p.device)
        cols = torch.cat([torch.cat([zero, p[:-1]], 0), p, torch.cat([p[1:], zero], 0)], dim=1).contiguous()
        sub = vo.linear_bias_act(cols, *self.conv, "relu").reshape(rows * s.factor, c)
        dense = vo.linear_bias_act(sub, *self.dense, "relu")
        return vo.linear_bias_act(dense, *self.out)[:, : s.speakers].float()

    def pool(self, logits: torch.Tensor, mask: list[bool]) -> torch.Tensor:
        """Frame logits -> per-row speaker probabilities [rows, speakers] on the host (the mean sigmoid of a row's
        ``factor`` frames; rows outside ``mask`` are zero)."""
        s = self.spec
        probs = torch.sigmoid(logits.float()).reshape(-1, s.factor, s.speakers).mean(dim=1).cpu()
        probs[~torch.tensor(mask, dtype=torch.bool)] = 0.0
        return probs

    def frame_logits(self, features: torch.Tensor, valid_frames: int | None = None) -> torch.Tensor:
        """One window without speaker memory: frames [n, mel] -> logits [ceil(n / factor) * factor, speakers]."""
        frames = features.shape[0]
        valid = frames if valid_frames is None else valid_frames
        if not (0 < valid <= frames):
            raise ValueError("invalid diarization valid frames")
        emb = self.embed(features)
        return self.classify(self.encode(emb, (valid + self.spec.factor - 1) // self.spec.factor))

    # -- speaker memory ------------------------------------------------------------------------------
    def new_state(self, config: ChunkConfig) -> SpeakerState:
        z = torch.zeros(0, self.spec.hidden, dtype=BF16, device=self.device)
        return SpeakerState(config, z, z.clone(), torch.zeros(0, self.spec.speakers))

    def update_state(self, state: SpeakerState, embeds: torch.Tensor, probs: torch.Tensor, chunk: int) -> bool:
        """Files the chunk's rows: ``embeds`` / ``probs`` are the window ``[cache | FIFO | chunk (| right)]`` as it went
        through the encoder and the pooled probabilities it produced. Returns True when the cache was compressed.
        (src/backend/cuda/engine_diarization.rs:875-1043 of the reference.)"""
        cfg, cap = state.config, self.spec.cache.frames
        cache_len, fifo_len = state.cache.shape[0], state.fifo.shape[0]
        fifo_rows = fifo_len + chunk
        fifo_end = cache_len + fifo_rows
        if not (fifo_end <= embeds.shape[0] == probs.shape[0]):
            raise ValueError("diarization state window")
        if fifo_rows <= cfg.fifo:
            state.fifo = embeds[cache_len:fifo_end].clone()
            return False
        popped = min(max(cfg.update, fifo_rows - cfg.fifo), fifo_rows)
        old = state.probs if state.compressed else probs[:cache_len]
        cache_probs = torch.cat([old, probs[cache_len:cache_len + popped]], 0)
        cache_rows = cache_len + popped
        did = False
        if cache_rows > cap:
            pick = select_cache_rows(self.spec, cache_probs)
            index = torch.tensor(pick, dtype=torch.long)
            source = torch.cat([embeds[:cache_rows], self.silence], 0)
            state.cache = source.index_select(0, index.to(source.device))
            state.probs = torch.cat([cache_probs, torch.zeros(1, cache_probs.shape[1])], 0).index_select(0, index)
            state.compressed = True
            state.updates += 1
            did = True
        else:
            state.cache = embeds[:cache_rows].clone()
            state.probs = cache_probs.clone()
        state.fifo = embeds[cache_len + popped:fifo_end].clone()
        return did

    def step(self, state: SpeakerState, new_rows: torch.Tensor, row_mask: list[bool], chunk: int) -> torch.Tensor:
        """Runs the window ``[cache | FIFO | new_rows]`` (``new_rows`` = the chunk followed by its look-ahead rows),
        updates the speaker memory with the first ``chunk`` new rows and returns their frame logits
        ``[chunk * factor, speakers]``."""
        s = self.spec
        cached = state.cached_rows
        window = torch.cat([state.cache, state.fifo, new_rows], 0)
        mask = [True] * cached + list(row_mask)
        if len(mask) != window.shape[0] or not (0 < chunk <= new_rows.shape[0]):
            raise ValueError("diarization step extents")
        hole = mask.index(False) if False in mask else len(mask)
        if any(mask[hole:]):
            raise ValueError(f"diarization mask is not a padding prefix: first hole at row {hole}")
        if hole == 0:
            raise ValueError("diarization step without a valid row")
        logits = self.classify(self.encode(window, hole))
        self.update_state(state, window, self.pool(logits, mask), chunk)
        return logits[cached * s.factor:(cached + chunk) * s.factor]

    # -- whole recordings ----------------------------------------------------------------------------
    def offline(self, features: torch.Tensor, valid_frames: int | None = None) -> torch.Tensor:
        """All frames of a recording -> logits [frames, speakers], through the offline chunking."""
        s, cfg = self.spec, self.spec.offline
        frames = features.shape[0]
        valid = frames if valid_frames is None else valid_frames
        rows_all = self.embed(features)
        n = rows_all.shape[0]
        state = self.new_state(cfg)
        out, start = [], 0
        while start < n:
            chunk = min(cfg.frames, n - start)
            right = min(cfg.right, n - start - chunk)
            mask = [(start + r) * s.factor < valid for r in range(chunk + right)]
            out.append(self.step(state, rows_all[start:start + chunk + right], mask, chunk))
            start += chunk
        self.last_state = state
        return torch.cat(out, 0)[:frames]

    def stream(self, mode: str | None = None) -> "DiarizationStream":
        return DiarizationStream(self, self.spec.stream_config(mode))

    def clip_logits(self, waveform: torch.Tensor, stream: bool = False, mode: str | None = None,
                    block_samples: int | None = None) -> torch.Tensor:
        """A mono waveform at the model's sampling rate -> frame logits [frames, speakers]: through the offline chunking,
        or chunk by chunk with look-ahead as live audio would arrive (``stream``; samples go in blocks of one second)."""
        s = self.spec
        if stream:
            st = self.stream(mode)
            block = block_samples or s.mel.sampling_rate
            pieces = []
            for off in range(0, waveform.numel(), block):
                pieces.append(st.push(waveform[off:off + block], last=off + block >= waveform.numel()))
            return torch.cat(pieces, 0)
        feat, lens = self.mel.extract([waveform], normalize=False)
        return self.offline(feat[0, : int(lens[0])])

    def diarize(self, waveform: torch.Tensor, stream: bool = False, threshold: float = DEFAULT_THRESHOLD,
                mode: str | None = None, block_samples: int | None = None) -> list[TextSegment]:
        """A mono waveform at the model's sampling rate -> speaker segments ``speaker_<slot>``."""
        logits = self.clip_logits(waveform, stream, mode, block_samples)
        if logits.shape[0] == 0:
            return []
        return speaker_segments(logits.cpu(), self.spec.speakers, [True] * logits.shape[0], threshold, self.spec.frame_seconds)


def speaker_masks(model: DiarizationModel, waveform: torch.Tensor, stream: bool = False, threshold: float = DEFAULT_THRESHOLD,
                  mode: str | None = None) -> tuple[torch.Tensor, float]:
    """Binarised speaker activity at the encoder's row grid, pooled as the speaker cache pools it: the mean sigmoid over
    each ``factor`` consecutive frames against the threshold (a trailing partial group is dropped). Returns
    ``([rows, speakers] bool, seconds per row)`` (src/diarization.rs ``speaker_masks`` of the reference)."""
    s = model.spec
    logits = model.clip_logits(waveform, stream, mode).float().cpu()
    rows = logits.shape[0] // s.factor
    pooled = torch.sigmoid(logits[: rows * s.factor].double()).reshape(rows, s.factor, s.speakers).mean(dim=1)
    return pooled > threshold, s.frame_seconds * s.factor


class DiarizationStream:
    """Incremental diarization of a growing waveform: log-mel frames are produced as samples arrive; whenever a chunk
    and its look-ahead are there, one window runs and the chunk's logits come out (the look-ahead rows are computed
    again with the next chunk). ``push(..., last=True)`` flushes the remaining frames without look-ahead."""

    def __init__(self, model: DiarizationModel, config: ChunkConfig):
        self.model, self.config = model, config
        self.state = model.new_state(config)
        self.mel = StreamingLogMel(model.mel)
        self.frames = torch.zeros(0, model.spec.mel.mel_bins, dtype=torch.float32, device=model.device)
        self.finished = False
        self.steps = 0

    def push(self, samples: torch.Tensor, last: bool = False) -> torch.Tensor:
        if self.finished:
            raise RuntimeError("the stream is finished")
        s, cfg = self.model.spec, self.config
        self.frames = torch.cat([self.frames, self.mel.push(samples, last)], 0)
        self.finished = last
        out = []
        need = (cfg.frames + cfg.right) * s.factor
        step = cfg.frames * s.factor
        while self.frames.shape[0] >= need:
            rows = self.model.embed(self.frames[:need])
            out.append(self.model.step(self.state, rows, [True] * rows.shape[0], cfg.frames))
            self.frames = self.frames[step:]
            self.steps += 1
        if last:
            while self.frames.shape[0] > 0:
                take = min(self.frames.shape[0], step)
                n_rows = (take + s.factor - 1) // s.factor
                rest = self.frames[: min(self.frames.shape[0], need)]
                rows = self.model.embed(rest)
                logits = self.model.step(self.state, rows, [True] * rows.shape[0], n_rows)
                out.append(logits[:take])
                self.frames = self.frames[take:]
                self.steps += 1
        if not out:
            return torch.zeros(0, s.speakers, dtype=torch.float32, device=self.model.device)
        return torch.cat(out, 0)


# ------------------------------------------------------------------------------------------------
# plain FP32 restatement (the numerics oracle of the tests) and loading
# ------------------------------------------------------------------------------------------------
def reference_logits(spec: DiarizationSpec, tensors: dict[str, torch.Tensor], embeds: torch.Tensor, valid: int) -> torch.Tensor:
    """Window rows [rows, hidden] FP32 -> logits [rows * factor, speakers], in plain PyTorch on the checkpoint tensors."""
    t = {k: v.float() for k, v in tensors.items()}
    h, d, rows = spec.heads, spec.head_dim, embeds.shape[0]
    ln = lambda x, p: F.layer_norm(x, (spec.hidden,), t[p + ".weight"], t[p + ".bias"], spec.eps)
    inv = 1.0 / torch.pow(torch.tensor(spec.rope_theta), torch.arange(d // 2, dtype=torch.float32) * 2 / d)
    ang = torch.arange(rows, dtype=torch.float32)[:, None] * inv[None, :]
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rot(x):
        x1, x2 = x[..., : d // 2], x[..., d // 2:]
        return torch.cat([x1 * cs - x2 * sn, x2 * cs + x1 * sn], -1)
    x = ln(embeds.float(), "model.audio_tower.input_layer_norm")
    for i in range(spec.layers):
        p = f"model.audio_tower.layers.{i}."
        n1 = ln(x, p + "layer_norm1")
        q, k, v = (F.linear(n1, t[p + f"self_attn.{n}.weight"]).reshape(rows, h, d) for n in ("q_proj", "k_proj", "v_proj"))
        att = torch.einsum("qhd,khd->hqk", rot(q), rot(k)) * d ** -0.5
        att[:, :, valid:] = float("-inf")
        a = torch.einsum("hqk,khd->qhd", torch.softmax(att, -1), v).reshape(rows, spec.hidden)
        x = x + F.linear(a, t[p + "self_attn.o_proj.weight"], t[p + "self_attn.o_proj.bias"])
        n2 = ln(x, p + "layer_norm2")
        x = x + F.linear(F.gelu(F.linear(n2, t[p + "mlp.fc1.weight"], t[p + "mlp.fc1.bias"])), t[p + "mlp.fc2.weight"], t[p + "mlp.fc2.bias"])
    y = ln(x, "model.audio_tower.layer_norm")
    y = F.linear(y, t["model.proj.weight"], t["model.proj.bias"])
    up = F.conv1d(y.t()[None], t["model.upsampler.conv.weight"], t["model.upsampler.conv.bias"], padding=1)[0].t()   # [rows, r c]
    sub = torch.relu(up.reshape(rows * spec.factor, spec.head_hidden))
    dense = torch.relu(F.linear(sub, t["classifier.dense.weight"], t["classifier.dense.bias"]))
    return F.linear(dense, t["classifier.out_proj.weight"], t["classifier.out_proj.bias"])


def save_model(directory: str | Path, spec: DiarizationSpec, tensors: dict[str, torch.Tensor]) -> None:
    from ..loaders.safetensors_io import save_safetensors
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    root, processor = spec.to_json()
    (d / "config.json").write_text(json.dumps(root))
    (d / "processor_config.json").write_text(json.dumps(processor))
    save_safetensors(d / "model.safetensors", {k: v.float().contiguous() for k, v in tensors.items()})


def load_model(directory: str | Path, device: torch.device | str = "cpu") -> DiarizationModel:
    from ..loaders.safetensors_io import MappedCheckpoint
    d = Path(directory)
    spec = DiarizationSpec.from_json(json.loads((d / "config.json").read_text()), json.loads((d / "processor_config.json").read_text()))
    ckpt = MappedCheckpoint(d)
    return DiarizationModel(spec, {n: ckpt.tensor(n) for n in ckpt.names()}, device)


def diarize_file(directory: str | Path, audio_path: str | Path, device: torch.device | str = "cpu", stream: bool = False,
                 threshold: float = DEFAULT_THRESHOLD, mode: str | None = None) -> list[TextSegment]:
    from .audio import load_audio
    model = load_model(directory, device)
    return model.diarize(load_audio(audio_path, model.spec.mel.sampling_rate), stream=stream, threshold=threshold, mode=mode)
