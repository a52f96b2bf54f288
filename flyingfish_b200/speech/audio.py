"""Audio input: RIFF/WAVE reading and writing, channel mix-down, band-limited resampling and the log-mel front end.

The reference decodes audio on the host (src/audio.rs: a radix-2 FFT loop per frame, src/media.rs for containers); here
the waveform goes to the device once and ``ops/speech_ops.logmel`` computes every frame in one launch."""
from __future__ import annotations

import math
import struct
from dataclasses import dataclass
from pathlib import Path

import torch

from ..ops import speech_ops


class AudioError(ValueError):
    pass


def read_wav(path: str | Path) -> tuple[torch.Tensor, int]:
    """Reads PCM (8/16/24/32-bit integer) or IEEE-float (32/64-bit) RIFF/WAVE data.
    Returns ``([channels, samples] FP32 in [-1, 1], sampling_rate)``."""
    data = Path(path).read_bytes()
    if len(data) < 12 or data[:4] != b"RIFF" or data[8:12] != b"WAVE":
        raise AudioError("not a RIFF/WAVE file")
    off, fmt, pcm = 12, None, None
    while off + 8 <= len(data):
        tag, size = data[off:off + 4], struct.unpack_from("<I", data, off + 4)[0]
        body = data[off + 8: off + 8 + size]
        if tag == b"fmt ":
            if size < 16:
                raise AudioError("short fmt chunk")
            code, channels, rate, _, align, bits = struct.unpack_from("<HHIIHH", body)
            if code == 0xFFFE and size >= 26:            # WAVE_FORMAT_EXTENSIBLE: the sub-format's first two bytes
                code = struct.unpack_from("<H", body, 24)[0]
            fmt = (code, channels, rate, align, bits)
        elif tag == b"data":
            pcm = body
        off += 8 + size + (size & 1)
    if fmt is None or pcm is None:
        raise AudioError("missing fmt or data chunk")
    code, channels, rate, align, bits = fmt
    if channels < 1 or rate < 1 or bits % 8 or align != channels * bits // 8:
        raise AudioError("inconsistent fmt chunk")
    count = len(pcm) // align
    pcm = pcm[: count * align]
    if code == 1:
        if bits == 8:
            x = (torch.frombuffer(bytearray(pcm), dtype=torch.uint8).float() - 128.0) / 128.0
        elif bits == 16:
            x = torch.frombuffer(bytearray(pcm), dtype=torch.int16).float() / 32768.0
        elif bits == 24:
            raw = torch.frombuffer(bytearray(pcm), dtype=torch.uint8).reshape(-1, 3).to(torch.int32)
            v = raw[:, 0] | (raw[:, 1] << 8) | (raw[:, 2] << 16)
            v = torch.where(v >= 1 << 23, v - (1 << 24), v)
            x = v.float() / float(1 << 23)
        elif bits == 32:
            x = torch.frombuffer(bytearray(pcm), dtype=torch.int32).double().div(2147483648.0).float()
        else:
            raise AudioError(f"unsupported PCM width {bits}")
    elif code == 3:
        if bits == 32:
            x = torch.frombuffer(bytearray(pcm), dtype=torch.float32).clone()
        elif bits == 64:
            x = torch.frombuffer(bytearray(pcm), dtype=torch.float64).float()
        else:
            raise AudioError(f"unsupported float width {bits}")
    else:
        raise AudioError(f"unsupported WAVE format code {code}")
    if not torch.isfinite(x).all():
        raise AudioError("non-finite samples")
    return x.reshape(count, channels).t().contiguous(), rate


def write_wav(path: str | Path, wave: torch.Tensor, rate: int) -> None:
    """Writes ``[channels, samples]`` (or ``[samples]``) FP32 in [-1, 1] as 16-bit PCM."""
    w = wave.detach().float().cpu()
    if w.dim() == 1:
        w = w[None, :]
    pcm = (w.clamp(-1.0, 1.0) * 32767.0).round().to(torch.int16).t().contiguous().numpy().tobytes()
    channels = w.shape[0]
    header = b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVE" + b"fmt " + struct.pack(
        "<IHHIIHH", 16, 1, channels, rate, rate * channels * 2, channels * 2, 16) + b"data" + struct.pack("<I", len(pcm))
    Path(path).write_bytes(header + pcm)


def mix_down(wave: torch.Tensor) -> torch.Tensor:
    """[channels, samples] -> [samples]: the mean of the channels."""
    return wave.mean(dim=0) if wave.dim() == 2 else wave


def resample(wave: torch.Tensor, src_rate: int, dst_rate: int, taps: int = 16) -> torch.Tensor:
    """Band-limited resampling of a mono waveform by a Hann-windowed sinc interpolator (``taps`` zero crossings on each
    side, cut-off at the lower Nyquist frequency)."""
    if src_rate == dst_rate:
        return wave
    g = math.gcd(src_rate, dst_rate)
    up, down = dst_rate // g, src_rate // g
    n_out = (wave.numel() * up + down - 1) // down
    cutoff = min(1.0, up / down)
    width = int(math.ceil(taps / cutoff))
    t_out = torch.arange(n_out, dtype=torch.float64) * down / up        # positions in source samples
    base = torch.floor(t_out).long()
    k = torch.arange(-width + 1, width + 1)
    idx = base[:, None] + k[None, :]
    dist = t_out[:, None] - idx.double()
    win = torch.where(dist.abs() < width, 0.5 * (1 + torch.cos(math.pi * dist / width)), torch.zeros_like(dist))
    kern = cutoff * torch.sinc(cutoff * dist) * win
    src = torch.nn.functional.pad(wave.double(), (width, width + 1))
    vals = src[(idx + width).clamp(0, src.numel() - 1)]
    return (vals * kern).sum(dim=1).float()


def load_audio(path: str | Path, rate: int = 16000) -> torch.Tensor:
    """A WAVE file as a mono FP32 waveform at ``rate`` Hz."""
    wave, src = read_wav(path)
    return resample(mix_down(wave), src, rate)


@dataclass(frozen=True)
class LogMelConfig:
    sampling_rate: int = 16000
    n_fft: int = 512
    win_length: int = 400
    hop_length: int = 160
    mel_bins: int = 128
    preemphasis: float = 0.97
    log_guard: float = 2.0 ** -24
    norm_eps: float = 1e-5
    normalize: bool = True             # per-utterance, per-band normalisation (off for streaming models)

    def check(self) -> None:
        if not (self.sampling_rate > 0 and self.hop_length > 0 and self.mel_bins > 0 and 1 < self.win_length <= self.n_fft
                and self.n_fft & (self.n_fft - 1) == 0 and 32 <= self.n_fft <= 1024 and self.log_guard > 0
                and self.norm_eps > 0 and math.isfinite(self.preemphasis)):
            raise AudioError("invalid log-mel geometry or constants")


class LogMel:
    """Log-mel feature extractor. ``window`` / ``filters`` may come from a checkpoint (a ``[win_length]`` window is
    centred into the ``n_fft`` frame); otherwise a Hann window and Slaney-scale filters are generated."""

    def __init__(self, config: LogMelConfig, device: torch.device | str = "cpu", window: torch.Tensor | None = None,
                 filters: torch.Tensor | None = None):
        config.check()
        self.config = config
        bins = config.n_fft // 2 + 1
        if window is None:
            win = speech_ops.hann_window(config.win_length, config.n_fft)
        else:
            if not (2 <= window.numel() <= config.n_fft) or not torch.isfinite(window).all():
                raise AudioError(f"published window length {window.numel()}")
            win = torch.zeros(config.n_fft)
            first = (config.n_fft - window.numel()) // 2
            win[first:first + window.numel()] = window.float().cpu()
        if filters is None:
            fb = speech_ops.mel_filterbank(config.sampling_rate, config.n_fft, config.mel_bins)
        else:
            if tuple(filters.shape) != (config.mel_bins, bins) or not torch.isfinite(filters).all():
                raise AudioError(f"published filterbank shape {tuple(filters.shape)}")
            fb = filters.float().cpu().contiguous()
        self.device = torch.device(device)
        self.window = win.to(self.device)
        self.filters = fb.to(self.device)
        self.ranges = speech_ops.band_ranges(fb).to(self.device)

    def extract(self, waveforms: list[torch.Tensor], normalize: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
        """Mono waveforms -> ``([batch, frames, mel_bins] FP32, valid frames [batch] int32)``; shorter utterances are
        zero padded and their frames beyond ``len // hop`` come back zero."""
        hop = self.config.hop_length
        if not waveforms:
            raise AudioError("empty audio batch")
        for w in waveforms:
            if w.numel() < 2 * hop or not torch.isfinite(w).all():
                raise AudioError("audio needs at least two valid frames and finite samples")
        longest = max(w.numel() for w in waveforms)
        batch = torch.zeros(len(waveforms), longest, dtype=torch.float32)
        for i, w in enumerate(waveforms):
            batch[i, : w.numel()] = w.float().cpu()
        lens = torch.tensor([w.numel() for w in waveforms], dtype=torch.int32)
        feat = speech_ops.logmel(batch.to(self.device), lens.to(self.device), self.window, self.filters, self.ranges, hop,
                                 self.config.preemphasis, self.config.log_guard, normalize, self.config.norm_eps)
        return feat, (lens // hop).to(torch.int32)


class StreamingLogMel:
    """Log-mel frames of a growing waveform, un-normalised, identical to what ``LogMel.extract(normalize=False)`` gives
    for the whole utterance. A frame is emitted once the samples under its window have arrived (``last`` flushes the
    frames that look past the end, as the offline path computes them); every call re-runs the extractor over the new
    frames plus two frames of lead-in so that windows and pre-emphasis see real samples on their left."""

    def __init__(self, mel: LogMel):
        self.mel = mel
        self.buf = torch.zeros(0, dtype=torch.float32)
        self.emitted = 0
        self.finished = False

    def push(self, samples: torch.Tensor, last: bool = False) -> torch.Tensor:
        if self.finished:
            raise RuntimeError("the stream is finished")
        cfg = self.mel.config
        hop, half = cfg.hop_length, cfg.n_fft // 2
        self.buf = torch.cat([self.buf, samples.detach().float().cpu().reshape(-1)])
        n = self.buf.numel()
        ready = n // hop if last else (max(0, (n - half) // hop + 1) if n >= half else 0)
        if last:
            self.finished = True
        t0 = self.emitted
        empty = torch.zeros(0, cfg.mel_bins, dtype=torch.float32, device=self.mel.device)
        if ready <= t0:
            return empty
        lead = min(2, t0)
        s0 = (t0 - lead) * hop
        end = n if last else min(n, (ready - 1) * hop + half + hop)
        sub = self.buf[s0:end]
        if sub.numel() < 2 * hop:
            if not last:
                return empty
            sub = torch.nn.functional.pad(sub, (0, 2 * hop - sub.numel()))
        feat, _ = self.mel.extract([sub], normalize=False)
        self.emitted = ready
        return feat[0, lead: lead + ready - t0]
