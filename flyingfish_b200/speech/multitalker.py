"""Speaker-attributed streaming recognition ("multitalker" streaming RNN-T in the NeMo archive layout).

One cache-aware streaming FastConformer / RNN-T serves up to four speaker lanes over the same audio. What tells the lanes
apart are two small *speaker kernels* in front of encoder layer 0 (src/multitalker.rs and
src/backend/cuda/engine_multitalker.rs of the reference; src/backend/cuda/engine_parakeet.rs:3365-3400 for the kernel):
with ``m`` the lane's own speaker activity per encoder row and ``b`` the activity of any *other* speaker,

    h <- h + W2 relu(W1 (m * h) + b1) + b2            (speaker kernel,    tensors ``spk_kernels.0.{0,3}``)
    h <- h + V2 relu(V1 (b * h) + c1) + c2            (background kernel, tensors ``bg_spk_kernels.0.{0,3}``)

The activity comes from a diarizer at the encoder's 80 ms row grid (``diarization.speaker_masks``). A lane runs only
while its speaker was active within the last 28 rows; a parked lane keeps its layer caches and prediction-network state
and continues on its own row grid when the speaker returns.

B200 mapping: the stem runs once per chunk for all lanes; every lane has a ``ConformerStream`` of its own for the layer
caches; the lanes' transducer states are rows of one batched decoder whose step is a replayed CUDA graph
(``TdtDecoder.extend_lanes``), so the lanes of a chunk decode together.

Word times: a token's row is mapped back from the lane's own row count to the row of the clip it was computed from, so
times are clip times also for lanes that were parked in between (the published wrapper adds the lane-local row to a
chunk offset counted in active steps; for a lane that never pauses both give the same times)."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch

from ..models.conformer import ConformerStream
from ..ops import vision_ops
from .audio import StreamingLogMel
from .nemo import UnigramVocab, canonical_tensors, spec_from_yaml
from .parakeet import ParakeetModel, ParakeetSpec
from .transcript import WORD_MARKER, TextSegment

BF16 = torch.bfloat16
GATE_ROWS = 28                        # a lane stays live this many rows after its speaker's last activity
KERNEL_TENSORS = ("spk_kernels.0.0", "spk_kernels.0.3", "bg_spk_kernels.0.0", "bg_spk_kernels.0.3")


@dataclass(frozen=True)
class MultitalkerSpec:
    asr: ParakeetSpec
    speakers: int = 4

    @classmethod
    def from_yaml(cls, text: str) -> "MultitalkerSpec":
        import yaml
        root = yaml.safe_load(text)
        try:
            if str(root["spk_kernel_type"]) != "ff" or [int(v) for v in root["spk_kernel_layers"]] != [0] or not root["add_bg_spk_kernel"]:
                raise ValueError("unsupported speaker-kernel variant (feed-forward kernels at layer 0 with a background kernel)")
            speakers = int(root["model_defaults"]["num_speakers"])
            max_symbols = int(root["decoding"]["greedy"]["max_symbols"])
        except KeyError as e:
            raise ValueError(f"model_config.yaml lacks {e}") from None
        if not (1 <= speakers <= 8):
            raise ValueError("speaker lanes outside 1..8")
        from dataclasses import replace
        return cls(replace(spec_from_yaml(text), max_symbols=max_symbols), speakers)

    def expected_tensors(self) -> dict[str, tuple[str, tuple[int, ...]]]:
        out = self.asr.expected_tensors()
        h = self.asr.encoder.hidden
        for name in KERNEL_TENSORS:
            out[name + ".weight"] = ("F32", (h, h))
            out[name + ".bias"] = ("F32", (h,))
        return out


@dataclass
class SpeakerTranscription:
    speaker: int
    start: float
    end: float
    text: str
    words: list[TextSegment] = field(default_factory=list)
    tokens: list[int] = field(default_factory=list)
    rows: list[int] = field(default_factory=list)            # clip row of every token


@dataclass
class MultitalkerTranscription:
    speakers: list[SpeakerTranscription]

    def to_json(self) -> str:
        return json.dumps({"speakers": [{"speaker": s.speaker, "start": s.start, "end": s.end, "text": s.text,
                                         "words": [asdict(w) for w in s.words]} for s in self.speakers]}, ensure_ascii=False)

    def to_text(self) -> str:
        return "".join(f"speaker_{s.speaker}: {s.text}\n" for s in self.speakers)


def speaker_words(tokens: list[int], rows: list[int], piece, frame_seconds: float) -> tuple[str, list[TextSegment]]:
    """Tokens with the clip row each was emitted at -> text and words: a word runs from its first token's row to one
    row past its last token's; a piece that starts with the word marker opens a word (src/multitalker.rs
    ``speaker_words`` of the reference)."""
    if len(tokens) != len(rows):
        raise ValueError("tokens and rows differ in length")
    words: list[TextSegment] = []
    for tok, row in zip(tokens, rows):
        p = piece(tok)
        if not p or (p.startswith("<") and p.endswith(">")):
            continue
        opens = p.startswith(WORD_MARKER)
        body = p.replace(WORD_MARKER, "")
        if opens or not words:
            if not body and opens:
                words.append(TextSegment(row * frame_seconds, (row + 1) * frame_seconds, ""))
                continue
            words.append(TextSegment(row * frame_seconds, (row + 1) * frame_seconds, body))
        else:
            words[-1].text += body
            words[-1].end = (row + 1) * frame_seconds
    words = [w for w in words if w.text]
    return " ".join(w.text for w in words), words


class MultitalkerModel(ParakeetModel):
    """The streaming RNN-T with its speaker and background kernels."""

    def __init__(self, spec: MultitalkerSpec, tensors: dict[str, torch.Tensor], device: torch.device | str = "cpu", tokenizer=None,
                 max_rows: int = 0):
        asr_names = set(spec.asr.expected_tensors())
        super().__init__(spec.asr, {n: t for n, t in tensors.items() if n in asr_names}, device, tokenizer=tokenizer, max_rows=max_rows,
                         max_batch=max(spec.speakers, 1))
        self.mt = spec
        h = spec.asr.encoder.hidden

        def lin(name: str):
            w, b = tensors[name + ".weight"], tensors[name + ".bias"]
            if tuple(w.shape) != (h, h) or tuple(b.shape) != (h,):
                raise ValueError(f"speaker kernel tensor {name} has shape {tuple(w.shape)} / {tuple(b.shape)}")
            return w.float().to(BF16).contiguous().to(self.device), b.float().to(BF16).contiguous().to(self.device)
        self.spk = (lin(KERNEL_TENSORS[0]), lin(KERNEL_TENSORS[1]))
        self.bg = (lin(KERNEL_TENSORS[2]), lin(KERNEL_TENSORS[3]))

    @classmethod
    def load(cls, path: str | Path, device: torch.device | str = "cpu") -> "MultitalkerModel":
        from ..loaders.pth import read_nemo, read_nemo_member
        text, weights = read_nemo(path)
        spec = MultitalkerSpec.from_yaml(text)
        try:
            raw = {n: weights.tensor(n).clone() for n in weights.records}
        finally:
            weights.close()
        tensors = canonical_tensors(spec.asr, raw)
        for name in KERNEL_TENSORS:
            for part in (".weight", ".bias"):
                if name + part not in raw:
                    raise ValueError(f"NeMo tensor missing: {name + part}")
                tensors[name + part] = raw[name + part]
        for name, (_, shape) in spec.expected_tensors().items():
            if name not in tensors:
                raise ValueError(f"NeMo tensor missing: {name}")
            if tuple(tensors[name].shape) != tuple(shape) and not name.endswith("num_batches_tracked"):
                raise ValueError(f"NeMo tensor shape mismatch: {name} {tuple(tensors[name].shape)} != {tuple(shape)}")
        try:
            vocab = UnigramVocab(read_nemo_member(path, "_tokenizer.vocab").decode("utf-8"))
        except ValueError:
            vocab = None
        return cls(spec, tensors, device, tokenizer=vocab)

    def speaker_kernels(self, h: torch.Tensor, own: torch.Tensor, others: torch.Tensor) -> torch.Tensor:
        """Layer-0 rows [n, hidden] conditioned on one lane: ``own`` / ``others`` [n] are the lane's speaker activity
        and the activity of any other speaker per row."""
        for (up, down), mask in ((self.spk, own), (self.bg, others)):
            scaled = (h.float() * mask.to(h.device, torch.float32)[:, None]).to(BF16)
            mid = vision_ops.linear_bias_act(scaled, up[0], up[1], "relu")
            h = (h.float() + vision_ops.linear_bias_act(mid, down[0], down[1], "none").float()).to(BF16)
        return h

    def stream(self, activity: torch.Tensor, gating: bool = True, masked: bool = False) -> "MultitalkerStream":
        return MultitalkerStream(self, activity, gating, masked)

    def transcribe_speakers(self, waveform: torch.Tensor, activity: torch.Tensor, gating: bool = True,
                            piece_seconds: float = 1.12, masked: bool = False) -> MultitalkerTranscription:
        """One clip with its speaker activity ``[rows, lanes]`` at the 80 ms grid -> one transcript per active speaker."""
        st = self.stream(activity, gating, masked)
        piece = max(1, int(piece_seconds * self.spec.mel.sampling_rate))
        for at in range(0, waveform.numel(), piece):
            nxt = min(waveform.numel(), at + piece)
            st.push(waveform[at:nxt], last=nxt == waveform.numel())
        return st.transcription()


class MultitalkerStream:
    """Audio in pieces, tokens per speaker lane out. ``activity`` [rows, lanes] (values above 0.5 = speaking) covers the
    clip at the encoder's row grid; rows beyond its end count as "own speaker active, nobody else"."""

    def __init__(self, model: MultitalkerModel, activity: torch.Tensor, gating: bool = True, masked: bool = False):
        """``masked``: the feature-masking variant -- instead of conditioning layer 0, every lane gets its own log-mel
        input in which the frames of rows where its speaker is silent are zeroed (frames that are exactly zero take the
        log floor), the kernels run with "own speaker active, nobody else", and every lane runs its own stem."""
        spec = model.spec
        if spec.mel.normalize:
            raise ValueError("streaming needs un-normalised features")
        act = activity.detach().float().cpu()
        if act.dim() != 2 or not (1 <= act.shape[1] <= model.mt.speakers):
            raise ValueError(f"speaker activity must be [rows, 1..{model.mt.speakers}]")
        self.model, self.activity, self.gating, self.masked = model, act, gating, masked
        self.frames_seen = 0
        self.lanes = act.shape[1]
        self.front = StreamingLogMel(model.mel)
        self.stem = ConformerStream(model.encoder)              # frames and stem only; its layer caches stay empty
        self.lane_streams = [ConformerStream(model.encoder) for _ in range(self.lanes)]
        model.decoder.begin_stream(self.lanes)
        self.tokens: list[list[int]] = [[] for _ in range(self.lanes)]
        self.token_rows: list[list[int]] = [[] for _ in range(self.lanes)]
        self.row_map: list[list[int]] = [[] for _ in range(self.lanes)]      # clip row of every row a lane has encoded
        self.steps = 0
        self.lane_steps = [0] * self.lanes

    def live_lanes(self, end_row: int) -> list[int]:
        """Lanes whose speaker was active within the ``GATE_ROWS`` rows before ``end_row``."""
        if not self.gating:
            return list(range(self.lanes))
        end = min(end_row, self.activity.shape[0])
        window = self.activity[max(0, end - GATE_ROWS): end]
        return [lane for lane in range(self.lanes) if window.shape[0] and bool((window[:, lane] > 0.5).any())]

    def masks(self, first_row: int, n: int, lane: int) -> tuple[torch.Tensor, torch.Tensor]:
        own, others = torch.ones(n), torch.zeros(n)
        have = max(0, min(n, self.activity.shape[0] - first_row))
        if have:
            rows = self.activity[first_row: first_row + have]
            own[:have] = rows[:, lane]
            rest = torch.cat([rows[:, :lane], rows[:, lane + 1:]], dim=1)
            if rest.shape[1]:
                others[:have] = (rest > 0.5).any(dim=1).float()
        return own, others

    def masked_frames(self, frames: torch.Tensor, lane: int) -> torch.Tensor:
        """The new log-mel frames as lane ``lane`` sees them in the feature-masking variant: a frame belongs to row
        ``frame // 8``; rows where the lane's speaker is silent are zeroed, rows beyond the activity count as active, and
        values that are exactly zero become the log floor (src/backend/cuda/engine_multitalker.rs:414-438 of the
        reference)."""
        n = frames.shape[0]
        rows = (torch.arange(n) + self.frames_seen) // 8
        inside = rows < self.activity.shape[0]
        keep = torch.ones(n)
        keep[inside] = (self.activity[rows[inside], lane] > 0.5).float()
        floor = float(torch.log(torch.tensor(self.model.spec.mel.log_guard)))
        f = frames.float()
        return torch.where(f == 0.0, torch.full_like(f, floor), f * keep.to(f.device)[:, None])

    def push(self, samples: torch.Tensor, last: bool = False) -> dict[int, list[int]]:
        """Feeds samples; returns the tokens each lane recognised in this call."""
        model, dec = self.model, self.model.decoder
        new: dict[int, list[int]] = {}
        frames = self.front.push(samples, last)
        if self.masked:
            per_lane = [list(self.lane_streams[lane].stem_chunks(self.masked_frames(frames, lane), last)) for lane in range(self.lanes)]
            chunks = [(per_lane[0][i][0], [per_lane[lane][i][1] for lane in range(self.lanes)]) for i in range(len(per_lane[0]))]
            self.frames_seen += frames.shape[0]
        else:
            chunks = [(first, [h] * self.lanes) for first, h in self.stem.stem_chunks(frames, last)]
        for first, hs in chunks:
            n = hs[0].shape[0]
            live = self.live_lanes(first + n)
            self.steps += 1
            if not live:
                continue
            projected = {}
            for lane in live:
                own, others = (torch.ones(n), torch.zeros(n)) if self.masked else self.masks(first, n, lane)
                rows = self.lane_streams[lane]._layers(model.speaker_kernels(hs[lane], own, others))
                projected[lane] = dec.project(rows)
                self.row_map[lane] += list(range(first, first + n))
                self.lane_steps[lane] += 1
            for lane, traj in dec.extend_lanes(projected).items():
                for tok, frm in zip(traj.tokens, traj.frames):
                    if tok != model.spec.blank:
                        self.tokens[lane].append(tok)
                        self.token_rows[lane].append(self.row_map[lane][min(frm, len(self.row_map[lane]) - 1)])
                        new.setdefault(lane, []).append(tok)
        return new

    def transcription(self) -> MultitalkerTranscription:
        tk = self.model.tokenizer
        if tk is None:
            piece = lambda t: f"{WORD_MARKER}{t}"
        else:
            piece = tk.piece
        out = []
        for lane in range(self.lanes):
            text, words = speaker_words(self.tokens[lane], self.token_rows[lane], piece, self.model.spec.frame_seconds)
            if not words:
                continue
            out.append(SpeakerTranscription(lane, words[0].start, words[-1].end, text, words, list(self.tokens[lane]),
                                            list(self.token_rows[lane])))
        return MultitalkerTranscription(out)


def transcribe_multitalker(nemo_path: str | Path, diarization_dir: str | Path, waveform: torch.Tensor,
                           device: torch.device | str = "cpu", threshold: float = 0.5, stream_diarizer: bool = True,
                           masked: bool = False) -> MultitalkerTranscription:
    """The whole pipeline on one 16 kHz mono clip: the diarizer's pooled speaker activity selects the lanes, the
    multitalker model transcribes each of them. A diarizer channel beyond the model's lanes that is ever active is an
    error (src/multitalker.rs ``transcribe`` of the reference)."""
    from .diarization import load_model as load_diarizer, speaker_masks
    diarizer = load_diarizer(diarization_dir, device)
    model = MultitalkerModel.load(nemo_path, device)
    masks, seconds = speaker_masks(diarizer, waveform, stream=stream_diarizer, threshold=threshold)
    if abs(seconds - model.spec.frame_seconds) > 1e-9:
        raise ValueError(f"diarization frame period {seconds} s vs the recognition grid {model.spec.frame_seconds} s")
    lanes = model.mt.speakers
    beyond = [c for c in range(lanes, masks.shape[1]) if bool(masks[:, c].any())]
    if beyond:
        raise ValueError(f"diarization activates speaker channels {beyond} beyond the {lanes} lanes the model serves")
    return model.transcribe_speakers(waveform, masks[:, :lanes].float(), masked=masked)
