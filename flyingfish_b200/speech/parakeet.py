"""Parakeet-style speech recognition: FastConformer encoder + token-and-duration transducer (TDT) decoder.

Configuration and tensor contract follow the published ``ParakeetForTDT`` layout (src/parakeet.rs:295-577 of the
reference); the greedy decode follows src/backend/cuda/engine_parakeet.rs:2550-2633. What differs is where the loop
runs: the prediction-network state, the current frame, the last token and the trajectory live on the device, one decode
step is a fixed sequence of launches replayed from a CUDA graph, and the host reads the state words once per
``CHECK_EVERY`` steps instead of one selection per step."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path

import torch

from .. import ops
from ..models.conformer import ConformerEncoder, ConformerSpec, random_tensors
from ..ops import speech_ops, vision_ops
from ..ops.speech_ops import (TS_ADVANCE, TS_CAP, TS_COUNT, TS_DONE, TS_ERROR, TS_FRAME, TS_MAXSYM, TS_TOKEN, TS_VALID,
                              TS_WORDS)
from .audio import LogMel, LogMelConfig
from .transcript import Transcription, WORD_MARKER, tdt_cues

BF16 = torch.bfloat16
CHECK_EVERY = 32           # decode steps replayed between two reads of the device state


@dataclass(frozen=True)
class ParakeetSpec:
    encoder: ConformerSpec = field(default_factory=ConformerSpec)
    decoder_hidden: int = 640
    decoder_layers: int = 2
    vocab: int = 8193                  # tokens including the blank
    blank: int = 8192
    max_symbols: int = 10
    eos: int = 3
    pad: int = 2
    durations: tuple[int, ...] = (0, 1, 2, 3, 4)       # empty: a plain transducer (RNN-T) without a duration head
    mel: LogMelConfig = field(default_factory=LogMelConfig)
    # prompt-conditioned streaming RNN-T (``Nemotron3_5AsrForRNNT``): every encoder row, extended by the one-hot of a
    # prompt id (a language), goes through a two-layer ReLU adapter before the joint projection
    prompts: int = 0
    prompt_intermediate: int = 0
    default_prompt: int = 0
    prompt_dictionary: tuple[tuple[str, int], ...] = ()

    @property
    def joint_out(self) -> int:
        return self.vocab + len(self.durations)

    @property
    def frame_seconds(self) -> float:
        return 8 * self.mel.hop_length / self.mel.sampling_rate

    def check(self) -> None:
        self.encoder.check()
        if not (0 <= self.blank < self.vocab and self.decoder_hidden % 8 == 0 and self.decoder_layers >= 1
                and self.max_symbols >= 1):
            raise ValueError("unsupported transducer decoder geometry")

    @classmethod
    def from_json(cls, root: dict, processor: dict, generation: dict) -> "ParakeetSpec":
        """``config.json``, ``processor_config.json`` and ``generation_config.json`` of a published checkpoint."""
        nemotron = root.get("model_type") == "nemotron3_5_asr" and root.get("architectures") == ["Nemotron3_5AsrForRNNT"]
        if not nemotron and (root.get("model_type") != "parakeet_tdt" or root.get("architectures") != ["ParakeetForTDT"]):
            raise ValueError("not a Parakeet TDT / Nemotron RNN-T configuration")
        if root.get("hidden_act") != "relu":
            raise ValueError("unsupported joint activation")
        enc = root.get("encoder_config")
        if not isinstance(enc, dict) or enc.get("model_type") != ("nemotron_asr_streaming_encoder" if nemotron else "parakeet_encoder"):
            raise ValueError("encoder_config missing")
        if nemotron and (list(root.get("durations", [])) != [] or "sliding_window" not in enc):
            raise ValueError("the prompt-conditioned RNN-T has no duration head and a streaming encoder")
        for key, want in (("hidden_act", "silu"), ("scale_input", False), ("subsampling_conv_kernel_size", 3),
                          ("subsampling_conv_stride", 2), ("subsampling_factor", 8)):
            if enc.get(key) != want:
                raise ValueError(f"unsupported encoder setting {key}={enc.get(key)!r}")
        if enc.get("num_key_value_heads", enc["num_attention_heads"]) != enc["num_attention_heads"]:
            raise ValueError("grouped-query encoders are not supported")
        feats = processor.get("feature_extractor")
        if not isinstance(feats, dict):
            raise ValueError("feature_extractor missing")
        if feats.get("padding_side", "right") != "right" or float(feats.get("padding_value", 0.0)) != 0.0:
            raise ValueError("unsupported feature padding")
        mel = LogMelConfig(sampling_rate=int(feats["sampling_rate"]), n_fft=int(feats["n_fft"]), win_length=int(feats["win_length"]),
                           hop_length=int(feats["hop_length"]), mel_bins=int(feats["feature_size"]),
                           preemphasis=float(feats["preemphasis"]))
        if mel.mel_bins != int(enc["num_mel_bins"]):
            raise ValueError("feature size and encoder mel bins differ")
        stream = {}
        if "sliding_window" in enc:
            # cache-aware streaming encoder (the layout of streaming RNN-T checkpoints): chunks of look-ahead + 1 rows,
            # a left context of whole chunks, causal convolutions and stem pads, layer norm in the convolution module,
            # un-normalised features
            chunk = int(enc.get("default_num_lookahead_tokens", 0)) + 1
            left = int(enc["sliding_window"])
            if left % chunk:
                raise ValueError(f"sliding-window left context {left} does not divide by chunk {chunk}")
            stream = dict(chunk_size=chunk, left_chunks=left // chunk, causal_conv=True, pad_left=2, pad_right=1, conv_batch_norm=False,
                          conv_names=("subsampling.conv_in", "subsampling.layers.0.depthwise_conv", "subsampling.layers.1.depthwise_conv"),
                          pointwise_names=("subsampling.layers.0.pointwise_conv", "subsampling.layers.1.pointwise_conv"))
            mel = LogMelConfig(sampling_rate=mel.sampling_rate, n_fft=mel.n_fft, win_length=mel.win_length, hop_length=mel.hop_length,
                               mel_bins=mel.mel_bins, preemphasis=mel.preemphasis, normalize=False)
        encoder = ConformerSpec(layers=int(enc["num_hidden_layers"]), hidden=int(enc["hidden_size"]),
                                heads=int(enc["num_attention_heads"]), intermediate=int(enc["intermediate_size"]),
                                conv_kernel=int(enc["conv_kernel_size"]), mel_bins=mel.mel_bins,
                                sub_channels=int(enc["subsampling_conv_channels"]), attention_bias=bool(enc["attention_bias"]),
                                convolution_bias=bool(enc["convolution_bias"]), max_position=int(enc["max_position_embeddings"]),
                                **stream)
        extra = {}
        if nemotron:
            table = processor.get("prompt_dictionary") or {}
            if not isinstance(table, dict) or any(not (0 <= int(v) < int(root["num_prompts"])) for v in table.values()):
                raise ValueError("prompt_dictionary is not a map of names to prompt ids")
            extra = dict(prompts=int(root["num_prompts"]), prompt_intermediate=int(root["prompt_intermediate_size"]),
                         default_prompt=int(root["default_prompt_id"]), prompt_dictionary=tuple(sorted((str(k), int(v)) for k, v in table.items())))
            if not (0 <= extra["default_prompt"] < extra["prompts"]):
                raise ValueError("default_prompt_id outside the prompt table")
        spec = cls(encoder=encoder, decoder_hidden=int(root["decoder_hidden_size"]), decoder_layers=int(root["num_decoder_layers"]),
                   vocab=int(root["vocab_size"]), blank=int(root["blank_token_id"]), max_symbols=int(root["max_symbols_per_step"]),
                   eos=int(generation.get("eos_token_id", -1 if nemotron else 3)), pad=int(root.get("pad_token_id", 2)),
                   durations=tuple(int(d) for d in root["durations"]), mel=mel, **extra)
        if generation.get("decoder_start_token_id", spec.blank) != spec.blank:
            raise ValueError("decoder start token differs from the blank")
        spec.check()
        return spec

    @classmethod
    def read(cls, directory: str | Path) -> "ParakeetSpec":
        d = Path(directory)
        load = lambda n: json.loads((d / n).read_text())
        return cls.from_json(load("config.json"), load("processor_config.json"), load("generation_config.json"))

    def to_json(self) -> tuple[dict, dict, dict]:
        """The three configuration files of this spec in the published layout."""
        e = self.encoder
        root = {"architectures": ["ParakeetForTDT"], "model_type": "parakeet_tdt", "dtype": "float32", "hidden_act": "relu",
                "initializer_range": 0.02, "is_encoder_decoder": True, "pad_token_id": self.pad, "vocab_size": self.vocab,
                "blank_token_id": self.blank, "durations": list(self.durations), "decoder_hidden_size": self.decoder_hidden,
                "num_decoder_layers": self.decoder_layers, "max_symbols_per_step": self.max_symbols,
                "encoder_config": {"model_type": "parakeet_encoder", "hidden_act": "silu", "scale_input": False,
                                   "attention_bias": e.attention_bias, "convolution_bias": e.convolution_bias,
                                   "conv_kernel_size": e.conv_kernel, "hidden_size": e.hidden, "intermediate_size": e.intermediate,
                                   "max_position_embeddings": e.max_position, "num_attention_heads": e.heads,
                                   "num_key_value_heads": e.heads, "num_hidden_layers": e.layers, "num_mel_bins": e.mel_bins,
                                   "subsampling_conv_channels": e.sub_channels, "subsampling_conv_kernel_size": 3,
                                   "subsampling_conv_stride": 2, "subsampling_factor": 8}}
        if e.chunk_size > 0:
            root["encoder_config"].update(sliding_window=e.left_chunks * e.chunk_size, default_num_lookahead_tokens=e.chunk_size - 1)
        m = self.mel
        if self.prompts > 0:
            root.update(architectures=["Nemotron3_5AsrForRNNT"], model_type="nemotron3_5_asr", num_prompts=self.prompts,
                        prompt_intermediate_size=self.prompt_intermediate, default_prompt_id=self.default_prompt)
            root["encoder_config"]["model_type"] = "nemotron_asr_streaming_encoder"
        processor = {"processor_class": "ParakeetProcessor", "blank_token": "<blank>",
                     "feature_extractor": {"feature_extractor_type": "ParakeetFeatureExtractor", "feature_size": m.mel_bins,
                                           "hop_length": m.hop_length, "n_fft": m.n_fft, "padding_side": "right", "padding_value": 0.0,
                                           "preemphasis": m.preemphasis, "return_attention_mask": True,
                                           "sampling_rate": m.sampling_rate, "win_length": m.win_length}}
        generation = {"decoder_start_token_id": self.blank, "eos_token_id": self.eos, "pad_token_id": self.pad}
        if self.prompts > 0:
            processor["prompt_dictionary"] = dict(self.prompt_dictionary)
        return root, processor, generation

    def expected_tensors(self) -> dict[str, tuple[str, tuple[int, ...]]]:
        out = self.encoder.expected_tensors()
        h, d = self.encoder.hidden, self.decoder_hidden
        if self.prompts > 0:
            out["prompt_projector.linear_1.weight"] = ("F32", (self.prompt_intermediate, h + self.prompts))
            out["prompt_projector.linear_1.bias"] = ("F32", (self.prompt_intermediate,))
            out["prompt_projector.linear_2.weight"] = ("F32", (h, self.prompt_intermediate))
            out["prompt_projector.linear_2.bias"] = ("F32", (h,))
        out["encoder_projector.weight"] = ("F32", (d, h))
        out["encoder_projector.bias"] = ("F32", (d,))
        out["decoder.embedding.weight"] = ("F32", (self.vocab, d))
        out["decoder.decoder_projector.weight"] = ("F32", (d, d))
        out["decoder.decoder_projector.bias"] = ("F32", (d,))
        for layer in range(self.decoder_layers):
            for kind in ("weight_ih", "weight_hh"):
                out[f"decoder.lstm.{kind}_l{layer}"] = ("F32", (4 * d, d))
            for kind in ("bias_ih", "bias_hh"):
                out[f"decoder.lstm.{kind}_l{layer}"] = ("F32", (4 * d,))
        out["joint.head.weight"] = ("F32", (self.joint_out, d))
        out["joint.head.bias"] = ("F32", (self.joint_out,))
        return out

    def validate(self, names_shapes: dict[str, tuple[str, tuple[int, ...]]]) -> int:
        """Checks a checkpoint's (dtype, shape) table against the contract; returns the tensor count."""
        expected = self.expected_tensors()
        for name in expected:
            if name not in names_shapes:
                raise ValueError(f"Parakeet tensor missing: {name}")
        for name in names_shapes:
            if name not in expected:
                raise ValueError(f"Parakeet tensor unexpected: {name}")
        for name, entry in expected.items():
            if (names_shapes[name][0], tuple(names_shapes[name][1])) != entry:
                raise ValueError(f"Parakeet tensor contract mismatch: {name}")
        return len(expected)


def parakeet_tiny() -> ParakeetSpec:
    """A small random-init shape for tests: 2 layers, 128 hidden, two 64-wide heads, 32 mel bins."""
    enc = ConformerSpec(layers=2, hidden=128, heads=2, intermediate=256, conv_kernel=9, mel_bins=32, sub_channels=32,
                        max_position=512)
    return ParakeetSpec(encoder=enc, decoder_hidden=64, decoder_layers=2, vocab=41, blank=40, max_symbols=10, eos=3,
                        durations=(0, 1, 2, 3, 4), mel=LogMelConfig(mel_bins=32))


SHAPES = {"parakeet-tdt-0.6b": ParakeetSpec, "parakeet-tiny": parakeet_tiny}


@dataclass
class TdtTrajectory:
    tokens: list[int]
    durations: list[int]
    frames: list[int]
    capacity: int
    steps: int = 0
    state_reads: int = 0


class TdtDecoder:
    """Prediction network (embedding + LSTM stack), joint network and the greedy TDT loop, for up to ``max_batch``
    utterances stepping together (their states, frames and trajectories are separate rows of the device buffers)."""

    def __init__(self, spec: ParakeetSpec, tensors: dict[str, torch.Tensor], device: torch.device | str, max_rows: int = 0,
                 max_batch: int = 8):
        self.spec, self.device = spec, torch.device(device)
        dev, d = self.device, spec.decoder_hidden

        def w16(t: torch.Tensor) -> torch.Tensor:
            return t.float().to(BF16).contiguous().to(dev)

        self.enc_proj = (w16(tensors["encoder_projector.weight"]), w16(tensors["encoder_projector.bias"]))
        self.adapter = None
        self.prompt_id = spec.default_prompt
        if spec.prompts > 0:
            # the one-hot prompt columns of the first layer are folded into one bias row per prompt id
            h = spec.encoder.hidden
            w1 = tensors["prompt_projector.linear_1.weight"].float()
            bias_rows = tensors["prompt_projector.linear_1.bias"].float()[None, :] + w1[:, h:].t()
            self.adapter = (w16(w1[:, :h]), w16(bias_rows), w16(tensors["prompt_projector.linear_2.weight"]),
                            w16(tensors["prompt_projector.linear_2.bias"]))
        self.table = w16(tensors["decoder.embedding.weight"])
        self.w_pred = w16(tensors["decoder.decoder_projector.weight"])
        self.b_pred = tensors["decoder.decoder_projector.bias"].float().contiguous().to(dev)
        self.lstm = []
        for layer in range(spec.decoder_layers):
            w = torch.cat([tensors[f"decoder.lstm.weight_ih_l{layer}"].float(), tensors[f"decoder.lstm.weight_hh_l{layer}"].float()], dim=1)
            b = tensors[f"decoder.lstm.bias_ih_l{layer}"].float() + tensors[f"decoder.lstm.bias_hh_l{layer}"].float()
            self.lstm.append((w16(w), b.contiguous().to(dev)))
        n = spec.joint_out
        n_pad = (n + 15) // 16 * 16
        head = torch.zeros(n_pad, d)
        head[:n] = tensors["joint.head.weight"].float()
        self.w_head = w16(head)
        self.b_head = tensors["joint.head.bias"].float().contiguous().to(dev)
        self.durations = torch.tensor(spec.durations or (0,), dtype=torch.int32, device=dev)[: len(spec.durations)]
        # step buffers (fixed addresses: the step is captured once); one row per utterance
        self.max_rows = max_rows or spec.encoder.max_position
        self.max_batch = nb = max(1, max_batch)
        self.enc = torch.zeros(nb, self.max_rows, d, dtype=BF16, device=dev)
        self.xh = [torch.zeros(nb, 2 * d, dtype=BF16, device=dev) for _ in range(spec.decoder_layers)]
        self.cell = [torch.zeros(nb, d, dtype=torch.float32, device=dev) for _ in range(spec.decoder_layers)]
        self.top = torch.zeros(nb, d, dtype=BF16, device=dev)
        self.jh = torch.zeros(nb, d, dtype=BF16, device=dev)
        self.state = torch.zeros(nb, TS_WORDS, dtype=torch.int32, device=dev)
        cap = spec.max_symbols * self.max_rows + 1
        self.traj = tuple(torch.zeros(nb, cap, dtype=torch.int32, device=dev) for _ in range(3))
        self._graph: torch.cuda.CUDAGraph | None = None
        self.use_graph = self.device.type == "cuda"
        self.graph_replays = 0

    def project(self, encoded: torch.Tensor) -> torch.Tensor:
        """[rows, hidden] BF16 encoder output -> [rows, decoder_hidden] BF16 in the joint space (through the prompt
        adapter of prompt-conditioned models: ``relu(W1 [row; onehot(prompt)] + b1)``, then ``W2 . + b2``)."""
        if self.adapter is not None:
            w1, bias_rows, w2, b2 = self.adapter
            u = vision_ops.linear_bias_act(encoded, w1, bias_rows[self.prompt_id].contiguous(), "relu")
            encoded = vision_ops.linear_bias_act(u, w2, b2, "none")
        return vision_ops.linear_bias_act(encoded, self.enc_proj[0], self.enc_proj[1], "none")

    def reset(self, valid_rows: list[int] | int) -> list[int]:
        """Fresh decode state for ``len(valid_rows)`` utterances (the other rows of the batch are parked as done)."""
        spec = self.spec
        valid = [valid_rows] if isinstance(valid_rows, int) else list(valid_rows)
        for t in self.xh:
            t.zero_()
        for t in self.cell:
            t.zero_()
        cap_len = self.traj[0].shape[1]
        init = torch.zeros(self.max_batch, TS_WORDS, dtype=torch.int32)
        init[:, TS_DONE] = 1
        caps = []
        for b, rows in enumerate(valid):
            cap = min(spec.max_symbols * rows + 1, cap_len)
            caps.append(cap)
            init[b, TS_TOKEN], init[b, TS_COUNT], init[b, TS_ADVANCE], init[b, TS_VALID], init[b, TS_CAP] = spec.blank, 1, 1, rows, cap
            init[b, TS_MAXSYM], init[b, TS_DONE] = spec.max_symbols, 0
        self.state.copy_(init)
        first = torch.tensor([spec.blank, 0, 0], dtype=torch.int32)
        for t, v in zip(self.traj, first):
            t[:, :1] = v
        return caps

    def step(self) -> None:
        """One decode step of every utterance on the current stream (the sequence a CUDA graph captures)."""
        spec, d = self.spec, self.spec.decoder_hidden
        speech_ops.tdt_embed(self.table, self.state, self.xh[0])
        for layer, (w, b) in enumerate(self.lstm):
            gates = ops.linear(self.xh[layer], w)
            nxt = self.xh[layer + 1][:, :d] if layer + 1 < len(self.lstm) else self.top
            speech_ops.lstm_cell(gates, b, self.cell[layer], self.xh[layer][:, d:], nxt, self.state)
        pred = ops.linear(self.top, self.w_pred)
        speech_ops.tdt_joint_in(self.enc, pred, self.b_pred, self.state, self.jh)
        logits = ops.linear(self.jh, self.w_head)
        speech_ops.tdt_select(logits, self.b_head, self.durations, self.state, self.traj, spec.vocab, spec.blank, spec.eos)

    def _capture(self) -> None:
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        saved = self.state.clone()
        with torch.cuda.stream(side):
            self.step()                                  # warm-up: workspaces and kernel attributes exist before capture
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
        self._graph = g
        self.state.copy_(saved)

    def _run_until_done(self, limit: int) -> tuple[list[list[int]], int, int]:
        steps = reads = 0
        while True:
            if self.use_graph:
                for _ in range(CHECK_EVERY):
                    self._graph.replay()
                self.graph_replays += CHECK_EVERY
                steps += CHECK_EVERY
            else:
                self.step()
                steps += 1
            st = self.state.tolist()
            reads += 1
            for b, row in enumerate(st):
                if row[TS_ERROR]:
                    raise RuntimeError(f"decode capacity exceeded: utterance {b}, capacity={row[TS_CAP]} frame={row[TS_FRAME]}")
            if all(row[TS_DONE] for row in st):
                return st, steps, reads
            if steps > limit + CHECK_EVERY:
                raise RuntimeError("decode did not finish within its capacity")

    # -- streaming: rows arrive in pieces, the device state carries on (one utterance row per lane) ----------
    def begin_stream(self, lanes: int = 1) -> None:
        """Opens ``lanes`` independent streams (batch rows 0 .. lanes - 1): separate prediction-network states, encoder
        row buffers and trajectories, stepping together whenever more than one has rows to decode."""
        if not (0 < lanes <= self.max_batch):
            raise ValueError(f"streams take 1..{self.max_batch} lanes")
        self.reset([1] * lanes)
        st = self.state.tolist()
        for lane in range(lanes):
            st[lane][TS_VALID], st[lane][TS_CAP], st[lane][TS_DONE] = 0, self.traj[0].shape[1], 1
        self.state.copy_(torch.tensor(st, dtype=torch.int32))
        self._lanes = lanes
        self._rows = [0] * lanes
        self._taken = [1] * lanes                        # trajectory entries already handed out (the initial blank)

    def extend(self, projected: torch.Tensor) -> TdtTrajectory:
        """Appends projected encoder rows and decodes as far as they reach; returns the new trajectory entries."""
        return self.extend_lanes({0: projected})[0]

    def extend_lanes(self, projected: dict[int, torch.Tensor]) -> dict[int, TdtTrajectory]:
        """Appends projected encoder rows to the named lanes and decodes them together as far as their rows reach; the
        other lanes stay parked with their state untouched. Returns the new trajectory entries per named lane (frames
        count the lane's own rows)."""
        for lane, rows in projected.items():
            if not (0 <= lane < self._lanes):
                raise ValueError(f"lane {lane} outside the {self._lanes} open streams")
            if self._rows[lane] + rows.shape[0] > self.max_rows:
                raise ValueError(f"stream longer than {self.max_rows} encoder rows")
        if self.use_graph and self._graph is None:
            self._capture()                              # the capture leaves the state as it found it
        for lane, rows in projected.items():
            n = rows.shape[0]
            if n:
                self.enc[lane, self._rows[lane]: self._rows[lane] + n].copy_(rows)
                self._rows[lane] += n
        st = self.state.tolist()
        for lane in range(self._lanes):
            s0 = st[lane]
            if lane not in projected:
                s0[TS_DONE] = 1
                continue
            stopped_on_eos = s0[TS_DONE] and s0[TS_COUNT] > 1 and int(self.traj[0][lane, s0[TS_COUNT] - 1]) == self.spec.eos
            s0[TS_VALID] = self._rows[lane]
            s0[TS_DONE] = int(stopped_on_eos or s0[TS_FRAME] >= self._rows[lane])
        self.state.copy_(torch.tensor(st, dtype=torch.int32))
        steps = reads = 0
        if not all(st[lane][TS_DONE] for lane in range(self._lanes)):
            st, steps, reads = self._run_until_done(self.traj[0].shape[1])
        out = {}
        for lane in projected:
            lo, hi = self._taken[lane], st[lane][TS_COUNT]
            self._taken[lane] = hi
            tok, dur, frm = (t[lane, lo:hi].tolist() for t in self.traj)
            out[lane] = TdtTrajectory(tokens=tok, durations=dur, frames=frm, capacity=self.traj[0].shape[1], steps=steps, state_reads=reads)
        return out

    def decode_batch(self, projected: list[torch.Tensor], valid_rows: list[int]) -> list[TdtTrajectory]:
        """Greedy decode of up to ``max_batch`` utterances at once from their projected encoder rows
        ([rows, decoder_hidden] each); all of them step together until the last one is done."""
        if not (0 < len(projected) <= self.max_batch) or len(projected) != len(valid_rows):
            raise ValueError(f"decode takes 1..{self.max_batch} utterances")
        for b, (p, v) in enumerate(zip(projected, valid_rows)):
            if not (0 < v <= p.shape[0] <= self.max_rows):
                raise ValueError("decode valid encoder rows outside the projected extent")
            self.enc[b, : p.shape[0]].copy_(p)
        if self.use_graph and self._graph is None:
            self.reset(valid_rows)
            self._capture()
        caps = self.reset(valid_rows)
        st, steps, reads = self._run_until_done(max(caps))
        out = []
        for b, cap in enumerate(caps):
            n = st[b][TS_COUNT]
            tok, dur, frm = (t[b, :n].tolist() for t in self.traj)
            out.append(TdtTrajectory(tokens=tok, durations=dur, frames=frm, capacity=cap, steps=steps, state_reads=reads))
        return out

    def decode(self, projected: torch.Tensor, valid_rows: int) -> TdtTrajectory:
        """Greedy decode of one utterance from its projected encoder rows [rows, decoder_hidden]."""
        return self.decode_batch([projected], [valid_rows])[0]


class ParakeetModel:
    """Log-mel front end + encoder + TDT decoder of one checkpoint (or of seeded random weights)."""

    def __init__(self, spec: ParakeetSpec, tensors: dict[str, torch.Tensor], device: torch.device | str = "cpu",
                 tokenizer=None, max_rows: int = 0, max_batch: int = 8):
        spec.check()
        self.spec, self.device, self.tokenizer = spec, torch.device(device), tokenizer
        self.mel = LogMel(spec.mel, self.device)
        self.encoder = ConformerEncoder(spec.encoder, tensors, self.device)
        self.decoder = TdtDecoder(spec, tensors, self.device, max_rows, max_batch)

    @classmethod
    def random(cls, spec: ParakeetSpec, device: torch.device | str = "cpu", seed: int = 0, **kw) -> "ParakeetModel":
        return cls(spec, random_tensors(spec.expected_tensors(), seed), device, **kw)

    @classmethod
    def load(cls, directory: str | Path, device: torch.device | str = "cpu", **kw) -> "ParakeetModel":
        from ..loaders.safetensors_io import MappedCheckpoint
        from ..loaders.tokenizer import load_tokenizer
        spec = ParakeetSpec.read(directory)
        ckpt = MappedCheckpoint(directory)
        table = {n: (ckpt.info(n).dtype, tuple(ckpt.info(n).shape)) for n in ckpt.names()}
        spec.validate(table)
        tensors = {n: ckpt.tensor(n) for n in ckpt.names()}
        return cls(spec, tensors, device, tokenizer=load_tokenizer(directory), **kw)

    def encode(self, waveforms: list[torch.Tensor]) -> tuple[torch.Tensor, list[int]]:
        feat, valid = self.mel.extract(waveforms, normalize=self.spec.mel.normalize)
        return self.encoder.encode(feat, valid.tolist())

    def decode(self, waveforms: list[torch.Tensor]) -> list[TdtTrajectory]:
        encoded, rows = self.encode(waveforms)
        batch, t, h = encoded.shape
        proj = self.decoder.project(encoded.reshape(batch * t, h)).reshape(batch, t, -1)
        out = []
        nb = self.decoder.max_batch
        for lo in range(0, batch, nb):                    # the decoder steps up to max_batch utterances together
            hi = min(batch, lo + nb)
            out += self.decoder.decode_batch([proj[b] for b in range(lo, hi)], rows[lo:hi])
        return out

    def transcription(self, traj: TdtTrajectory) -> Transcription:
        tk = self.tokenizer
        if tk is None:
            raise RuntimeError("no tokenizer: the model directory holds no tokenizer.json")
        pieces = {}
        inner = getattr(tk, "tk", None)
        if inner is not None:
            pieces = {i: p for p, i in inner.get_vocab(False).items()}
        return tdt_cues(traj.tokens, traj.durations, self.spec.blank, lambda ids: tk.decode(list(ids)),
                        lambda t: pieces.get(t, "").startswith(WORD_MARKER), self.spec.frame_seconds, self.spec.pad)

    def transcribe(self, waveforms: list[torch.Tensor]) -> list[Transcription]:
        return [self.transcription(t) for t in self.decode(waveforms)]


@dataclass(frozen=True)
class ParakeetCtcSpec:
    """FastConformer encoder with a CTC head (``ParakeetForCTC``: ``ctc_head`` is a kernel-1 convolution)."""
    encoder: ConformerSpec = field(default_factory=ConformerSpec)
    vocab: int = 1025                  # tokens including the blank
    blank: int = 1024
    pad: int = 2
    mel: LogMelConfig = field(default_factory=lambda: LogMelConfig(mel_bins=80))

    @property
    def frame_seconds(self) -> float:
        return 8 * self.mel.hop_length / self.mel.sampling_rate

    def expected_tensors(self) -> dict[str, tuple[str, tuple[int, ...]]]:
        out = self.encoder.expected_tensors()
        out["ctc_head.weight"] = ("F32", (self.vocab, self.encoder.hidden, 1))
        out["ctc_head.bias"] = ("F32", (self.vocab,))
        return out

    @classmethod
    def read(cls, directory: str | Path) -> "ParakeetCtcSpec":
        d = Path(directory)
        root = json.loads((d / "config.json").read_text())
        if root.get("architectures") != ["ParakeetForCTC"]:
            raise ValueError("not a Parakeet CTC configuration")
        proc = json.loads((d / "processor_config.json").read_text())
        tdt_like = dict(root, architectures=["ParakeetForTDT"], model_type="parakeet_tdt", hidden_act="relu", durations=[0],
                        decoder_hidden_size=8, num_decoder_layers=1, max_symbols_per_step=1,
                        blank_token_id=root.get("blank_token_id", root.get("pad_token_id", root["vocab_size"] - 1)))
        base = ParakeetSpec.from_json(tdt_like, proc, {})
        return cls(encoder=base.encoder, vocab=base.vocab, blank=base.blank, pad=base.pad, mel=base.mel)


class ParakeetCtcModel:
    """Log-mel front end + encoder + CTC head; greedy decoding merges repeats and drops blanks."""

    def __init__(self, spec: ParakeetCtcSpec, tensors: dict[str, torch.Tensor], device: torch.device | str = "cpu", tokenizer=None):
        spec.encoder.check()
        self.spec, self.device, self.tokenizer = spec, torch.device(device), tokenizer
        self.mel = LogMel(spec.mel, self.device)
        self.encoder = ConformerEncoder(spec.encoder, tensors, self.device)
        n_pad = (spec.vocab + 15) // 16 * 16
        head = torch.zeros(n_pad, spec.encoder.hidden)
        head[: spec.vocab] = tensors["ctc_head.weight"].float().reshape(spec.vocab, spec.encoder.hidden)
        bias = torch.full((n_pad,), -1.0e4)
        bias[: spec.vocab] = tensors["ctc_head.bias"].float()
        self.head = (head.to(BF16).contiguous().to(self.device), bias.to(BF16).contiguous().to(self.device))

    @classmethod
    def random(cls, spec: ParakeetCtcSpec, device: torch.device | str = "cpu", seed: int = 0, **kw) -> "ParakeetCtcModel":
        return cls(spec, random_tensors(spec.expected_tensors(), seed), device, **kw)

    @classmethod
    def load(cls, directory: str | Path, device: torch.device | str = "cpu") -> "ParakeetCtcModel":
        from ..loaders.safetensors_io import MappedCheckpoint
        from ..loaders.tokenizer import load_tokenizer
        spec = ParakeetCtcSpec.read(directory)
        ckpt = MappedCheckpoint(directory)
        expected = spec.expected_tensors()
        for n in expected:
            if not ckpt.has(n):
                raise ValueError(f"Parakeet tensor missing: {n}")
        return cls(spec, {n: ckpt.tensor(n) for n in expected}, device, tokenizer=load_tokenizer(directory))

    def decode(self, waveforms: list[torch.Tensor]) -> list[tuple[list[int], list[int], list[int]]]:
        """Per utterance: (tokens, first frame of each token, frames each token was held)."""
        feat, valid = self.mel.extract(waveforms, normalize=True)
        encoded, rows = self.encoder.encode(feat, valid.tolist())
        b, t, h = encoded.shape
        logits = vision_ops.linear_bias_act(encoded.reshape(b * t, h), self.head[0], self.head[1], "none")
        ids = ops.argmax_rows(logits).reshape(b, t).cpu()
        return [speech_ops.ctc_collapse(ids[i], rows[i], self.spec.blank) for i in range(b)]

    def transcribe(self, waveforms: list[torch.Tensor]) -> list[Transcription]:
        tk = self.tokenizer
        if tk is None:
            raise RuntimeError("no tokenizer: the model directory holds no tokenizer.json")
        inner = getattr(tk, "tk", None)
        pieces = {i: p for p, i in inner.get_vocab(False).items()} if inner is not None else {}
        out = []
        for tokens, starts, runs in self.decode(waveforms):
            # the same cue rules as the transducer: blanks carry the gaps between emissions
            traj_t, traj_d, frame = [], [], 0
            for tok, f, r in zip(tokens, starts, runs):
                if f > frame:
                    traj_t.append(self.spec.blank)
                    traj_d.append(f - frame)
                traj_t.append(tok)
                traj_d.append(r)
                frame = f + r
            out.append(tdt_cues(traj_t, traj_d, self.spec.blank, lambda ids: tk.decode([i for i in ids if i != self.spec.blank]),
                                lambda t: pieces.get(t, "").startswith(WORD_MARKER), self.spec.frame_seconds, self.spec.pad))
        return out


def load_model(directory: str | Path, device: torch.device | str = "cpu"):
    """The recognition model a checkpoint directory names in ``config.json``."""
    arch = json.loads((Path(directory) / "config.json").read_text()).get("architectures", [None])[0]
    if arch in ("ParakeetForTDT", "Nemotron3_5AsrForRNNT"):
        return ParakeetModel.load(directory, device)
    if arch == "ParakeetForCTC":
        return ParakeetCtcModel.load(directory, device)
    if arch == "CanaryForConditionalGeneration":
        from .canary import CanaryModel
        return CanaryModel.load(directory, device)
    raise ValueError(f"unsupported transcription architecture {arch}")


def transcribe(directory: str | Path, waveform: torch.Tensor, device: torch.device | str = "cpu") -> Transcription:
    """Loads the checkpoint in ``directory`` and transcribes one 16 kHz mono waveform."""
    return load_model(directory, device).transcribe([waveform])[0]


def streaming_tiny() -> ParakeetSpec:
    """A small cache-aware streaming shape: chunks of 4 encoder rows seeing 3 earlier chunks, causal convolutions and
    stem pads, layer-norm convolution module, plain RNN-T decoder, un-normalised features."""
    enc = ConformerSpec(layers=2, hidden=128, heads=2, intermediate=256, conv_kernel=9, mel_bins=32, sub_channels=32,
                        conv_batch_norm=False, pad_left=2, pad_right=1, max_position=512, chunk_size=4, left_chunks=3,
                        causal_conv=True, conv_names=("subsampling.conv_in", "subsampling.layers.0.depthwise_conv",
                                                      "subsampling.layers.1.depthwise_conv"),
                        pointwise_names=("subsampling.layers.0.pointwise_conv", "subsampling.layers.1.pointwise_conv"))
    return ParakeetSpec(encoder=enc, decoder_hidden=64, decoder_layers=1, vocab=41, blank=40, max_symbols=10, eos=3, durations=(),
                        mel=LogMelConfig(mel_bins=32, normalize=False))


class StreamingRecognizer:
    """Incremental recognition with a streaming-capable model: audio in pieces, tokens out as soon as the encoder rows
    they depend on are complete (front end, encoder stream and transducer state all carry on between calls)."""

    def __init__(self, model: ParakeetModel):
        from ..models.conformer import ConformerStream
        from .audio import StreamingLogMel
        if model.spec.mel.normalize:
            raise ValueError("streaming needs un-normalised features (per-utterance statistics are not causal)")
        self.model = model
        self.front = StreamingLogMel(model.mel)
        self.stream = ConformerStream(model.encoder)
        model.decoder.begin_stream()
        self.tokens: list[int] = [model.spec.blank]
        self.durations: list[int] = [0]
        self.frames: list[int] = [0]

    def push(self, samples: torch.Tensor, last: bool = False) -> list[int]:
        """Feeds samples; returns the non-blank tokens recognised by this call."""
        frames = self.front.push(samples, last)
        rows = self.stream.push(frames, last)
        new = self.model.decoder.extend(self.model.decoder.project(rows) if rows.shape[0] else rows[:, : self.model.spec.decoder_hidden])
        self.tokens += new.tokens
        self.durations += new.durations
        self.frames += new.frames
        return [t for t in new.tokens if t != self.model.spec.blank]

    def trajectory(self) -> TdtTrajectory:
        return TdtTrajectory(self.tokens, self.durations, self.frames, self.model.decoder.traj[0].numel())

    def transcription(self) -> Transcription:
        return self.model.transcription(self.trajectory())


def nemotron_tiny() -> ParakeetSpec:
    """The streaming test shape with a prompt adapter: 6 prompt ids, 96-wide adapter, "auto" = id 4."""
    from dataclasses import replace
    return replace(streaming_tiny(), eos=-1, prompts=6, prompt_intermediate=96, default_prompt=4,
                   prompt_dictionary=(("auto", 4), ("de", 2), ("en", 1)))
