"""Streaming RNN-T checkpoints in the NeMo archive layout (``.nemo``: a tar with ``model_config.yaml``, the pickled
``model_weights.ckpt`` and a unigram ``*_tokenizer.vocab``), such as the realtime end-of-utterance models
(src/eou.rs:317-600 of the reference; tensor names src/backend/cuda/engine_eou.rs:40-115).

The archive is mapped onto the same ``ParakeetModel`` / ``StreamingRecognizer`` the other speech models use: the YAML
becomes a ``ParakeetSpec`` with a chunk-wise streaming encoder and an empty duration head, the NeMo tensor names are
translated to the canonical ones, and the end-of-utterance token cuts the token stream into timed utterances."""
from __future__ import annotations

from pathlib import Path

import torch

from ..models.conformer import ConformerSpec
from .audio import LogMelConfig
from .parakeet import ParakeetModel, ParakeetSpec, StreamingRecognizer
from .transcript import TextSegment, Transcription

NEMO_ATTENTION = ("linear_q", "linear_k", "linear_v", "linear_out", "linear_pos", "pos_bias_u", "pos_bias_v")


def spec_from_yaml(text: str) -> ParakeetSpec:
    import yaml
    root = yaml.safe_load(text)
    try:
        pre, enc, dec, joint = root["preprocessor"], root["encoder"], root["decoder"], root["joint"]
        prednet, jointnet = dec["prednet"], joint["jointnet"]
        if str(pre.get("normalize")) != "NA":
            raise ValueError("the streaming front end takes un-normalised features (preprocessor.normalize: NA)")
        if (enc["subsampling"], enc["self_attention_model"], enc["att_context_style"], enc["conv_context_size"], enc["conv_norm_type"]) != \
                ("dw_striding", "rel_pos", "chunked_limited", "causal", "layer_norm") or enc["xscaling"] or enc["use_bias"]:
            raise ValueError("unsupported encoder architecture variant")
        if jointnet["activation"] != "relu" or not dec["blank_as_pad"] or not enc["causal_downsampling"]:
            raise ValueError("unsupported decoder / joint variant")
        if int(enc["subsampling_factor"]) != 8 or int(pre.get("frame_splicing", 1)) != 1:
            raise ValueError("unsupported sub-sampling")
        context = enc["att_context_size"]
        if context and isinstance(context[0], (list, tuple)):
            # several training-time context modes: inference runs the first one, and all share the left context
            if any(len(pair) != 2 or int(pair[0]) != int(context[0][0]) for pair in context):
                raise ValueError("att_context_size modes differ in their left context")
            context = context[0]
        left, right = (int(v) for v in context)
        chunk = right + 1
        if left % chunk:
            raise ValueError(f"left context {left} does not divide by the chunk of {chunk} rows")
        rate = int(pre["sample_rate"])
        mel = LogMelConfig(sampling_rate=rate, n_fft=int(pre["n_fft"]), win_length=int(round(float(pre["window_size"]) * rate)),
                           hop_length=int(round(float(pre["window_stride"]) * rate)), mel_bins=int(pre["features"]), normalize=False)
        hidden = int(enc["d_model"])
        encoder = ConformerSpec(layers=int(enc["n_layers"]), hidden=hidden, heads=int(enc["n_heads"]),
                                intermediate=hidden * int(enc["ff_expansion_factor"]), conv_kernel=int(enc["conv_kernel_size"]),
                                mel_bins=int(enc["feat_in"]), sub_channels=int(enc["subsampling_conv_channels"]),
                                conv_batch_norm=False, pad_left=2, pad_right=1, max_position=int(enc["pos_emb_max_len"]),
                                chunk_size=chunk, left_chunks=left // chunk, causal_conv=True,
                                conv_names=("pre_encode.conv.0", "pre_encode.conv.2", "pre_encode.conv.5"),
                                pointwise_names=("pre_encode.conv.3", "pre_encode.conv.6"), linear_name="pre_encode.out",
                                attention_names=NEMO_ATTENTION, conv_norm_name="batch_norm")
        vocab = int(dec["vocab_size"])
        d = int(prednet["pred_hidden"])
        if int(jointnet["joint_hidden"]) != d or int(joint["num_classes"]) != vocab:
            raise ValueError("joint width differs from the prediction network's")
        spec = ParakeetSpec(encoder=encoder, decoder_hidden=d, decoder_layers=int(prednet["pred_rnn_layers"]), vocab=vocab + 1,
                            blank=vocab, max_symbols=10, eos=-1, durations=(), mel=mel)
    except KeyError as e:
        raise ValueError(f"model_config.yaml lacks {e}") from None
    spec.check()
    return spec


def canonical_tensors(spec: ParakeetSpec, tensors: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """NeMo names -> the names ``ParakeetSpec.expected_tensors`` lists (the encoder keeps its names: the spec carries
    the NeMo spellings)."""
    out = {n: t for n, t in tensors.items() if n.startswith("encoder.")}
    ren = {"decoder.prediction.embed.weight": "decoder.embedding.weight", "joint.pred.weight": "decoder.decoder_projector.weight",
           "joint.pred.bias": "decoder.decoder_projector.bias", "joint.enc.weight": "encoder_projector.weight",
           "joint.enc.bias": "encoder_projector.bias", "joint.joint_net.2.weight": "joint.head.weight",
           "joint.joint_net.2.bias": "joint.head.bias"}
    for layer in range(spec.decoder_layers):
        for kind in ("weight_ih", "weight_hh", "bias_ih", "bias_hh"):
            ren[f"decoder.prediction.dec_rnn.lstm.{kind}_l{layer}"] = f"decoder.lstm.{kind}_l{layer}"
    for src, dst in ren.items():
        if src not in tensors:
            raise ValueError(f"NeMo tensor missing: {src}")
        out[dst] = tensors[src]
    return out


class UnigramVocab:
    """``piece<TAB>score`` vocabulary rows; decoding joins the pieces and turns the word marker into spaces."""

    def __init__(self, text: str):
        self.pieces = []
        for line in text.splitlines():
            if not line:
                continue
            piece, _, score = line.rpartition("\t")
            if not piece or float(score) != float(score):
                raise ValueError("vocabulary row is not piece<TAB>score")
            self.pieces.append(piece)

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        text = "".join(self.pieces[i] for i in ids if 0 <= i < len(self.pieces) and not (skip_special_tokens and self.pieces[i].startswith("<")
                                                                                     and self.pieces[i].endswith(">")))
        return text.replace("▁", " ").strip()

    def piece(self, token: int) -> str:
        return self.pieces[token] if 0 <= token < len(self.pieces) else ""


def load_nemo(path: str | Path, device: torch.device | str = "cpu") -> ParakeetModel:
    from ..loaders.pth import read_nemo, read_nemo_member
    text, weights = read_nemo(path)
    spec = spec_from_yaml(text)
    try:
        tensors = canonical_tensors(spec, {n: weights.tensor(n).clone() for n in weights.records})
    finally:
        weights.close()
    expected = spec.expected_tensors()
    for name, (_, shape) in expected.items():
        if name not in tensors:
            raise ValueError(f"NeMo tensor missing: {name}")
        if tuple(tensors[name].shape) != tuple(shape) and not name.endswith("num_batches_tracked"):
            raise ValueError(f"NeMo tensor shape mismatch: {name} {tuple(tensors[name].shape)} != {tuple(shape)}")
    try:
        vocab = UnigramVocab(read_nemo_member(path, "_tokenizer.vocab").decode("utf-8"))
    except ValueError:
        vocab = None
    return ParakeetModel(spec, tensors, device, tokenizer=vocab)


def split_utterances(tokens: list[int], frames: list[int], durations: list[int], blank: int, eou: int,
                     frame_seconds: float = 0.08) -> list[tuple[list[int], float, float]]:
    """Cuts a trajectory at every end-of-utterance token: (tokens without blanks and the marker, start, end) per
    utterance, an utterance ending at the step its marker was emitted."""
    out, cur, start = [], [], 0.0
    for tok, frm, dur in zip(tokens, frames, durations):
        if tok == blank:
            continue
        if tok == eou:
            end = (frm + dur) * frame_seconds
            out.append((cur, start, end))
            cur, start = [], end
        else:
            cur.append(tok)
    if cur:
        last = (frames[-1] + durations[-1]) * frame_seconds if frames else start
        out.append((cur, start, last))
    return out


def transcribe_nemo(path: str | Path, waveform: torch.Tensor, device: torch.device | str = "cpu", stream: bool = True,
                    piece_seconds: float = 0.32) -> Transcription:
    """Recognition with a ``.nemo`` streaming RNN-T: ``stream`` feeds the audio in pieces and returns one segment per
    utterance (cut at the end-of-utterance token, ``vocab - 2``); otherwise the whole clip is one segment."""
    model = load_nemo(path, device)
    spec = model.spec
    eou = spec.blank - 2
    rec = StreamingRecognizer(model)
    piece = max(1, int(piece_seconds * spec.mel.sampling_rate)) if stream else waveform.numel()
    for at in range(0, waveform.numel(), piece):
        nxt = min(waveform.numel(), at + piece)
        rec.push(waveform[at:nxt], last=nxt == waveform.numel())
    decode = (lambda ids: model.tokenizer.decode(ids)) if model.tokenizer is not None else (lambda ids: " ".join(str(i) for i in ids))
    if not stream:
        ids = [t for t in rec.tokens if t not in (spec.blank, eou)]
        return Transcription.whole_clip(decode(ids), waveform.numel() / float(spec.mel.sampling_rate))
    segs = [TextSegment(s, e, decode(ids)) for ids, s, e in split_utterances(rec.tokens, rec.frames, rec.durations, spec.blank, eou,
                                                                            spec.frame_seconds)]
    return Transcription(text=" ".join(s.text for s in segs), segments=segs, words=[])
