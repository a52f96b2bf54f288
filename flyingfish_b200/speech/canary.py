"""Canary-style speech recognition / translation: FastConformer encoder + attention encoder-decoder (a pre-norm
transformer decoder with causal self-attention and cross-attention over the encoder rows), prompted with task tokens.

Configuration, tensor contract and prompt follow the published ``CanaryForConditionalGeneration`` layout
(src/canary.rs:16-440 of the reference); the decoder program follows src/backend/cuda/engine_canary.rs:817-916. Here the
decoder runs on the paged-attention kernels of the text engine: the self-attention keys of every utterance live in a
small paged cache written by the rotary kernel at position 0 (the identity rotation), the projected encoder rows of a
layer are written once into a second paged cache that every later step reads through the same decode-attention kernel,
all utterances of a batch step together, and the host looks at the generated tokens once per ``CHECK_EVERY`` steps."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path

import torch

from .. import ops
from ..models.conformer import ConformerEncoder, ConformerSpec, random_tensors
from ..ops import speech_ops, vision_ops
from .audio import LogMel, LogMelConfig
from .transcript import Transcription

BF16 = torch.bfloat16
CHECK_EVERY = 8
LANGUAGES = ("bg", "hr", "cs", "da", "nl", "en", "et", "fi", "fr", "de", "el", "hu", "it", "lv", "lt", "mt", "pl", "pt", "ro",
             "sk", "sl", "es", "sv", "ru", "uk")


def _canary_encoder() -> ConformerSpec:
    return ConformerSpec(attention_bias=True, convolution_bias=True, prefix="model.encoder")


@dataclass(frozen=True)
class CanarySpec:
    encoder: ConformerSpec = field(default_factory=_canary_encoder)
    vocab: int = 16384
    decoder_layers: int = 8
    intermediate: int = 4096
    max_positions: int = 1024
    bos: int = 4
    eos: int = 3
    pad: int = 2
    decoder_start: int = 7
    mel: LogMelConfig = field(default_factory=LogMelConfig)

    @property
    def hidden(self) -> int:
        return self.encoder.hidden

    @property
    def heads(self) -> int:
        return self.hidden // 128

    def check(self) -> None:
        self.encoder.check()
        if self.hidden % 128 or self.max_positions % 64 or self.decoder_layers < 1:
            raise ValueError("the decoder runs 128-wide heads and 64-token cache blocks")

    @classmethod
    def from_json(cls, root: dict, processor: dict, generation: dict) -> "CanarySpec":
        if root.get("model_type") != "canary" or root.get("architectures") != ["CanaryForConditionalGeneration"]:
            raise ValueError("not a Canary configuration")
        if not root.get("tie_word_embeddings", True):
            raise ValueError("untied output projection")
        enc, dec = root.get("encoder_config"), root.get("decoder_config")
        if not isinstance(enc, dict) or not isinstance(dec, dict) or dec.get("model_type") != "canary_decoder":
            raise ValueError("encoder_config / decoder_config missing")
        if dec.get("hidden_act") != "relu" or not dec.get("attention_bias", True) or int(dec.get("head_dim", 128)) != 128:
            raise ValueError("unsupported decoder setting")
        if int(dec["hidden_size"]) != int(enc["hidden_size"]) or int(dec["num_attention_heads"]) * 128 != int(dec["hidden_size"]):
            raise ValueError("decoder width differs from the encoder")
        feats = processor.get("feature_extractor")
        if not isinstance(feats, dict):
            raise ValueError("feature_extractor missing")
        mel = LogMelConfig(sampling_rate=int(feats["sampling_rate"]), n_fft=int(feats["n_fft"]), win_length=int(feats["win_length"]),
                           hop_length=int(feats["hop_length"]), mel_bins=int(feats["feature_size"]), preemphasis=float(feats["preemphasis"]))
        encoder = ConformerSpec(layers=int(enc["num_hidden_layers"]), hidden=int(enc["hidden_size"]), heads=int(enc["num_attention_heads"]),
                                intermediate=int(enc["intermediate_size"]), conv_kernel=int(enc["conv_kernel_size"]),
                                mel_bins=int(enc["num_mel_bins"]), sub_channels=int(enc["subsampling_conv_channels"]),
                                attention_bias=bool(enc["attention_bias"]), convolution_bias=bool(enc["convolution_bias"]),
                                max_position=int(enc["max_position_embeddings"]), prefix="model.encoder")
        spec = cls(encoder=encoder, vocab=int(root["vocab_size"]), decoder_layers=int(dec["num_hidden_layers"]),
                   intermediate=int(dec["intermediate_size"]), max_positions=int(dec["max_position_embeddings"]),
                   bos=int(root["bos_token_id"]), eos=int(root["eos_token_id"]), pad=int(root["pad_token_id"]),
                   decoder_start=int(generation.get("decoder_start_token_id", root.get("decoder_start_token_id", 7))), mel=mel)
        spec.check()
        return spec

    @classmethod
    def read(cls, directory: str | Path) -> "CanarySpec":
        d = Path(directory)
        load = lambda n: json.loads((d / n).read_text())
        return cls.from_json(load("config.json"), load("processor_config.json"), load("generation_config.json"))

    def to_json(self) -> tuple[dict, dict, dict]:
        e, m = self.encoder, self.mel
        root = {"architectures": ["CanaryForConditionalGeneration"], "model_type": "canary", "dtype": "float32",
                "is_encoder_decoder": True, "tie_word_embeddings": True, "bos_token_id": self.bos, "eos_token_id": self.eos,
                "pad_token_id": self.pad, "decoder_start_token_id": self.decoder_start, "use_cache": True, "vocab_size": self.vocab,
                "encoder_config": {"model_type": "parakeet_encoder", "hidden_act": "silu", "scale_input": False,
                                   "attention_bias": e.attention_bias, "convolution_bias": e.convolution_bias,
                                   "conv_kernel_size": e.conv_kernel, "hidden_size": e.hidden, "intermediate_size": e.intermediate,
                                   "max_position_embeddings": e.max_position, "num_attention_heads": e.heads,
                                   "num_key_value_heads": e.heads, "num_hidden_layers": e.layers, "num_mel_bins": e.mel_bins,
                                   "subsampling_conv_channels": e.sub_channels, "subsampling_conv_kernel_size": 3,
                                   "subsampling_conv_stride": 2, "subsampling_factor": 8},
                "decoder_config": {"model_type": "canary_decoder", "attention_bias": True, "hidden_act": "relu", "head_dim": 128,
                                   "hidden_size": self.hidden, "intermediate_size": self.intermediate,
                                   "max_position_embeddings": self.max_positions, "num_attention_heads": self.heads,
                                   "num_key_value_heads": self.heads, "num_hidden_layers": self.decoder_layers,
                                   "vocab_size": self.vocab, "bos_token_id": self.bos, "eos_token_id": self.eos,
                                   "pad_token_id": self.pad, "use_cache": True}}
        processor = {"processor_class": "CanaryProcessor",
                     "feature_extractor": {"feature_extractor_type": "ParakeetFeatureExtractor", "feature_size": m.mel_bins,
                                           "hop_length": m.hop_length, "n_fft": m.n_fft, "padding_side": "right", "padding_value": 0.0,
                                           "preemphasis": m.preemphasis, "return_attention_mask": True,
                                           "sampling_rate": m.sampling_rate, "win_length": m.win_length}}
        generation = {"bos_token_id": self.bos, "decoder_start_token_id": self.decoder_start, "eos_token_id": self.eos,
                      "pad_token_id": self.pad, "use_cache": True}
        return root, processor, generation

    def expected_tensors(self) -> dict[str, tuple[str, tuple[int, ...]]]:
        out = self.encoder.expected_tensors()
        h, v, f = self.hidden, self.vocab, self.intermediate

        def wb(name: str, w: tuple[int, ...], b: tuple[int, ...]) -> None:
            out[f"{name}.weight"] = ("F32", w)
            out[f"{name}.bias"] = ("F32", b)

        out["model.decoder.embed_tokens.weight"] = ("F32", (v, h))
        wb("model.decoder.embedding_layernorm", (h,), (h,))
        wb("model.decoder.norm", (h,), (h,))
        wb("proj_out", (v, h), (v,))
        for layer in range(self.decoder_layers):
            p = f"model.decoder.layers.{layer}"
            for att in ("self_attn", "encoder_attn"):
                for proj in ("q_proj", "k_proj", "v_proj", "o_proj"):
                    wb(f"{p}.{att}.{proj}", (h, h), (h,))
            for norm in ("input_layernorm", "post_attention_layernorm", "final_layernorm"):
                wb(f"{p}.{norm}", (h,), (h,))
            wb(f"{p}.mlp.fc1", (f, h), (f,))
            wb(f"{p}.mlp.fc2", (h, f), (h,))
        return out


def canary_tiny() -> CanarySpec:
    enc = ConformerSpec(layers=2, hidden=256, heads=2, intermediate=256, conv_kernel=9, mel_bins=32, sub_channels=32,
                        attention_bias=True, convolution_bias=True, max_position=512, prefix="model.encoder")
    return CanarySpec(encoder=enc, vocab=96, decoder_layers=2, intermediate=384, max_positions=128, mel=LogMelConfig(mel_bins=32))


def sinusoidal_rows(length: int, channels: int) -> torch.Tensor:
    """[length, channels] decoder position rows: sin in the first half, cos in the second, time scales from 1 to
    ``10000 ** ((channels - 2) / channels)``, all divided by ``sqrt(channels)``."""
    half = channels // 2
    max_timescale = 10000.0 ** ((channels - 2.0) / channels)
    increment = math.log(max_timescale) / (half - 1.0)
    inv = torch.exp(-increment * torch.arange(half, dtype=torch.float32))
    phase = torch.arange(length, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([torch.sin(phase), torch.cos(phase)], dim=1) / math.sqrt(channels)


def canary_prompt(encode, source_language: str, target_language: str, punctuation: bool) -> list[int]:
    """The nine task tokens that start every decode; ``encode`` maps one special-token string to its ids."""
    for lang in (source_language, target_language):
        if lang not in LANGUAGES:
            raise ValueError(f"unsupported Canary language {lang}; published set: {','.join(LANGUAGES)}")
    tokens = []
    for text in ("<|startofcontext|>", "<|startoftranscript|>", "<|emo:undefined|>", f"<|{source_language}|>", f"<|{target_language}|>",
                 "<|pnc|>" if punctuation else "<|nopnc|>", "<|noitn|>", "<|notimestamp|>", "<|nodiarize|>"):
        ids = list(encode(text))
        if len(ids) != 1:
            raise ValueError(f"Canary prompt token {text} is not atomic")
        tokens += ids
    return tokens


class CanaryDecoder:
    def __init__(self, spec: CanarySpec, tensors: dict[str, torch.Tensor], device: torch.device | str):
        self.spec, self.device = spec, torch.device(device)
        dev, h = self.device, spec.hidden

        def w16(t: torch.Tensor) -> torch.Tensor:
            return t.float().to(BF16).contiguous().to(dev)

        def f32(name: str) -> torch.Tensor:
            return tensors[name].float().contiguous().to(dev)

        self.embed = w16(tensors["model.decoder.embed_tokens.weight"])
        self.positions = w16(sinusoidal_rows(spec.max_positions, h))
        self.embed_norm = (f32("model.decoder.embedding_layernorm.weight"), f32("model.decoder.embedding_layernorm.bias"))
        self.norm = (f32("model.decoder.norm.weight"), f32("model.decoder.norm.bias"))
        n_pad = (spec.vocab + 15) // 16 * 16
        head = torch.zeros(n_pad, h)
        head[: spec.vocab] = tensors["proj_out.weight"].float()
        hb = torch.full((n_pad,), -1.0e4)
        hb[: spec.vocab] = tensors["proj_out.bias"].float()
        self.head = (w16(head), w16(hb))
        self.layers = []
        for i in range(spec.decoder_layers):
            p = f"model.decoder.layers.{i}"
            cat = lambda att, names, kind: torch.cat([tensors[f"{p}.{att}.{n}_proj.{kind}"].float() for n in names], dim=0)
            self.layers.append(dict(
                ln_in=(f32(f"{p}.input_layernorm.weight"), f32(f"{p}.input_layernorm.bias")),
                wqkv=w16(cat("self_attn", "qkv", "weight")), bqkv=w16(cat("self_attn", "qkv", "bias")),
                wo=w16(tensors[f"{p}.self_attn.o_proj.weight"]), bo=f32(f"{p}.self_attn.o_proj.bias"),
                ln_post=(f32(f"{p}.post_attention_layernorm.weight"), f32(f"{p}.post_attention_layernorm.bias")),
                xq=w16(tensors[f"{p}.encoder_attn.q_proj.weight"]), xqb=w16(tensors[f"{p}.encoder_attn.q_proj.bias"]),
                xkv=w16(cat("encoder_attn", "kv", "weight")), xkvb=w16(cat("encoder_attn", "kv", "bias")),
                xo=w16(tensors[f"{p}.encoder_attn.o_proj.weight"]), xob=f32(f"{p}.encoder_attn.o_proj.bias"),
                ln_final=(f32(f"{p}.final_layernorm.weight"), f32(f"{p}.final_layernorm.bias")),
                fc1=w16(tensors[f"{p}.mlp.fc1.weight"]), fc1b=w16(tensors[f"{p}.mlp.fc1.bias"]),
                fc2=w16(tensors[f"{p}.mlp.fc2.weight"]), fc2b=f32(f"{p}.mlp.fc2.bias")))

    # --------------------------------------------------------------------------------------------
    def open(self, encoded: torch.Tensor, rows: list[int]) -> dict:
        """Per-batch decode state: empty self-attention caches and, per layer, the projected encoder rows written into a
        paged cross-attention cache. ``encoded``: [batch, T, hidden] BF16."""
        spec, dev = self.spec, self.device
        batch, t, h = encoded.shape
        heads = spec.heads
        sb, xb = spec.max_positions // 64, (t + 63) // 64
        st = dict(batch=batch, sb=sb, xb=xb, filled=0,
                  self_bt=torch.arange(batch * sb, dtype=torch.int32, device=dev).reshape(batch, sb).contiguous(),
                  x_bt=torch.arange(batch * xb, dtype=torch.int32, device=dev).reshape(batch, xb).contiguous(),
                  x_len=torch.tensor(rows, dtype=torch.int32, device=dev), self_k=[], self_v=[], x_k=[], x_v=[])
        flat = encoded.reshape(batch * t, h)
        pad = xb * 64 - t
        for L in self.layers:
            st["self_k"].append(torch.zeros(batch * sb, heads, 64, 128, dtype=encoded.dtype, device=dev))
            st["self_v"].append(torch.zeros(batch * sb, heads, 64, 128, dtype=encoded.dtype, device=dev))
            kv = vision_ops.linear_bias_act(flat, L["xkv"], L["xkvb"], "none").reshape(batch, t, 2, heads, 128)
            if pad:
                kv = torch.nn.functional.pad(kv, (0, 0, 0, 0, 0, 0, 0, pad))
            paged = kv.reshape(batch, xb, 64, 2, heads, 128).permute(3, 0, 1, 4, 2, 5).reshape(2, batch * xb, heads, 64, 128)
            st["x_k"].append(paged[0].contiguous())
            st["x_v"].append(paged[1].contiguous())
        return st

    def forward(self, st: dict, ids: torch.Tensor, n_new: int) -> torch.Tensor:
        """``n_new`` new tokens per utterance (ids packed utterance-major, int32 on the device) -> logits of each
        utterance's last new row, [batch, padded vocab]."""
        spec, dev = self.spec, self.device
        batch, heads, h = st["batch"], spec.heads, spec.hidden
        p0 = st["filled"]
        if p0 + n_new > spec.max_positions:
            raise ValueError(f"decoder position {spec.max_positions}")
        rows = batch * n_new
        pos = torch.arange(p0, p0 + n_new, device=dev)
        pos_rows = self.positions[pos].repeat(batch, 1)
        slots = (torch.arange(batch, device=dev)[:, None] * spec.max_positions + pos[None, :]).reshape(-1).to(torch.int32)
        zero_pos = torch.zeros(rows, dtype=torch.int32, device=dev)
        ctx = torch.full((batch,), p0 + n_new, dtype=torch.int32, device=dev)
        q_lens = torch.full((batch,), n_new, dtype=torch.int32, device=dev)
        q_start = (torch.arange(batch, device=dev) * n_new).to(torch.int32)
        scale = 1.0 / math.sqrt(128.0)
        hid = ops.embed(ids, self.embed)
        hid = speech_ops.scale_add_layernorm(hid, pos_rows, None, 1.0, *self.embed_norm)
        x = speech_ops.scale_add_layernorm(hid, None, None, 0.0, *self.layers[0]["ln_in"])
        for i, L in enumerate(self.layers):
            qkv = vision_ops.linear_bias_act(x, L["wqkv"], L["bqkv"], "none")
            # rotation by position 0 is the identity: the kernel only files K and V into the paged cache
            ops.rope_kv_paged(qkv, zero_pos, slots, st["self_k"][i], st["self_v"][i], heads, heads, 128, 10000.0)
            if n_new == 1:
                a = ops.attn_decode(qkv, st["self_k"][i], st["self_v"][i], st["self_bt"], ctx, heads, heads, 128, scale)
            else:
                a = ops.attn_prefill(qkv, st["self_k"][i], st["self_v"][i], st["self_bt"], q_start, q_lens, ctx, n_new, heads,
                                     heads, 128, scale)
            x = speech_ops.scale_add_layernorm(hid, ops.linear(a, L["wo"]), L["bo"], 1.0, *L["ln_post"])
            q = vision_ops.linear_bias_act(x, L["xq"], L["xqb"], "none")
            if n_new == 1:
                a = ops.attn_decode(q, st["x_k"][i], st["x_v"][i], st["x_bt"], st["x_len"], heads, heads, 128, scale)
            else:
                a = ops.attn_prefill(q, st["x_k"][i], st["x_v"][i], st["x_bt"], q_start, q_lens, st["x_len"], n_new, heads, heads,
                                     128, scale, window=-1)
            x = speech_ops.scale_add_layernorm(hid, ops.linear(a, L["xo"]), L["xob"], 1.0, *L["ln_final"])
            u = vision_ops.linear_bias_act(x, L["fc1"], L["fc1b"], "relu")
            nxt = self.layers[i + 1]["ln_in"] if i + 1 < len(self.layers) else self.norm
            x = speech_ops.scale_add_layernorm(hid, ops.linear(u, L["fc2"]), L["fc2b"], 1.0, *nxt)
        st["filled"] = p0 + n_new
        last = x.reshape(batch, n_new, h)[:, -1].contiguous() if n_new > 1 else x
        return vision_ops.linear_bias_act(last, self.head[0], self.head[1], "none")

    def greedy(self, encoded: torch.Tensor, rows: list[int], prompt: list[int], max_new: int | None = None) -> list[list[int]]:
        """Greedy decode of every utterance from the same prompt; returns prompt + generated ids up to and including
        the end-of-sequence token (or the position limit)."""
        spec, dev = self.spec, self.device
        batch = encoded.shape[0]
        if not prompt or len(prompt) >= spec.max_positions or any(not (0 <= t < spec.vocab) for t in prompt):
            raise ValueError("prompt length or token id outside the decoder's range")
        limit = spec.max_positions - len(prompt)
        if max_new is not None:
            limit = min(limit, max_new)
        st = self.open(encoded, rows)
        ids = torch.tensor(prompt * batch, dtype=torch.int32, device=dev)
        out = torch.zeros(limit, batch, dtype=torch.int32, device=dev)
        logits = self.forward(st, ids, len(prompt))
        done_at = [None] * batch
        step = 0
        while step < limit:
            picked = ops.argmax_rows(logits, out=out[step])
            if not picked.is_cuda:
                out[step] = picked
            step += 1
            if step % CHECK_EVERY == 0 or step == limit:
                host = out[:step].cpu()
                for b in range(batch):
                    if done_at[b] is None:
                        hit = (host[:, b] == spec.eos).nonzero()
                        if hit.numel():
                            done_at[b] = int(hit[0]) + 1
                if all(d is not None for d in done_at):
                    break
            if step < limit:
                logits = self.forward(st, out[step - 1], 1)
        host = out[:step].cpu()
        return [list(prompt) + host[: (done_at[b] or step), b].tolist() for b in range(batch)]


class CanaryModel:
    def __init__(self, spec: CanarySpec, tensors: dict[str, torch.Tensor], device: torch.device | str = "cpu", tokenizer=None):
        spec.check()
        self.spec, self.device, self.tokenizer = spec, torch.device(device), tokenizer
        self.mel = LogMel(spec.mel, self.device)
        self.encoder = ConformerEncoder(spec.encoder, tensors, self.device)
        self.decoder = CanaryDecoder(spec, tensors, self.device)

    @classmethod
    def random(cls, spec: CanarySpec, device: torch.device | str = "cpu", seed: int = 0, **kw) -> "CanaryModel":
        t = random_tensors(spec.expected_tensors(), seed)
        t["proj_out.weight"] = t["model.decoder.embed_tokens.weight"].clone()          # tied
        return cls(spec, t, device, **kw)

    @classmethod
    def load(cls, directory: str | Path, device: torch.device | str = "cpu") -> "CanaryModel":
        from ..loaders.safetensors_io import MappedCheckpoint
        from ..loaders.tokenizer import load_tokenizer
        spec = CanarySpec.read(directory)
        ckpt = MappedCheckpoint(directory)
        expected = spec.expected_tensors()
        for n in expected:
            if not ckpt.has(n):
                raise ValueError(f"Canary tensor missing: {n}")
        for n in ckpt.names():
            if n not in expected:
                raise ValueError(f"Canary tensor unexpected: {n}")
        tensors = {n: ckpt.tensor(n) for n in expected}
        if not torch.equal(tensors["proj_out.weight"], tensors["model.decoder.embed_tokens.weight"]):
            raise ValueError("proj_out.weight and model.decoder.embed_tokens.weight differ")
        return cls(spec, tensors, device, tokenizer=load_tokenizer(directory))

    def generate(self, waveforms: list[torch.Tensor], prompt: list[int], max_new: int | None = None) -> list[list[int]]:
        feat, valid = self.mel.extract(waveforms, normalize=True)
        encoded, rows = self.encoder.encode(feat, valid.tolist())
        return self.decoder.greedy(encoded, rows, prompt, max_new)

    def prompt(self, source_language: str = "en", target_language: str = "en", punctuation: bool = True) -> list[int]:
        tk = self.tokenizer
        if tk is None:
            raise RuntimeError("no tokenizer: the model directory holds no tokenizer.json")
        return canary_prompt(lambda text: tk.encode(text), source_language, target_language, punctuation)

    def transcribe(self, waveforms: list[torch.Tensor], source_language: str = "en", target_language: str = "en",
                   punctuation: bool = True) -> list[Transcription]:
        prompt = self.prompt(source_language, target_language, punctuation)
        outs = self.generate(waveforms, prompt)
        res = []
        for w, ids in zip(waveforms, outs):
            text = self.tokenizer.decode(ids[len(prompt):], skip_special_tokens=True)
            res.append(Transcription.whole_clip(text.strip(), w.numel() / float(self.spec.mel.sampling_rate)))
        return res
