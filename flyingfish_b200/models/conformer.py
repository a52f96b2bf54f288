"""FastConformer speech encoder: an 8x sub-sampling stem of depthwise-separable stride-2 convolutions followed by
conformer layers (half-step feed-forward, relative-position self-attention, convolution module, half-step
feed-forward, output norm).

Published tensor layout (src/parakeet.rs:64-217 of the reference) and the launch sequence it is run with
(src/backend/cuda/engine_parakeet.rs:1058-1147 stem, :1168-1305 layer). Differences of this implementation, all at
load time: activations are channels-last so the pointwise convolutions are plain GEMMs, the stem's final linear has its
columns permuted to that layout instead of repacking activations, Q/K/V are one fused projection, and the convolution
module's batch norm is folded into the depthwise taps so that GLU, mask, depthwise convolution, norm and SiLU are one
kernel (``ops/speech_ops.glu_dwconv1d``)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..ops import speech_ops, vision_ops

BF16 = torch.bfloat16


@dataclass(frozen=True)
class ConformerSpec:
    layers: int = 24
    hidden: int = 1024
    heads: int = 8
    intermediate: int = 4096
    conv_kernel: int = 9
    mel_bins: int = 128
    sub_channels: int = 256
    attention_bias: bool = False
    convolution_bias: bool = False
    conv_batch_norm: bool = True
    pad_left: int = 1
    pad_right: int = 1
    max_position: int = 5000
    att_left: int = -1                 # attention context in frames on each side, -1 = unlimited
    att_right: int = -1
    chunk_size: int = 0                # > 0: chunk-wise context (cache-aware streaming encoders): a query chunk sees
    left_chunks: int = 0               #      ``left_chunks`` earlier chunks, itself and ``right_chunks`` later ones
    right_chunks: int = 0
    causal_conv: bool = False          # the conv module's depthwise taps look back only (left = kernel - 1)
    prefix: str = "encoder"
    conv_names: tuple[str, str, str] = ("subsampling.layers.0", "subsampling.layers.2", "subsampling.layers.5")
    pointwise_names: tuple[str, str] = ("subsampling.layers.3", "subsampling.layers.6")
    linear_name: str = "subsampling.linear"
    # q, k, v, output, position projection, the two position biases; the norm inside the convolution module
    attention_names: tuple[str, ...] = ("q_proj", "k_proj", "v_proj", "o_proj", "relative_k_proj", "bias_u", "bias_v")
    conv_norm_name: str = "norm"

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def conv_left(self) -> int:
        return self.conv_kernel - 1 if self.causal_conv else self.conv_kernel // 2

    @property
    def attention_window(self) -> tuple[int, int, int]:
        """(left, right, chunk) as the attention operator takes them."""
        if self.chunk_size > 0:
            return self.left_chunks, self.right_chunks, self.chunk_size
        return self.att_left, self.att_right, 0

    @property
    def pads(self) -> tuple[int, int]:
        return (self.pad_left, self.pad_right)

    @property
    def sub_freq(self) -> int:
        f = self.mel_bins
        for _ in range(3):
            f = speech_ops.conv_out_len(f, *self.pads)
        return f

    @property
    def linear_in(self) -> int:
        return self.sub_channels * self.sub_freq

    def check(self) -> None:
        if self.hidden % self.heads or self.head_dim not in (64, 128):
            raise ValueError("conformer heads must be 64 or 128 wide")
        if self.conv_kernel < 1 or self.conv_kernel > 32 or self.sub_channels % 8 or self.hidden % 8:
            raise ValueError("unsupported conformer geometry")

    def sub_len(self, n: int) -> int:
        for _ in range(3):
            n = speech_ops.conv_out_len(n, *self.pads)
        return n

    def expected_tensors(self) -> dict[str, tuple[str, tuple[int, ...]]]:
        """Name -> (dtype, shape) of every encoder tensor a published checkpoint holds."""
        h, i, c, k = self.hidden, self.intermediate, self.sub_channels, self.conv_kernel
        out: dict[str, tuple[str, tuple[int, ...]]] = {}
        for layer in range(self.layers):
            p = f"{self.prefix}.layers.{layer}"
            for branch in ("feed_forward1", "feed_forward2"):
                out[f"{p}.{branch}.linear1.weight"] = ("F32", (i, h))
                out[f"{p}.{branch}.linear2.weight"] = ("F32", (h, i))
                if self.attention_bias:
                    out[f"{p}.{branch}.linear1.bias"] = ("F32", (i,))
                    out[f"{p}.{branch}.linear2.bias"] = ("F32", (h,))
            for norm in ("norm_feed_forward1", "norm_self_att", "norm_conv", "norm_feed_forward2", "norm_out"):
                out[f"{p}.{norm}.weight"] = ("F32", (h,))
                out[f"{p}.{norm}.bias"] = ("F32", (h,))
            an = self.attention_names
            for proj in an[:5]:
                out[f"{p}.self_attn.{proj}.weight"] = ("F32", (h, h))
            if self.attention_bias:
                for proj in an[:4]:
                    out[f"{p}.self_attn.{proj}.bias"] = ("F32", (h,))
            out[f"{p}.self_attn.{an[5]}"] = ("F32", (self.heads, self.head_dim))
            out[f"{p}.self_attn.{an[6]}"] = ("F32", (self.heads, self.head_dim))
            out[f"{p}.conv.pointwise_conv1.weight"] = ("F32", (2 * h, h, 1))
            out[f"{p}.conv.pointwise_conv2.weight"] = ("F32", (h, h, 1))
            out[f"{p}.conv.depthwise_conv.weight"] = ("F32", (h, 1, k))
            if self.convolution_bias:
                out[f"{p}.conv.pointwise_conv1.bias"] = ("F32", (2 * h,))
                out[f"{p}.conv.pointwise_conv2.bias"] = ("F32", (h,))
                out[f"{p}.conv.depthwise_conv.bias"] = ("F32", (h,))
            names = ("weight", "bias", "running_mean", "running_var") if self.conv_batch_norm else ("weight", "bias")
            for n in names:
                out[f"{p}.conv.{self.conv_norm_name}.{n}"] = ("F32", (h,))
            if self.conv_batch_norm:
                out[f"{p}.conv.{self.conv_norm_name}.num_batches_tracked"] = ("I64", ())
        for n in self.conv_names:
            out[f"{self.prefix}.{n}.weight"] = ("F32", (c, 1, 3, 3))
            out[f"{self.prefix}.{n}.bias"] = ("F32", (c,))
        for n in self.pointwise_names:
            out[f"{self.prefix}.{n}.weight"] = ("F32", (c, c, 1, 1))
            out[f"{self.prefix}.{n}.bias"] = ("F32", (c,))
        out[f"{self.prefix}.{self.linear_name}.weight"] = ("F32", (h, self.linear_in))
        out[f"{self.prefix}.{self.linear_name}.bias"] = ("F32", (h,))
        return out


def random_tensors(expected: dict[str, tuple[str, tuple[int, ...]]], seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    """Seeded random tensors in the published layout (norm weights near one, variances positive)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(expected):
        dtype, shape = expected[name]
        if dtype == "I64":
            out[name] = torch.zeros(shape, dtype=torch.int64)
        elif name.endswith("running_var"):
            out[name] = 0.5 + torch.rand(shape, generator=g)
        elif ("norm" in name and name.endswith(".weight")):
            out[name] = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("depthwise_conv.weight") or ".subsampling.layers." in name and name.endswith("weight"):
            out[name] = 0.3 * torch.randn(shape, generator=g)
        else:
            out[name] = std * torch.randn(shape, generator=g)
    return out


class ConformerEncoder:
    """Encoder weights in their device forms and the forward pass over a batch of utterances."""

    def __init__(self, spec: ConformerSpec, tensors: dict[str, torch.Tensor], device: torch.device | str = "cpu"):
        spec.check()
        self.spec, self.device = spec, torch.device(device)
        dev = self.device
        p = spec.prefix

        def f32(name: str) -> torch.Tensor:
            return tensors[name].float().contiguous().to(dev)

        def opt32(name: str) -> torch.Tensor | None:
            return f32(name) if name in tensors else None

        def w16(t: torch.Tensor) -> torch.Tensor:
            return t.to(BF16).contiguous().to(dev)

        c = spec.sub_channels
        self.sub_conv = []
        for name in spec.conv_names:
            w = tensors[f"{p}.{name}.weight"].float().reshape(c, 9).t().contiguous()          # [9, C]
            self.sub_conv.append((w.to(dev), f32(f"{p}.{name}.bias")))
        self.sub_pw = [(w16(tensors[f"{p}.{n}.weight"].float().reshape(c, c)), w16(tensors[f"{p}.{n}.bias"].float()))
                       for n in spec.pointwise_names]
        fq = spec.sub_freq
        lw = tensors[f"{p}.{spec.linear_name}.weight"].float()                               # columns: ch * F + f
        lw = lw.reshape(spec.hidden, c, fq).permute(0, 2, 1).reshape(spec.hidden, fq * c)     # columns: f * C + ch
        self.sub_linear = (w16(lw), w16(tensors[f"{p}.{spec.linear_name}.bias"].float()))
        self.layers = []
        h = spec.hidden
        for li in range(spec.layers):
            q = f"{p}.layers.{li}"
            L: dict[str, object] = {}
            for tag, branch, norm in (("ff1", "feed_forward1", "norm_feed_forward1"), ("ff2", "feed_forward2", "norm_feed_forward2")):
                b1 = tensors.get(f"{q}.{branch}.linear1.bias")
                L[tag] = dict(norm=(f32(f"{q}.{norm}.weight"), f32(f"{q}.{norm}.bias")),
                              w1=w16(tensors[f"{q}.{branch}.linear1.weight"].float()),
                              b1=w16(b1.float()) if b1 is not None else None,
                              w2=w16(tensors[f"{q}.{branch}.linear2.weight"].float()),
                              b2=opt32(f"{q}.{branch}.linear2.bias"))
            a = f"{q}.self_attn"
            an = spec.attention_names
            wqkv = torch.cat([tensors[f"{a}.{n}.weight"].float() for n in an[:3]], dim=0)
            bqkv = None
            if f"{a}.{an[0]}.bias" in tensors:
                bqkv = w16(torch.cat([tensors[f"{a}.{n}.bias"].float() for n in an[:3]]))
            L["attn"] = dict(norm=(f32(f"{q}.norm_self_att.weight"), f32(f"{q}.norm_self_att.bias")), wqkv=w16(wqkv), bqkv=bqkv,
                             wrel=w16(tensors[f"{a}.{an[4]}.weight"].float()), wo=w16(tensors[f"{a}.{an[3]}.weight"].float()),
                             bo=opt32(f"{a}.{an[3]}.bias"), u=f32(f"{a}.{an[5]}"), v=f32(f"{a}.{an[6]}"))
            cv = f"{q}.conv"
            dw = tensors[f"{cv}.depthwise_conv.weight"].float().reshape(h, spec.conv_kernel)
            dwb = tensors[f"{cv}.depthwise_conv.bias"].float() if f"{cv}.depthwise_conv.bias" in tensors else torch.zeros(h)
            post = None
            cn = f"{cv}.{spec.conv_norm_name}"
            if spec.conv_batch_norm:
                g = tensors[f"{cn}.weight"].float() * torch.rsqrt(tensors[f"{cn}.running_var"].float() + 1e-5)
                dw = dw * g[:, None]
                dwb = (dwb - tensors[f"{cn}.running_mean"].float()) * g + tensors[f"{cn}.bias"].float()
            else:
                post = (f32(f"{cn}.weight"), f32(f"{cn}.bias"))
            L["conv"] = dict(norm=(f32(f"{q}.norm_conv.weight"), f32(f"{q}.norm_conv.bias")),
                             w1=w16(tensors[f"{cv}.pointwise_conv1.weight"].float().reshape(2 * h, h)),
                             b1=opt32(f"{cv}.pointwise_conv1.bias"), dw=dw.t().contiguous().to(dev), dwb=dwb.contiguous().to(dev),
                             post=post, w2=w16(tensors[f"{cv}.pointwise_conv2.weight"].float().reshape(h, h)),
                             b2=opt32(f"{cv}.pointwise_conv2.bias"))
            L["out"] = (f32(f"{q}.norm_out.weight"), f32(f"{q}.norm_out.bias"))
            self.layers.append(L)
        self._pos: dict[int, torch.Tensor] = {}

    # --------------------------------------------------------------------------------------------
    def positions(self, rows: int) -> torch.Tensor:
        if rows < 1 or rows > self.spec.max_position:
            raise ValueError(f"position rows {rows} exceed max_position_embeddings {self.spec.max_position}")
        t = self._pos.get(rows)
        if t is None:
            t = speech_ops.relative_positions(rows, self.spec.hidden).to(BF16).to(self.device)
            self._pos[rows] = t
        return t

    def subsample(self, feat: torch.Tensor, valid: list[int]) -> tuple[torch.Tensor, list[int]]:
        """[batch, frames, mel] FP32 + valid frames -> ([batch * T', hidden] BF16, valid rows per utterance)."""
        s, dev = self.spec, self.device
        batch = feat.shape[0]
        v = list(valid)
        x = None
        for idx in range(3):
            v_out = [speech_ops.conv_out_len(n, *s.pads) for n in v]
            w, b = self.sub_conv[idx]
            if idx == 0:
                x = speech_ops.sub_conv_first(feat, w, b, torch.tensor(v_out, dtype=torch.int32, device=dev), s.pads)
            else:
                x = speech_ops.sub_dwconv(x, w, b, torch.tensor(v, dtype=torch.int32, device=dev), s.pads)
                pw, pb = self.sub_pw[idx - 1]
                shape = x.shape
                x = vision_ops.linear_bias_act(x.reshape(-1, s.sub_channels), pw, pb, "relu").reshape(shape)
            v = v_out
        t3, f3 = x.shape[1], x.shape[2]
        lw, lb = self.sub_linear
        hdn = vision_ops.linear_bias_act(x.reshape(batch * t3, f3 * s.sub_channels), lw, lb, "none")
        return hdn, v

    def layer(self, index: int, h: torch.Tensor, x: torch.Tensor, lens: torch.Tensor, batch: int, pos: torch.Tensor) -> torch.Tensor:
        """One conformer layer. ``h`` is the residual stream (updated in place), ``x`` = LayerNorm_ff1(h); returns the
        layer's normalised output, which is the next layer's residual stream."""
        s, L = self.spec, self.layers[index]
        hd = s.hidden
        ff = L["ff1"]
        u = vision_ops.linear_bias_act(x, ff["w1"], ff["b1"], "silu")
        d = ops.linear(u, ff["w2"])
        at = L["attn"]
        x = speech_ops.scale_add_layernorm(h, d, ff["b2"], 0.5, *at["norm"])
        qkv = vision_ops.linear_bias_act(x, at["wqkv"], at["bqkv"], "none")
        rel = ops.linear(pos, at["wrel"])
        core = speech_ops.relpos_attention(qkv[:, :hd], qkv[:, hd:2 * hd], qkv[:, 2 * hd:], rel, at["u"], at["v"], lens, batch,
                                           s.heads, *s.attention_window)
        d = ops.linear(core, at["wo"])
        cv = L["conv"]
        x = speech_ops.scale_add_layernorm(h, d, at["bo"], 1.0, *cv["norm"])
        e = ops.linear(x, cv["w1"])
        if cv["post"] is None:
            cvd = speech_ops.glu_dwconv1d(e, cv["b1"], cv["dw"], cv["dwb"], lens, batch, s.conv_left, silu=True)
        else:
            cvd = speech_ops.glu_dwconv1d(e, cv["b1"], cv["dw"], cv["dwb"], lens, batch, s.conv_left, silu=False)
            cvd = speech_ops.scale_add_layernorm(cvd, None, None, 0.0, *cv["post"])
            cvd = vision_ops.bias_act_(cvd, None, "silu")
        d = ops.linear(cvd, cv["w2"])
        ff = L["ff2"]
        x = speech_ops.scale_add_layernorm(h, d, cv["b2"], 1.0, *ff["norm"])
        u = vision_ops.linear_bias_act(x, ff["w1"], ff["b1"], "silu")
        d = ops.linear(u, ff["w2"])
        return speech_ops.scale_add_layernorm(h, d, ff["b2"], 0.5, *L["out"])

    def encode(self, feat: torch.Tensor, valid: list[int]) -> tuple[torch.Tensor, list[int]]:
        """Log-mel features [batch, frames, mel] FP32 with ``valid`` frames per utterance ->
        ([batch, T', hidden] BF16, valid rows per utterance). Rows beyond an utterance's valid rows are unspecified."""
        batch = feat.shape[0]
        h, rows = self.subsample(feat.to(self.device), valid)
        t = h.shape[0] // batch
        lens = torch.tensor(rows, dtype=torch.int32, device=self.device)
        pos = self.positions(t)
        for li in range(self.spec.layers):
            x = speech_ops.scale_add_layernorm(h, None, None, 0.0, *self.layers[li]["ff1"]["norm"])
            h = self.layer(li, h, x, lens, batch, pos)
        return h.reshape(batch, t, self.spec.hidden), rows


class ConformerStream:
    """Incremental encoding with a cache-aware streaming encoder (chunk-wise attention context, causal convolutions,
    causal stem pads; src/backend/cuda/engine_parakeet.rs:1508-2010 of the reference keeps the same three caches).
    Mel frames go in as they arrive, encoder rows come out chunk by chunk and equal the rows an offline ``encode`` of the
    whole utterance produces: per layer the stream keeps the fused Q/K/V rows of the last ``left_chunks`` chunks and the
    last ``kernel - 1`` rows entering the depthwise convolution; the stem is re-run over the few frames a chunk's rows
    look back on."""

    def __init__(self, encoder: ConformerEncoder):
        s = encoder.spec
        if not (s.chunk_size > 0 and s.right_chunks == 0 and s.causal_conv and s.pad_left == 2 and s.pad_right == 1):
            raise ValueError("streaming needs chunk-wise attention without look-ahead, causal convolutions and causal stem pads")
        self.enc, self.spec = encoder, s
        self.frames = torch.zeros(0, s.mel_bins, dtype=torch.float32, device=encoder.device)
        self.rows_out = 0                                   # encoder rows emitted so far
        self.qkv = [None] * s.layers                        # [cached rows, 3 * hidden]
        self.conv = [None] * s.layers                       # [cached rows, 2 * hidden]
        self.finished = False

    def _stem(self, first_row: int, n_rows: int, last: bool) -> torch.Tensor:
        """Rows ``first_row .. first_row + n_rows`` of the stem's output from the buffered frames. A row looks back 14
        frames; the window starts 16 frames (two rows) early so that stride phases line up, and those rows are dropped."""
        s = self.spec
        lead = min(2, first_row)
        f0 = 8 * (first_row - lead)
        f1 = self.frames.shape[0] if last else min(self.frames.shape[0], 8 * (first_row + n_rows - 1) + 1)
        window = self.frames[f0:f1][None]
        hid, rows = self.enc.subsample(window, [f1 - f0])
        return hid[lead: lead + n_rows]

    def _layers(self, h: torch.Tensor) -> torch.Tensor:
        enc, s = self.enc, self.spec
        n_new, hd = h.shape[0], s.hidden
        keep = s.left_chunks * s.chunk_size
        dev = enc.device
        for li in range(s.layers):
            L = enc.layers[li]
            x = speech_ops.scale_add_layernorm(h, None, None, 0.0, *L["ff1"]["norm"])
            ff = L["ff1"]
            d = ops.linear(vision_ops.linear_bias_act(x, ff["w1"], ff["b1"], "silu"), ff["w2"])
            at = L["attn"]
            x = speech_ops.scale_add_layernorm(h, d, ff["b2"], 0.5, *at["norm"])
            qkv_new = vision_ops.linear_bias_act(x, at["wqkv"], at["bqkv"], "none")
            qkv = qkv_new if self.qkv[li] is None else torch.cat([self.qkv[li], qkv_new], dim=0)
            t = qkv.shape[0]
            rel = ops.linear(enc.positions(t), at["wrel"])
            lens = torch.tensor([t], dtype=torch.int32, device=dev)
            # the cached rows start on a chunk boundary, so local chunk indices differ from the absolute ones by a constant
            core = speech_ops.relpos_attention(qkv[:, :hd], qkv[:, hd:2 * hd], qkv[:, 2 * hd:], rel, at["u"], at["v"], lens, 1,
                                               s.heads, s.left_chunks, 0, s.chunk_size)[t - n_new:]
            self.qkv[li] = qkv[max(0, t - keep):].contiguous()
            cv = L["conv"]
            x = speech_ops.scale_add_layernorm(h, ops.linear(core.contiguous(), at["wo"]), at["bo"], 1.0, *cv["norm"])
            e_new = ops.linear(x, cv["w1"])
            e = e_new if self.conv[li] is None else torch.cat([self.conv[li], e_new], dim=0)
            te = e.shape[0]
            lens_e = torch.tensor([te], dtype=torch.int32, device=dev)
            cvd = speech_ops.glu_dwconv1d(e, cv["b1"], cv["dw"], cv["dwb"], lens_e, 1, s.conv_left, silu=cv["post"] is None)[te - n_new:]
            self.conv[li] = e[max(0, te - (s.conv_kernel - 1)):].contiguous()
            cvd = cvd.contiguous()
            if cv["post"] is not None:
                cvd = vision_ops.bias_act_(speech_ops.scale_add_layernorm(cvd, None, None, 0.0, *cv["post"]), None, "silu")
            ff = L["ff2"]
            x = speech_ops.scale_add_layernorm(h, ops.linear(cvd, cv["w2"]), cv["b2"], 1.0, *ff["norm"])
            d = ops.linear(vision_ops.linear_bias_act(x, ff["w1"], ff["b1"], "silu"), ff["w2"])
            h = speech_ops.scale_add_layernorm(h, d, ff["b2"], 0.5, *L["out"])
        return h

    def push(self, frames: torch.Tensor, last: bool = False) -> torch.Tensor:
        """Appends mel frames [n, mel_bins] (FP32, un-normalised or normalised by the caller) and returns the encoder
        rows [m, hidden] that became complete, whole chunks at a time; ``last`` flushes the tail of the utterance."""
        if self.finished:
            raise RuntimeError("the stream is finished")
        out = [self._layers(h) for _, h in self.stem_chunks(frames, last)]
        if not out:
            return torch.zeros(0, self.spec.hidden, dtype=torch.bfloat16, device=self.enc.device)
        return torch.cat(out, dim=0)

    def stem_chunks(self, frames: torch.Tensor, last: bool = False):
        """Appends mel frames and yields ``(first_row, stem rows)`` for every chunk that became complete: the rows as
        they enter the first layer. ``push`` runs them through this stream's layers; a caller that conditions the
        rows first (several lanes over one audio stream, each with layer caches of its own) drives ``_layers`` of
        other streams with them."""
        if self.finished:
            raise RuntimeError("the stream is finished")
        s = self.spec
        self.frames = torch.cat([self.frames, frames.to(self.frames.device, torch.float32)], dim=0)
        n = self.frames.shape[0]
        if last:
            self.finished = True
        while True:
            # row r is complete once frame 8r (its newest input) has arrived
            complete = (n - 1) // 8 + 1 if n > 0 else 0
            total = s.sub_len(n) if (last and n > 0) else complete
            avail = total - self.rows_out
            if avail >= s.chunk_size:
                take = s.chunk_size
            elif last and avail > 0:
                take = avail
            else:
                break
            h = self._stem(self.rows_out, take, last and take == avail)
            first = self.rows_out
            self.rows_out += take
            yield first, h.contiguous()
