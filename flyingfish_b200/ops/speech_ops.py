"""Operators of the speech models. CUDA: ``csrc/speech.cu``; CPU: FP32 oracles restating the same arithmetic with BF16
rounding at the points where the kernels round. Reference counterparts: src/audio.rs (log-mel), kernels/speech_ops.cu
(LSTM step, conv2d, depthwise conv, batch norm, relative attention) and the launch sequences of
src/backend/cuda/engine_parakeet.rs (sub-sampling :1058-1147, conformer layer :1168-1305, greedy decode :2550-2633)."""
from __future__ import annotations

import math
from ctypes import c_float, c_longlong

import torch

from . import _count, _require
from .lib import check, kernels, ptr, stream_ptr

BF16 = torch.bfloat16

# words of the device-resident transducer decode state (csrc/speech.cu)
TS_FRAME, TS_TOKEN, TS_COUNT, TS_DONE, TS_ADVANCE, TS_ERROR, TS_VALID, TS_CAP, TS_SYMS, TS_MAXSYM, TS_WORDS = 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 16


def _r(x: torch.Tensor) -> torch.Tensor:
    return x.to(BF16).float()


# ------------------------------------------------------------------------------------------------
# log-mel features
# ------------------------------------------------------------------------------------------------
def hann_window(win_length: int, n_fft: int) -> torch.Tensor:
    """Symmetric Hann window of ``win_length`` taps centred in an ``n_fft`` frame (FP32)."""
    w = torch.zeros(n_fft, dtype=torch.float32)
    step = torch.tensor(2.0 * math.pi / (win_length - 1), dtype=torch.float32)
    idx = torch.arange(win_length, dtype=torch.float32)
    first = (n_fft - win_length) // 2
    w[first:first + win_length] = -0.5 * torch.cos(idx * step) + 0.5
    return w


def mel_filterbank(sampling_rate: int, n_fft: int, mel_bins: int) -> torch.Tensor:
    """[mel_bins, n_fft/2+1] triangular filters on the Slaney mel scale (linear below 1 kHz, logarithmic above), each
    scaled by 2 / (its band width in Hz)."""
    def hz_to_mel(hz: float) -> float:
        return hz / (200.0 / 3.0) if hz < 1000.0 else 15.0 + math.log(hz / 1000.0) / (math.log(6.4) / 27.0)

    def mel_to_hz(mel: float) -> float:
        return mel * (200.0 / 3.0) if mel < 15.0 else 1000.0 * math.exp((mel - 15.0) * (math.log(6.4) / 27.0))

    low, high = hz_to_mel(0.0), hz_to_mel(sampling_rate / 2.0)
    edges = [mel_to_hz(low + (high - low) * i / (mel_bins + 1)) for i in range(mel_bins + 2)]
    bins = n_fft // 2 + 1
    hz = torch.arange(bins, dtype=torch.float64) * sampling_rate / n_fft
    out = torch.zeros(mel_bins, bins, dtype=torch.float32)
    for band in range(mel_bins):
        lower = (hz - edges[band]) / (edges[band + 1] - edges[band])
        upper = (edges[band + 2] - hz) / (edges[band + 2] - edges[band + 1])
        tri = torch.minimum(lower, upper).clamp_min(0.0).float()
        out[band] = tri * float(2.0 / (edges[band + 2] - edges[band]))
    return out


def band_ranges(filters: torch.Tensor) -> torch.Tensor:
    """[mel_bins, 2] int32: first bin and one-past-last bin with a non-zero weight of every band."""
    nz = filters != 0
    bins = filters.shape[1]
    idx = torch.arange(bins)
    first = torch.where(nz, idx, bins).min(dim=1).values
    last = torch.where(nz, idx, -1).max(dim=1).values + 1
    first = torch.minimum(first, last.clamp_min(0))
    return torch.stack([first, last.clamp_min(0)], dim=1).to(torch.int32).contiguous()


def logmel(wave: torch.Tensor, lens: torch.Tensor, window: torch.Tensor, filters: torch.Tensor,
           ranges: torch.Tensor | None, hop: int, preemph: float, log_guard: float, normalize: bool,
           norm_eps: float) -> torch.Tensor:
    """``wave`` [batch, samples] FP32 (zero padded), ``lens`` [batch] int32 -> [batch, frames, mel_bins] FP32 with
    ``frames = samples // hop + 1``. Frame t covers samples ``t * hop - n_fft / 2 ...`` (zero beyond the utterance),
    pre-emphasis ``x[i] - p * x[i-1]`` is applied before the window; frames at or beyond ``len // hop`` are zero and
    the per-band normalisation (mean, unbiased standard deviation + eps) runs over the frames before that."""
    batch, samples = wave.shape
    n_fft, mel_bins = window.numel(), filters.shape[0]
    frames = samples // hop + 1
    if not wave.is_cuda:
        out = torch.zeros(batch, frames, mel_bins, dtype=torch.float32)
        half = n_fft // 2
        for b in range(batch):
            n = int(lens[b])
            valid = n // hop
            x = wave[b, :n].float()
            em = torch.cat([x[:1], x[1:] - preemph * x[:-1]]) if n > 1 else x.clone()
            padded = torch.cat([torch.zeros(half), em, torch.zeros(half + frames * hop)])
            idx = torch.arange(valid)[:, None] * hop + torch.arange(n_fft)[None, :]
            fr = padded[idx] * window[None, :]
            spec = torch.fft.rfft(fr.double(), dim=1)
            power = (spec.real ** 2 + spec.imag ** 2).float()
            feat = torch.log(power @ filters.t() + log_guard)
            if normalize:
                mean = feat.mean(0, keepdim=True)
                std = torch.sqrt(((feat - mean) ** 2).sum(0, keepdim=True) / max(valid - 1, 1))
                feat = (feat - mean) / (std + norm_eps)
            out[b, :valid] = feat
        return out
    _require(wave.dtype == torch.float32 and wave.is_contiguous() and lens.dtype == torch.int32, "logmel: fp32 rows, int32 lens")
    if ranges is None:
        ranges = band_ranges(filters.cpu()).to(wave.device)
    out = torch.empty(batch, frames, mel_bins, dtype=torch.float32, device=wave.device)
    rc = kernels().ff_logmel(ptr(wave), ptr(lens), ptr(window), ptr(filters), ptr(ranges), ptr(out), batch,
                             c_longlong(samples), frames, n_fft, hop, mel_bins, c_float(preemph), c_float(log_guard),
                             stream_ptr())
    check(rc, "ff_logmel")
    _count()
    if normalize:
        rc = kernels().ff_feat_normalize(ptr(out), ptr(lens), batch, frames, mel_bins, hop, c_float(norm_eps), stream_ptr())
        check(rc, "ff_feat_normalize")
        _count()
    return out


# ------------------------------------------------------------------------------------------------
# sub-sampling stem (channels-last)
# ------------------------------------------------------------------------------------------------
def conv_out_len(n: int, pad_left: int, pad_right: int) -> int:
    """Output length of a kernel-3 stride-2 convolution over ``n`` samples with the given pads."""
    span = n + pad_left + pad_right
    if span < 3:
        raise ValueError(f"convolution span {span} is shorter than the kernel")
    return (span - 3) // 2 + 1


def _conv_ref(x: torch.Tensor, w9c: torch.Tensor, bias: torch.Tensor, pad: tuple[int, int], depthwise: bool) -> torch.Tensor:
    # x: [B, T, F, Cin] fp32; w9c: [9, C]
    c = w9c.shape[1]
    xin = x.permute(0, 3, 1, 2)
    xin = torch.nn.functional.pad(xin, (pad[0], pad[1], pad[0], pad[1]))
    w = w9c.t().reshape(c, 1, 3, 3)
    y = torch.nn.functional.conv2d(xin, w, bias, stride=2, groups=c if depthwise else 1)
    return y.permute(0, 2, 3, 1)


def sub_conv_first(feat: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, valid_out: torch.Tensor,
                   pads: tuple[int, int]) -> torch.Tensor:
    """[batch, T, F] FP32 -> [batch, T1, F1, C] BF16 = relu(conv3x3 stride 2); rows at or beyond ``valid_out`` zero.
    ``w`` is [9, C] FP32 (tap-major), ``pads`` = (left, right) used on both axes."""
    batch, t, f = feat.shape
    c = w.shape[1]
    t1, f1 = conv_out_len(t, *pads), conv_out_len(f, *pads)
    if not feat.is_cuda:
        y = torch.relu(_conv_ref(feat.float()[..., None], w.float(), bias.float(), pads, False))
        mask = torch.arange(t1)[None, :] < valid_out[:, None]
        return (y * mask[:, :, None, None]).to(BF16)
    _require(feat.dtype == torch.float32 and feat.is_contiguous() and w.dtype == torch.float32 and w.is_contiguous(),
             "sub_conv_first: fp32 input and weights")
    out = torch.empty(batch, t1, f1, c, dtype=BF16, device=feat.device)
    rc = kernels().ff_sub_conv_first(ptr(feat), ptr(w), ptr(bias), ptr(valid_out), ptr(out), batch, t, f, t1, f1, c,
                                     pads[0], pads[0], stream_ptr())
    check(rc, "ff_sub_conv_first")
    _count()
    return out


def sub_dwconv(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, valid_in: torch.Tensor,
               pads: tuple[int, int]) -> torch.Tensor:
    """[batch, T, F, C] BF16 -> [batch, T1, F1, C] BF16: depthwise 3x3 stride 2, input rows at or beyond ``valid_in``
    read as zero, no activation."""
    batch, t, f, c = x.shape
    t1, f1 = conv_out_len(t, *pads), conv_out_len(f, *pads)
    if not x.is_cuda:
        mask = torch.arange(t)[None, :] < valid_in[:, None]
        xin = x.float() * mask[:, :, None, None]
        return _conv_ref(xin, w.float(), bias.float(), pads, True).to(BF16)
    _require(x.dtype == BF16 and x.is_contiguous() and w.dtype == torch.float32 and w.is_contiguous(), "sub_dwconv: layout")
    out = torch.empty(batch, t1, f1, c, dtype=BF16, device=x.device)
    rc = kernels().ff_sub_dwconv(ptr(x), ptr(w), ptr(bias), ptr(valid_in), ptr(out), batch, t, f, t1, f1, c, pads[0],
                                 pads[0], stream_ptr())
    check(rc, "ff_sub_dwconv")
    _count()
    return out


# ------------------------------------------------------------------------------------------------
# conformer layer pieces
# ------------------------------------------------------------------------------------------------
def glu_dwconv1d(x: torch.Tensor, xbias: torch.Tensor | None, w: torch.Tensor, bias: torch.Tensor, lens: torch.Tensor,
                 batch: int, left: int, silu: bool = True) -> torch.Tensor:
    """``x`` [batch * T, 2H] BF16 (value half, gate half) -> [batch * T, H] BF16:
    ``u = bf16((value + b) * sigmoid(gate + b))`` with frames outside ``[0, len)`` zero, a depthwise convolution over
    time (``w`` [K, H] FP32, tap k reads frame ``t + k - left``), ``bias`` [H] and an optional SiLU."""
    rows, h2 = x.shape
    h, t, k = h2 // 2, rows // batch, w.shape[0]
    if not x.is_cuda:
        xf = x.float()
        if xbias is not None:
            xf = xf + xbias.float()
        u = _r(xf[:, :h] * torch.sigmoid(xf[:, h:])).reshape(batch, t, h)
        mask = torch.arange(t)[None, :] < lens[:, None]
        u = u * mask[:, :, None]
        up = torch.nn.functional.pad(u.permute(0, 2, 1), (left, k - 1 - left))
        y = torch.nn.functional.conv1d(up, w.float().t().reshape(h, 1, k), bias.float(), groups=h).permute(0, 2, 1)
        if silu:
            y = y * torch.sigmoid(y)
        return y.reshape(rows, h).to(BF16)
    _require(x.dtype == BF16 and x.is_contiguous() and w.dtype == torch.float32 and w.is_contiguous()
             and bias.dtype == torch.float32, "glu_dwconv1d: layout")
    y = torch.empty(rows, h, dtype=BF16, device=x.device)
    rc = kernels().ff_glu_dwconv1d(ptr(x), ptr(xbias), ptr(w), ptr(bias), ptr(lens), ptr(y), batch, t, h, k, left,
                                   1 if silu else 0, stream_ptr())
    check(rc, "ff_glu_dwconv1d")
    _count()
    return y


def scale_add_layernorm(h: torch.Tensor, delta: torch.Tensor | None, dbias: torch.Tensor | None, scale: float,
                        w: torch.Tensor | None, b: torch.Tensor | None, eps: float = 1e-5) -> torch.Tensor | None:
    """In place ``h = bf16(h + scale * (delta + dbias))`` (skipped without ``delta``), then returns
    ``LayerNorm(h) * w + b`` in BF16 (``None`` without ``w``). ``dbias``, ``w``, ``b`` are FP32."""
    if not h.is_cuda:
        if delta is not None:
            d = delta.float() + (dbias.float() if dbias is not None else 0.0)
            h.copy_((h.float() + scale * d).to(h.dtype))
        if w is None:
            return None
        hf = h.float()
        mean = hf.mean(-1, keepdim=True)
        var = ((hf - mean) ** 2).mean(-1, keepdim=True)
        y = (hf - mean) * torch.rsqrt(var + eps) * w.float()
        return (y + b.float() if b is not None else y).to(h.dtype)
    rows, hidden = h.shape
    _require(h.dtype == BF16 and h.stride(1) == 1 and (delta is None or (delta.dtype == BF16 and delta.stride(1) == 1))
             and (w is None or w.dtype == torch.float32), "scale_add_layernorm: layout")
    y = torch.empty(rows, hidden, dtype=BF16, device=h.device) if w is not None else None
    rc = kernels().ff_scale_add_layernorm(ptr(h), ptr(delta), ptr(dbias), ptr(w), ptr(b), ptr(y), rows, hidden, h.stride(0),
                                          delta.stride(0) if delta is not None else hidden, hidden, c_float(scale),
                                          c_float(eps), stream_ptr())
    check(rc, "ff_scale_add_layernorm")
    _count()
    return y


def relative_positions(rows: int, hidden: int, device=None) -> torch.Tensor:
    """[2 * rows - 1, hidden] sinusoidal table: row c encodes relative offset ``rows - 1 - c`` with interleaved
    (sin, cos) pairs of frequency ``10000 ** (-2i / hidden)``."""
    inv = 1.0 / torch.pow(torch.tensor(10000.0), torch.arange(0, hidden, 2, dtype=torch.float32) / hidden)
    posn = torch.arange(rows - 1, -rows, -1, dtype=torch.float32)
    phase = posn[:, None] * inv[None, :]
    tab = torch.stack([torch.sin(phase), torch.cos(phase)], dim=-1).reshape(2 * rows - 1, hidden)
    return tab.to(device) if device is not None else tab


def relpos_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos: torch.Tensor, bias_u: torch.Tensor,
                     bias_v: torch.Tensor, lens: torch.Tensor, batch: int, heads: int, left: int = -1,
                     right: int = -1, chunk: int = 0) -> torch.Tensor:
    """Relative-position self-attention. ``q``, ``k``, ``v``: [batch * T, heads * D] BF16 views (column slices of a
    packed projection are fine), ``pos``: [2T - 1, heads * D] BF16 projected position table (row ``T - 1 - i + j`` serves
    query i / key j), ``bias_u`` / ``bias_v``: [heads, D] FP32. score = ((q + u) . k + (q + v) . p) / sqrt(D); keys at or
    beyond ``lens[b]`` and outside ``[i - left, i + right]`` are masked; rows at or beyond ``lens[b]`` come back zero.
    With ``chunk > 0`` the context is chunk-wise instead (streaming encoders): a query in chunk ``c = i // chunk`` sees the
    keys of chunks ``c - left .. c + right``."""
    rows, width = q.shape
    t, d = rows // batch, width // heads
    if not q.is_cuda:
        qf = q.float().reshape(batch, t, heads, d)
        kf = k.float().reshape(batch, t, heads, d)
        vf = v.float().reshape(batch, t, heads, d)
        pf = pos.float().reshape(2 * t - 1, heads, d)
        qu, qv = _r(qf + bias_u.float()), _r(qf + bias_v.float())
        ac = torch.einsum("bihd,bjhd->bhij", qu, kf)
        raw = torch.einsum("bihd,chd->bhic", qv, pf)
        i = torch.arange(t)[:, None]
        j = torch.arange(t)[None, :]
        idx = (t - 1 - i + j).expand(batch, heads, t, t)
        bd = torch.gather(raw, 3, idx)
        sc = (ac + bd) / math.sqrt(d)
        ok = (j < lens[:, None, None, None])
        if chunk > 0:
            qc, kc = i // chunk, j // chunk
            ok = ok & (kc >= qc - left) & (kc <= qc + right)
        else:
            if left >= 0:
                ok = ok & (j >= i - left)
            if right >= 0:
                ok = ok & (j <= i + right)
        sc = sc.masked_fill(~ok, float("-inf"))
        p = torch.nan_to_num(torch.softmax(sc, dim=-1))       # a row without any visible key (padding rows) is zero
        o = torch.einsum("bhij,bjhd->bihd", p, vf)
        o = o * (torch.arange(t)[None, :, None, None] < lens[:, None, None, None])
        return o.reshape(rows, width).to(BF16)
    _require(q.dtype == BF16 and q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and pos.stride(1) == 1
             and pos.dtype == BF16 and bias_u.dtype == torch.float32 and bias_u.is_contiguous() and bias_v.is_contiguous()
             and pos.shape[0] == 2 * t - 1, "relpos_attention: layout")
    out = torch.empty(rows, width, dtype=BF16, device=q.device)
    rc = kernels().ff_relpos_attention(ptr(q), ptr(k), ptr(v), ptr(pos), ptr(bias_u), ptr(bias_v), ptr(lens), ptr(out),
                                       batch, t, heads, d, q.stride(0), k.stride(0), v.stride(0), pos.stride(0), width,
                                       left, right, chunk, c_float(1.0 / math.sqrt(d)), stream_ptr())
    check(rc, "ff_relpos_attention")
    _count()
    return out


# ------------------------------------------------------------------------------------------------
# transducer decoder steps (device-resident state)
# ------------------------------------------------------------------------------------------------
def _rows(t: torch.Tensor | None) -> torch.Tensor | None:
    """Decoder step buffers are [batch, width]; a 1-D tensor is the batch of one."""
    return None if t is None else (t if t.dim() >= 2 else t[None])


def tdt_embed(table: torch.Tensor, state: torch.Tensor, xh0: torch.Tensor) -> None:
    """``xh0[b, :Hd] = table[state[b].token]`` for every utterance whose step advances the prediction network.
    ``state``: [batch, TS_WORDS] int32, ``xh0``: [batch, >= Hd] (rows may be wider: the input half of ``[x; h]``)."""
    hd = table.shape[1]
    st, x = _rows(state), _rows(xh0)
    if not table.is_cuda:
        for b in range(st.shape[0]):
            if int(st[b, TS_DONE]) or not int(st[b, TS_ADVANCE]):
                continue
            x[b, :hd] = table[min(max(int(st[b, TS_TOKEN]), 0), table.shape[0] - 1)]
        return
    _require(st.is_contiguous() and x.stride(1) == 1, "tdt_embed: layout")
    rc = kernels().ff_tdt_embed(ptr(table), ptr(st), ptr(x), st.shape[0], hd, table.shape[0], x.stride(0), stream_ptr())
    check(rc, "ff_tdt_embed")
    _count()


def lstm_cell(gates: torch.Tensor, bias: torch.Tensor, c: torch.Tensor, h_self: torch.Tensor,
              h_next: torch.Tensor | None, state: torch.Tensor | None) -> None:
    """One LSTM cell update per utterance from the gate pre-activations ``gates`` [batch, 4 Hd] BF16 (i, f, g, o;
    ``W [x; h]``) and ``bias`` [4 Hd] FP32. ``c`` [batch, Hd] (FP32) is updated in place, the new hidden state is written
    (BF16) to ``h_self`` and ``h_next`` (row views of wider buffers are fine). With ``state`` an utterance is only updated
    when its decode step advances."""
    g, cc, hs, hn, st = _rows(gates), _rows(c), _rows(h_self), _rows(h_next), _rows(state)
    batch, hd = cc.shape
    if not g.is_cuda:
        for b in range(batch):
            if st is not None and (int(st[b, TS_DONE]) or not int(st[b, TS_ADVANCE])):
                continue
            z = g[b].float().reshape(4, hd) + bias.float().reshape(4, hd)
            cn = torch.sigmoid(z[1]) * cc[b] + torch.sigmoid(z[0]) * torch.tanh(z[2])
            hv = torch.sigmoid(z[3]) * torch.tanh(cn)
            cc[b].copy_(cn)
            hs[b].copy_(hv.to(hs.dtype))
            if hn is not None:
                hn[b].copy_(hv.to(hn.dtype))
        return
    _require(cc.is_contiguous() and g.stride(1) == 1 and hs.stride(1) == 1 and (hn is None or hn.stride(1) == 1)
             and (st is None or st.is_contiguous()), "lstm_cell: layout")
    rc = kernels().ff_lstm_cell(ptr(g), ptr(bias), ptr(cc), ptr(hs), ptr(hn), ptr(st), batch, hd, g.stride(0), hs.stride(0),
                                hn.stride(0) if hn is not None else hd, stream_ptr())
    check(rc, "ff_lstm_cell")
    _count()


def tdt_joint_in(enc: torch.Tensor, pred: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor,
                 out: torch.Tensor) -> None:
    """``out[b] = bf16(relu(enc[b, state[b].frame] + pred[b] + bias))``: the joint network's hidden vector of this step.
    ``enc``: [batch, frames, J] (or [frames, J] for one utterance)."""
    e = enc if enc.dim() == 3 else enc[None]
    pr, st, o = _rows(pred), _rows(state), _rows(out)
    batch, frames, j = e.shape
    if not e.is_cuda:
        for b in range(batch):
            f = min(max(int(st[b, TS_FRAME]), 0), frames - 1)
            x = e[b, f].float() + pr[b].float() + (bias.float() if bias is not None else 0.0)
            o[b].copy_(torch.relu(x).to(o.dtype))
        return
    _require(e.is_contiguous() and pr.stride(1) == 1 and o.stride(1) == 1 and st.is_contiguous(), "tdt_joint_in: layout")
    rc = kernels().ff_tdt_joint_in(ptr(e), ptr(pr), ptr(bias), ptr(st), ptr(o), batch, j, frames, pr.stride(0), o.stride(0), stream_ptr())
    check(rc, "ff_tdt_joint_in")
    _count()


def tdt_select(logits: torch.Tensor, out_bias: torch.Tensor | None, durations: torch.Tensor, state: torch.Tensor,
               traj: tuple[torch.Tensor, torch.Tensor, torch.Tensor], n_tok: int, blank: int, eos: int) -> None:
    """Greedy selection of one step per utterance and the state update: token = argmax of the first ``n_tok`` logits
    (lowest index on ties), duration = ``durations[argmax of the rest]``, a blank with duration 0 advances one frame and
    so does the ``TS_MAXSYM``-th consecutive token that would stay on its frame; the (token, duration, frame) entry is
    appended to ``traj`` (three [batch, capacity] int32 tensors) and the state moves to the next frame, or ``done`` is set
    on the end-of-sequence token or when the frames (state word ``TS_VALID``) are used up. A trajectory longer than
    ``TS_CAP`` entries sets the error word. An empty ``durations`` selects the plain transducer rule: a token stays on its
    frame, a blank moves one frame."""
    n_dur = durations.numel()
    lg, st = _rows(logits), _rows(state)
    tr = tuple(_rows(t) for t in traj)
    traj_len = tr[0].shape[1]
    if not lg.is_cuda:
        for b in range(st.shape[0]):
            s1 = st[b]
            if int(s1[TS_DONE]):
                continue
            x = lg[b].float().reshape(-1)[: n_tok + n_dur]
            if out_bias is not None:
                x = x + out_bias.float()[: n_tok + n_dur]
            tok = int(torch.argmax(x[:n_tok]))
            dur = int(durations[int(torch.argmax(x[n_tok:n_tok + n_dur]))]) if n_dur > 0 else 0
            count, frame = int(s1[TS_COUNT]), int(s1[TS_FRAME])
            valid_rows, capacity = int(s1[TS_VALID]), min(int(s1[TS_CAP]), traj_len)
            if count >= capacity:
                s1[TS_ERROR] = 1
                s1[TS_DONE] = 1
                continue
            if tok == blank and dur == 0:
                dur = 1
            syms = int(s1[TS_SYMS])
            if tok != blank and dur == 0:
                syms += 1
                if syms >= int(s1[TS_MAXSYM]):
                    dur = 1
            s1[TS_SYMS] = 0 if dur > 0 else syms
            tr[0][b, count], tr[1][b, count], tr[2][b, count] = tok, dur, frame
            s1[TS_COUNT] = count + 1
            nxt = frame + dur
            s1[TS_FRAME], s1[TS_TOKEN], s1[TS_ADVANCE] = nxt, tok, int(tok != blank)
            if tok == eos or nxt >= valid_rows:
                s1[TS_DONE] = 1
        return
    _require(st.is_contiguous() and lg.stride(1) == 1 and all(t.is_contiguous() for t in tr), "tdt_select: layout")
    rc = kernels().ff_tdt_select(ptr(lg), ptr(out_bias), ptr(durations), ptr(st), ptr(tr[0]), ptr(tr[1]), ptr(tr[2]), st.shape[0],
                                 n_tok, n_dur, blank, eos, traj_len, lg.stride(0), stream_ptr())
    check(rc, "ff_tdt_select")
    _count()


def ctc_collapse(ids: torch.Tensor, valid: int, blank: int) -> tuple[list[int], list[int], list[int]]:
    """Greedy CTC path -> (tokens, first frame, frames held): repeats merge, blanks drop. ``ids``: [frames] arg-max ids."""
    path = ids[:valid].tolist()
    tokens, starts, runs = [], [], []
    prev = None
    for f, t in enumerate(path):
        if t != prev and t != blank:
            tokens.append(t)
            starts.append(f)
            runs.append(1)
        elif t == prev and t != blank:
            runs[-1] += 1
        prev = t
    return tokens, starts, runs
