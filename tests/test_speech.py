"""Speech family on the CPU path: audio input, log-mel features, the FastConformer encoder against a plain PyTorch
model in the published (channels-first, un-fused) layout, the transducer state machine, transcripts, configuration and
the checkpoint contract."""
import json
import math

import pytest
import torch
import torch.nn.functional as F

from flyingfish_b200.loaders.safetensors_io import save_safetensors
from flyingfish_b200.models.conformer import ConformerEncoder, random_tensors
from flyingfish_b200.ops import speech_ops
from flyingfish_b200.ops.speech_ops import (TS_ADVANCE, TS_CAP, TS_COUNT, TS_DONE, TS_ERROR, TS_FRAME, TS_MAXSYM, TS_TOKEN,
                                           TS_VALID, TS_WORDS)
from flyingfish_b200.speech import (LogMel, LogMelConfig, ParakeetModel, ParakeetSpec, TextSegment, Transcription,
                                    parakeet_tiny, read_wav, resample, tdt_cues, word_segments, write_wav)
from flyingfish_b200.speech.audio import AudioError, load_audio, mix_down


# ------------------------------------------------------------------------------------------------
# audio input
# ------------------------------------------------------------------------------------------------
def test_wav_round_trip_and_formats(tmp_path):
    t = torch.arange(1600) / 16000.0
    wave = torch.stack([0.5 * torch.sin(2 * math.pi * 440 * t), 0.25 * torch.cos(2 * math.pi * 220 * t)])
    write_wav(tmp_path / "a.wav", wave, 16000)
    back, rate = read_wav(tmp_path / "a.wav")
    assert rate == 16000 and back.shape == wave.shape
    assert (back - wave).abs().max() < 1.0 / 32768 + 1e-6
    assert torch.allclose(mix_down(back), back.mean(0))
    (tmp_path / "bad.wav").write_bytes(b"RIFFxxxxWAVX")
    with pytest.raises(AudioError):
        read_wav(tmp_path / "bad.wav")
    # 32-bit float data chunk
    import struct
    pcm = wave[0].numpy().astype("float32").tobytes()
    hdr = b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 3, 1, 8000, 32000, 4, 32)
    (tmp_path / "f.wav").write_bytes(hdr + b"data" + struct.pack("<I", len(pcm)) + pcm)
    f32, r2 = read_wav(tmp_path / "f.wav")
    assert r2 == 8000 and torch.equal(f32[0], wave[0])


def test_resample_keeps_a_tone(tmp_path):
    rate_in, rate_out, hz = 44100, 16000, 1000.0
    t = torch.arange(rate_in // 2) / rate_in
    tone = torch.sin(2 * math.pi * hz * t)
    out = resample(tone, rate_in, rate_out)
    assert abs(out.numel() - rate_out // 2) <= 1
    t2 = torch.arange(out.numel()) / rate_out
    want = torch.sin(2 * math.pi * hz * t2)
    assert (out[200:-200] - want[200:-200]).abs().max() < 2e-2
    # a tone above the new Nyquist frequency is removed
    high = torch.sin(2 * math.pi * 15000.0 * t)
    assert resample(high, rate_in, rate_out)[200:-200].abs().max() < 5e-2
    write_wav(tmp_path / "t.wav", tone, rate_in)
    assert abs(load_audio(tmp_path / "t.wav").numel() - rate_out // 2) <= 1


# ------------------------------------------------------------------------------------------------
# log-mel
# ------------------------------------------------------------------------------------------------
def _naive_logmel(x, cfg, window, filters):
    n, hop, nfft = x.numel(), cfg.hop_length, cfg.n_fft
    valid = n // hop
    em = x.double().clone()
    em[1:] = x[1:].double() - cfg.preemphasis * x[:-1].double()
    k = torch.arange(nfft // 2 + 1, dtype=torch.float64)
    i = torch.arange(nfft, dtype=torch.float64)
    dft = torch.exp(-2j * math.pi * k[:, None] * i[None, :] / nfft)
    feats = []
    for t in range(valid):
        frame = torch.zeros(nfft, dtype=torch.float64)
        for j in range(nfft):
            pos = t * hop + j - nfft // 2
            if 0 <= pos < n:
                frame[j] = em[pos]
        spec = dft @ (frame * window.double()).to(torch.complex128)
        power = spec.real ** 2 + spec.imag ** 2
        feats.append(torch.log(filters.double() @ power + cfg.log_guard))
    feat = torch.stack(feats)
    mean = feat.mean(0)
    std = torch.sqrt(((feat - mean) ** 2).sum(0) / (valid - 1))
    return ((feat - mean) / (std + cfg.norm_eps)).float()


def test_logmel_matches_a_direct_dft():
    cfg = LogMelConfig(n_fft=64, win_length=50, hop_length=20, mel_bins=12, sampling_rate=8000)
    g = torch.Generator().manual_seed(1)
    a, b = torch.randn(415, generator=g), torch.randn(260, generator=g)
    mel = LogMel(cfg)
    feat, valid = mel.extract([a, b])
    assert feat.shape == (2, 415 // 20 + 1, 12) and valid.tolist() == [20, 13]
    for x, row, n in ((a, 0, 20), (b, 1, 13)):
        want = _naive_logmel(x, cfg, mel.window, mel.filters)
        assert (feat[row, :n] - want).abs().max() < 2e-3
        assert feat[row, n:].abs().max() == 0
    with pytest.raises(AudioError):
        mel.extract([torch.zeros(30)])
    with pytest.raises(AudioError):
        LogMel(LogMelConfig(n_fft=500))


def test_filterbank_and_window_shape():
    fb = speech_ops.mel_filterbank(16000, 512, 128)
    assert fb.shape == (128, 257) and (fb >= 0).all()
    peak = fb.argmax(dim=1)
    assert (peak[1:] >= peak[:-1]).all() and peak[0] >= 1 and peak[-1] <= 256
    # Slaney scale: below 1 kHz the band centres are evenly spaced in Hz
    low = peak[:20].float() * 16000 / 512
    assert (low[1:] - low[:-1]).std() < 20.0
    rng = speech_ops.band_ranges(fb)
    for m in (0, 64, 127):
        lo, hi = rng[m].tolist()
        assert fb[m, :lo].abs().sum() == 0 and fb[m, hi:].abs().sum() == 0 and fb[m, lo] > 0 and fb[m, hi - 1] > 0
    w = speech_ops.hann_window(400, 512)
    assert w[:56].abs().sum() == 0 and w[56 + 400:].abs().sum() == 0 and abs(float(w[56 + 199]) - 1.0) < 1e-3
    assert torch.allclose(w[56:456], torch.flip(w[56:456], [0]), atol=1e-6)


def test_relative_positions_are_signed_and_interleaved():
    tab = speech_ops.relative_positions(4, 8)
    assert tab.shape == (7, 8)
    assert torch.allclose(tab[3], torch.tensor([0.0, 1.0] * 4))                  # offset 0
    assert torch.allclose(tab[0, 0], torch.sin(torch.tensor(3.0))) and torch.allclose(tab[0, 1], torch.cos(torch.tensor(3.0)))
    assert torch.allclose(tab[6, 0], torch.sin(torch.tensor(-3.0)))
    assert torch.allclose(tab[2, 2], torch.sin(torch.tensor(1.0 / 10000 ** (2 / 8))))
    assert speech_ops.conv_out_len(128, 1, 1) == 64 and speech_ops.conv_out_len(5, 1, 1) == 3
    with pytest.raises(ValueError):
        speech_ops.conv_out_len(0, 1, 1)


# ------------------------------------------------------------------------------------------------
# encoder against a plain PyTorch model in the published layout
# ------------------------------------------------------------------------------------------------
def _rel_shift(x):
    b, h, t, c = x.shape                                # c = 2t - 1, column = relative row index
    x = F.pad(x, (1, 0)).reshape(b, h, c + 1, t)[:, :, 1:].reshape(b, h, t, c)
    return x[..., :t]


def _plain_encoder(spec, tensors, feat, valid):
    """FP32, channels-first, un-fused: convolutions through conv2d / conv1d, explicit batch norm, the pad-and-reshape
    relative shift."""
    W = {k: v.float() for k, v in tensors.items() if v.dtype != torch.int64}
    p = spec.prefix
    b = feat.shape[0]
    x = feat[:, None]                                    # [B, 1, T, F]
    v = list(valid)

    def tmask(x, v):
        m = torch.arange(x.shape[2])[None, :] < torch.tensor(v)[:, None]
        return x * m[:, None, :, None]

    names = spec.conv_names
    x = F.conv2d(x, W[f"{p}.{names[0]}.weight"], W[f"{p}.{names[0]}.bias"], stride=2, padding=1)
    v = [speech_ops.conv_out_len(n, 1, 1) for n in v]
    x = torch.relu(tmask(x, v))
    for i in (1, 2):
        c = spec.sub_channels
        x = F.conv2d(x, W[f"{p}.{names[i]}.weight"], W[f"{p}.{names[i]}.bias"], stride=2, padding=1, groups=c)
        pw = spec.pointwise_names[i - 1]
        x = F.conv2d(x, W[f"{p}.{pw}.weight"], W[f"{p}.{pw}.bias"])
        v = [speech_ops.conv_out_len(n, 1, 1) for n in v]
        x = torch.relu(tmask(x, v))
    t = x.shape[2]
    x = x.permute(0, 2, 1, 3).reshape(b, t, -1)          # [B, T, C * F]
    h = x @ W[f"{p}.{spec.linear_name}.weight"].t() + W[f"{p}.{spec.linear_name}.bias"]
    lens = torch.tensor(v)
    key_ok = torch.arange(t)[None, :] < lens[:, None]
    pos = speech_ops.relative_positions(t, spec.hidden)
    hd, nh = spec.head_dim, spec.heads
    for li in range(spec.layers):
        q = f"{p}.layers.{li}"
        ln = lambda x, n: F.layer_norm(x, (spec.hidden,), W[f"{q}.{n}.weight"], W[f"{q}.{n}.bias"], 1e-5)
        ff = lambda x, br: F.silu(x @ W[f"{q}.{br}.linear1.weight"].t()) @ W[f"{q}.{br}.linear2.weight"].t()
        h = h + 0.5 * ff(ln(h, "norm_feed_forward1"), "feed_forward1")
        x = ln(h, "norm_self_att")
        a = f"{q}.self_attn"
        qq = (x @ W[f"{a}.q_proj.weight"].t()).reshape(b, t, nh, hd)
        kk = (x @ W[f"{a}.k_proj.weight"].t()).reshape(b, t, nh, hd)
        vv = (x @ W[f"{a}.v_proj.weight"].t()).reshape(b, t, nh, hd)
        pp = (pos @ W[f"{a}.relative_k_proj.weight"].t()).reshape(2 * t - 1, nh, hd)
        ac = torch.einsum("bihd,bjhd->bhij", qq + W[f"{a}.bias_u"], kk)
        bd = _rel_shift(torch.einsum("bihd,chd->bhic", qq + W[f"{a}.bias_v"], pp))
        sc = ((ac + bd) / math.sqrt(hd)).masked_fill(~key_ok[:, None, None, :], float("-inf"))
        o = torch.einsum("bhij,bjhd->bihd", torch.softmax(sc, -1), vv).reshape(b, t, spec.hidden)
        h = h + o @ W[f"{a}.o_proj.weight"].t()
        x = ln(h, "norm_conv").transpose(1, 2)           # [B, H, T]
        cv = f"{q}.conv"
        x = F.glu(F.conv1d(x, W[f"{cv}.pointwise_conv1.weight"]), dim=1)
        x = x * key_ok[:, None, :]
        x = F.conv1d(x, W[f"{cv}.depthwise_conv.weight"], padding=spec.conv_kernel // 2, groups=spec.hidden)
        x = F.batch_norm(x, W[f"{cv}.norm.running_mean"], W[f"{cv}.norm.running_var"], W[f"{cv}.norm.weight"],
                         W[f"{cv}.norm.bias"], False, 0.0, 1e-5)
        x = F.conv1d(F.silu(x), W[f"{cv}.pointwise_conv2.weight"]).transpose(1, 2)
        h = h + x
        h = h + 0.5 * ff(ln(h, "norm_feed_forward2"), "feed_forward2")
        h = ln(h, "norm_out")
    return h, v


def test_encoder_matches_the_plain_model():
    spec = parakeet_tiny().encoder
    tensors = random_tensors(spec.expected_tensors(), seed=3)
    # weights as the BF16 GEMMs see them, so that the comparison measures the pipeline and not the rounding of weights
    tensors = {k: (v.to(torch.bfloat16).float() if v.dtype == torch.float32 and v.dim() >= 2 else v) for k, v in tensors.items()}
    g = torch.Generator().manual_seed(4)
    feat = torch.randn(2, 131, spec.mel_bins, generator=g)
    valid = [131, 77]
    feat[1, 77:] = 0
    enc = ConformerEncoder(spec, tensors)
    got, rows = enc.encode(feat, valid)
    want, rows2 = _plain_encoder(spec, tensors, feat, valid)
    assert rows == rows2 == [spec.sub_len(131), spec.sub_len(77)]
    assert got.shape == want.shape
    for b, n in enumerate(rows):
        err = (got[b, :n].float() - want[b, :n]).abs()
        assert err.max() < 0.12 and err.mean() < 0.02, (float(err.max()), float(err.mean()))


def test_relpos_attention_oracle_against_loops():
    g = torch.Generator().manual_seed(5)
    b, t, h, d = 2, 7, 2, 8
    q, k, v = (torch.randn(b * t, h * d, generator=g).to(torch.bfloat16) for _ in range(3))
    pos = torch.randn(2 * t - 1, h * d, generator=g).to(torch.bfloat16)
    u, vb = torch.randn(h, d, generator=g), torch.randn(h, d, generator=g)
    lens = torch.tensor([7, 4], dtype=torch.int32)
    got = speech_ops.relpos_attention(q, k, v, pos, u, vb, lens, b, h, left=3, right=1).float().reshape(b, t, h, d)
    r = lambda x: x.to(torch.bfloat16).float()
    for bi in range(b):
        for hi in range(h):
            for i in range(t):
                if i >= int(lens[bi]):
                    assert got[bi, i, hi].abs().sum() == 0
                    continue
                qi = q.float().reshape(b, t, h, d)[bi, i, hi]
                sc, vals = [], []
                for j in range(int(lens[bi])):
                    if j < i - 3 or j > i + 1:
                        continue
                    kj = k.float().reshape(b, t, h, d)[bi, j, hi]
                    pj = pos.float().reshape(2 * t - 1, h, d)[t - 1 - i + j, hi]
                    sc.append((r(qi + u[hi]) @ kj + r(qi + vb[hi]) @ pj) / math.sqrt(d))
                    vals.append(v.float().reshape(b, t, h, d)[bi, j, hi])
                w = torch.softmax(torch.stack(sc), 0)
                want = (w[:, None] * torch.stack(vals)).sum(0)
                assert (got[bi, i, hi] - want).abs().max() < 2e-2


# ------------------------------------------------------------------------------------------------
# transducer state machine
# ------------------------------------------------------------------------------------------------
def _run_script(script, valid_rows, capacity, n_tok=6, blank=5, eos=3, durations=(0, 1, 2, 3, 4), max_symbols=10):
    state = torch.zeros(TS_WORDS, dtype=torch.int32)
    state[TS_TOKEN], state[TS_COUNT], state[TS_ADVANCE], state[TS_VALID], state[TS_CAP] = blank, 1, 1, valid_rows, capacity
    state[TS_MAXSYM] = max_symbols
    traj = tuple(torch.zeros(64, dtype=torch.int32) for _ in range(3))
    traj[0][0] = blank
    dur = torch.tensor(durations, dtype=torch.int32)
    advanced = []
    for tok, di in script:
        advanced.append(int(state[TS_ADVANCE]))
        logits = torch.zeros(n_tok + len(durations))
        logits[tok] = 5.0
        if durations:
            logits[n_tok + di] = 5.0
        speech_ops.tdt_select(logits.to(torch.bfloat16), None, dur, state, traj, n_tok, blank, eos)
    n = int(state[TS_COUNT])
    return state, [t[:n].tolist() for t in traj], advanced


def test_tdt_duration_and_capacity_rules():
    # token with duration 2, blank with duration 0 (moves one frame), token with duration 0 (stays), blank 4 -> past the end
    state, (tok, dur, frm), adv = _run_script([(1, 2), (5, 0), (2, 0), (4, 1), (5, 4), (1, 1)], valid_rows=6, capacity=60)
    assert tok == [5, 1, 5, 2, 4, 5] and dur == [0, 2, 1, 0, 1, 4] and frm == [0, 0, 2, 3, 3, 4]
    assert int(state[TS_DONE]) == 1 and int(state[TS_ERROR]) == 0
    assert adv[:5] == [1, 1, 0, 1, 1]                    # the prediction network only advances after a non-blank token
    # end-of-sequence token stops at once
    state, (tok, _, _), _ = _run_script([(1, 1), (3, 1), (2, 1)], valid_rows=50, capacity=60)
    assert tok == [5, 1, 3] and int(state[TS_DONE]) == 1
    # a token that never moves on exhausts the capacity and raises the error word
    state, (tok, _, _), _ = _run_script([(1, 0)] * 8, valid_rows=50, capacity=5)
    assert int(state[TS_ERROR]) == 1 and int(state[TS_DONE]) == 1 and len(tok) == 5
    # the third token in a row that would stay on its frame moves one frame on (symbols-per-step limit)
    state, (tok, dur, frm), _ = _run_script([(1, 0), (2, 0), (1, 0), (2, 0), (5, 1), (1, 0)], valid_rows=50, capacity=60, max_symbols=3)
    assert dur == [0, 0, 0, 1, 0, 1, 0] and frm == [0, 0, 0, 0, 1, 1, 2]
    # lowest index wins ties
    st = torch.zeros(TS_WORDS, dtype=torch.int32)
    st[TS_TOKEN], st[TS_COUNT], st[TS_VALID], st[TS_CAP], st[TS_MAXSYM] = 5, 1, 10, 10, 10
    traj = tuple(torch.zeros(8, dtype=torch.int32) for _ in range(3))
    speech_ops.tdt_select(torch.zeros(11).to(torch.bfloat16), None, torch.tensor([0, 1, 2, 3, 4], dtype=torch.int32), st, traj, 6, 5, 3)
    assert int(traj[0][1]) == 0 and int(traj[1][1]) == 0


def test_lstm_cell_matches_torch():
    g = torch.Generator().manual_seed(6)
    hd = 16
    cell = torch.nn.LSTMCell(hd, hd)
    x, h0, c0 = torch.randn(hd, generator=g), torch.randn(hd, generator=g), torch.randn(hd, generator=g)
    with torch.no_grad():
        hn, cn = cell(x[None], (h0[None], c0[None]))
        w = torch.cat([cell.weight_ih, cell.weight_hh], dim=1)
        gates = w @ torch.cat([x, h0])
        c = c0.clone()
        h_self, h_next = torch.zeros(hd), torch.zeros(hd)
        speech_ops.lstm_cell(gates, cell.bias_ih + cell.bias_hh, c, h_self, h_next, None)
    assert torch.allclose(c, cn[0], atol=1e-5) and torch.allclose(h_self, hn[0], atol=1e-5) and torch.equal(h_self, h_next)
    # a step that does not advance leaves the state alone
    st = torch.zeros(TS_WORDS, dtype=torch.int32)
    before = c.clone()
    speech_ops.lstm_cell(gates, cell.bias_ih + cell.bias_hh, c, h_self, h_next, st)
    assert torch.equal(c, before)


def test_model_decodes_and_checkpoint_round_trip(tmp_path):
    spec = parakeet_tiny()
    model = ParakeetModel.random(spec, seed=7)
    g = torch.Generator().manual_seed(8)
    waves = [0.1 * torch.randn(16000, generator=g), 0.1 * torch.randn(9000, generator=g)]
    trajs = model.decode(waves)
    for tr, n in zip(trajs, (16000, 9000)):
        rows = spec.encoder.sub_len(n // 160)
        assert tr.tokens[0] == spec.blank and tr.durations[0] == 0 and tr.capacity == spec.max_symbols * rows + 1
        assert len(tr.tokens) == len(tr.durations) == len(tr.frames) <= tr.capacity
        assert all(b >= a for a, b in zip(tr.frames, tr.frames[1:])) and tr.frames[-1] < rows
        assert all(0 <= t < spec.vocab for t in tr.tokens)
        for (f0, d0), f1 in zip(zip(tr.frames[1:], tr.durations[1:]), tr.frames[2:]):
            assert f1 == f0 + d0
    # the same model through the published files
    d = tmp_path / "ckpt"
    d.mkdir()
    root, processor, generation = spec.to_json()
    for name, obj in (("config.json", root), ("processor_config.json", processor), ("generation_config.json", generation)):
        (d / name).write_text(json.dumps(obj))
    tensors = random_tensors(spec.expected_tensors(), 7)
    save_safetensors(d / "model.safetensors", tensors)
    assert ParakeetSpec.read(d) == spec
    loaded = ParakeetModel.load(d)
    again = loaded.decode(waves)
    assert [t.tokens for t in again] == [t.tokens for t in trajs] and [t.durations for t in again] == [t.durations for t in trajs]
    # contract violations are named
    table = {n: (dt, sh) for n, (dt, sh) in spec.expected_tensors().items()}
    assert spec.validate(table) == len(table)
    missing = dict(table); missing.pop("joint.head.bias")
    with pytest.raises(ValueError, match="missing: joint.head.bias"):
        spec.validate(missing)
    extra = dict(table); extra["encoder.extra"] = ("F32", (1,))
    with pytest.raises(ValueError, match="unexpected: encoder.extra"):
        spec.validate(extra)
    wrong = dict(table); wrong["joint.head.weight"] = ("F32", (3, 3))
    with pytest.raises(ValueError, match="mismatch: joint.head.weight"):
        spec.validate(wrong)


def test_published_geometry_and_config_checks():
    spec = ParakeetSpec()
    assert spec.encoder.linear_in == 4096 and spec.encoder.head_dim == 128 and spec.joint_out == 8198
    assert abs(spec.frame_seconds - 0.08) < 1e-12
    exp = spec.expected_tensors()
    assert exp["encoder.subsampling.linear.weight"] == ("F32", (1024, 4096))
    assert exp["encoder.layers.23.conv.depthwise_conv.weight"] == ("F32", (1024, 1, 9))
    assert exp["decoder.lstm.weight_hh_l1"] == ("F32", (2560, 640)) and exp["joint.head.weight"] == ("F32", (8198, 640))
    root, processor, generation = spec.to_json()
    assert ParakeetSpec.from_json(root, processor, generation) == spec
    bad = dict(root); bad["model_type"] = "whisper"
    with pytest.raises(ValueError):
        ParakeetSpec.from_json(bad, processor, generation)
    bad_enc = json.loads(json.dumps(root)); bad_enc["encoder_config"]["subsampling_factor"] = 4
    with pytest.raises(ValueError):
        ParakeetSpec.from_json(bad_enc, processor, generation)


# ------------------------------------------------------------------------------------------------
# transcripts
# ------------------------------------------------------------------------------------------------
def test_cues_use_durations_and_previous_token_punctuation():
    tokens = [8192, 10, 11, 12, 2, 13, 14, 15, 16, 17, 18]
    durations = [0, 2, 1, 1, 0, 1, 1, 1, 2, 1, 1]
    table = {(10,): "hello", (11,): " wo", (12,): "rld", (13,): ".", (14,): " Next", (15,): " sentence", (16,): "!",
             (17,): "'", (18,): "cause", tuple(tokens): "hello world. Next sentence!'cause"}
    calls = []

    def decode(ids):
        calls.append(tuple(ids))
        return table.get(tuple(ids), "")

    res = tdt_cues(tokens, durations, 8192, decode, lambda t: t == 17)
    assert res.text == "hello world. Next sentence!'cause" and len(calls) == 10
    got = [(w.text, round(w.start, 6), round(w.end, 6)) for w in res.words]
    assert got == [("hello", 0.0, 0.16), ("world.", 0.16, 0.32), ("Next", 0.4, 0.48), ("sentence!", 0.48, 0.56), ("'cause", 0.72, 0.88)]
    segs = [(s.text, round(s.start, 6), round(s.end, 6)) for s in res.segments]
    assert segs == [("hello world.", 0.0, 0.32), ("Next sentence!", 0.4, 0.56), ("'cause", 0.72, 0.88)]
    _, undelimited = word_segments([(False, TextSegment(0.0, 0.08, "hello")), (False, TextSegment(0.08, 0.16, " world"))])
    assert len(undelimited) == 1 and undelimited[0].text == "hello world" and (undelimited[0].start, undelimited[0].end) == (0.0, 0.16)
    t2 = {(20,): "hello", (21,): " ", (22,): "world", (8192, 20, 21, 22): "hello world"}
    res2 = tdt_cues([8192, 20, 21, 22], [0, 1, 1, 1], 8192, lambda ids: t2.get(tuple(ids), ""), lambda t: t == 21)
    assert [w.text for w in res2.words] == ["hello", "world"] and len(res2.segments) == 1
    assert (round(res2.words[1].start, 6), round(res2.words[1].end, 6)) == (0.16, 0.24)
    with pytest.raises(ValueError):
        tdt_cues([1, 2], [1], 0, lambda ids: "", lambda t: False)


def test_transcription_writers():
    tr = Transcription("a b. c", [TextSegment(0.0, 1.5, "a b."), TextSegment(3661.25, 3662.0, "c")], [])
    srt = tr.to_srt()
    assert "1\n00:00:00,000 --> 00:00:01,500\na b.\n" in srt and "2\n01:01:01,250 --> 01:01:02,000\nc\n" in srt
    assert tr.to_vtt().startswith("WEBVTT\n") and "01:01:01.250 --> 01:01:02.000" in tr.to_vtt()
    assert json.loads(tr.to_json())["segments"][1]["text"] == "c"
    whole = Transcription.whole_clip("hi", 2.0)
    assert whole.segments[0].end == 2.0
    with pytest.raises(ValueError):
        Transcription.whole_clip("hi", float("nan"))


# ------------------------------------------------------------------------------------------------
# command line
# ------------------------------------------------------------------------------------------------
def _write_model_dir(d, spec, seed):
    from tokenizers import Tokenizer, decoders, models
    d.mkdir()
    root, processor, generation = spec.to_json()
    for name, obj in (("config.json", root), ("processor_config.json", processor), ("generation_config.json", generation)):
        (d / name).write_text(json.dumps(obj))
    save_safetensors(d / "model.safetensors", random_tensors(spec.expected_tensors(), seed))
    pieces = ["<unk>", "<s>", "<pad>", "</s>"] + [("▁" if i % 3 == 0 else "") + chr(ord("a") + i % 26) * (1 + i % 2) for i in range(spec.vocab - 7)]
    pieces += [".", "?", "<blank>"]
    vocab = {}
    for i, p in enumerate(pieces):
        vocab.setdefault(p if p not in vocab else f"{p}{i}", i)
    assert len(vocab) == spec.vocab
    tk = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tk.decoder = decoders.Metaspace()
    tk.save(str(d / "tokenizer.json"))


def test_transcribe_command(tmp_path, capsys):
    from flyingfish_b200 import cli
    spec = parakeet_tiny()
    d = tmp_path / "asr"
    _write_model_dir(d, spec, 11)
    g = torch.Generator().manual_seed(12)
    write_wav(tmp_path / "in.wav", 0.2 * torch.randn(2, 22050, generator=g), 22050)
    assert cli.main(["--cpu", "--model", str(d), "transcribe", str(tmp_path / "in.wav"), "--format", "json"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert set(out) == {"text", "segments", "words"} and isinstance(out["text"], str)
    for w in out["words"]:
        assert w["end"] >= w["start"] >= 0 and w["text"] == w["text"].strip() and w["text"]
    model = ParakeetModel.load(d)
    direct = model.transcribe([load_audio(tmp_path / "in.wav")])[0]
    assert direct.text == out["text"] and len(direct.words) == len(out["words"])
    target = tmp_path / "out.srt"
    assert cli.main(["--cpu", "--model", str(d), "transcribe", str(tmp_path / "in.wav"), "--format", "srt", "--output", str(target)]) == 0
    assert target.read_text() == direct.to_srt()
    with pytest.raises(SystemExit, match="refusing to overwrite"):
        cli.main(["--cpu", "--model", str(d), "transcribe", str(tmp_path / "in.wav"), "--output", str(target)])
    with pytest.raises(SystemExit, match="streaming transcription is not available"):
        cli.main(["--cpu", "--model", str(d), "transcribe", str(tmp_path / "in.wav"), "--stream"])
    cfg = json.loads((d / "config.json").read_text())
    cfg["architectures"] = ["WhisperForConditionalGeneration"]
    (d / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(SystemExit, match="unsupported transcription architecture"):
        cli.main(["--cpu", "--model", str(d), "transcribe", str(tmp_path / "in.wav")])


def test_plain_transducer_and_ctc_variants(tmp_path):
    from dataclasses import replace
    from flyingfish_b200.speech import ParakeetCtcModel, ParakeetCtcSpec, load_model
    # RNN-T rule (no duration head): a token stays on its frame, a blank moves one frame
    state, (tok, dur, frm), _ = _run_script([(1, 0), (5, 0), (2, 0), (2, 0), (5, 0)], valid_rows=3, capacity=60, durations=())
    assert tok == [5, 1, 5, 2, 2, 5] and dur == [0, 0, 1, 0, 0, 1] and frm == [0, 0, 0, 1, 1, 1]
    spec = replace(parakeet_tiny(), durations=())
    assert spec.joint_out == spec.vocab
    g = torch.Generator().manual_seed(21)
    wave = 0.1 * torch.randn(12000, generator=g)
    tr = ParakeetModel.random(spec, seed=5).decode([wave])[0]
    assert all(d in (0, 1) for d in tr.durations) and tr.frames[-1] < spec.encoder.sub_len(75)
    # CTC: repeats merge, blanks drop, first frames and run lengths are kept
    ids = torch.tensor([4, 4, 9, 9, 9, 1, 1, 9, 2, 2, 4, 9])
    assert speech_ops.ctc_collapse(ids, 11, 9) == ([4, 1, 2, 4], [0, 5, 8, 10], [2, 2, 2, 1])
    cspec = ParakeetCtcSpec(encoder=parakeet_tiny().encoder, vocab=41, blank=40, mel=LogMelConfig(mel_bins=32))
    model = ParakeetCtcModel.random(cspec, seed=6)
    tokens, starts, runs = model.decode([wave])[0]
    assert len(tokens) == len(starts) == len(runs) and all(0 <= t < 40 for t in tokens)
    assert all(b >= a + r for a, r, b in zip(starts, runs, starts[1:]))
    # through files and the architecture switch
    d = tmp_path / "ctc"
    _write_model_dir(d, parakeet_tiny(), 6)
    cfg = json.loads((d / "config.json").read_text())
    cfg["architectures"] = ["ParakeetForCTC"]
    (d / "config.json").write_text(json.dumps(cfg))
    (d / "model.safetensors").unlink()
    save_safetensors(d / "model.safetensors", random_tensors(cspec.expected_tensors(), 6))
    loaded = load_model(d)
    assert isinstance(loaded, ParakeetCtcModel) and loaded.decode([wave])[0] == (tokens, starts, runs)
    res = loaded.transcribe([wave])[0]
    assert isinstance(res.text, str) and all(w.end >= w.start for w in res.words)


def test_speaker_segments_from_frame_logits():
    from flyingfish_b200.speech import speaker_segments
    hi, lo = 4.0, -4.0
    # frames x 2 speakers: speaker 0 active on frames 0-2 and 5; speaker 1 on frames 2-4
    rows = [[hi, lo], [hi, lo], [hi, hi], [lo, hi], [lo, hi], [hi, lo]]
    segs = speaker_segments(torch.tensor(rows), 2)
    assert [(s.text, s.start, s.end) for s in segs] == [("speaker_0", 0.0, 0.24), ("speaker_1", 0.16, 0.4), ("speaker_0", 0.4, 0.48)]
    masked = speaker_segments(torch.tensor(rows), 2, attention_mask=[True, True, False, True, True, True])
    assert [(s.text, s.start, s.end) for s in masked] == [("speaker_0", 0.0, 0.16), ("speaker_1", 0.24, 0.4), ("speaker_0", 0.4, 0.48)]
    assert speaker_segments([0.0, 0.0], 2, threshold=0.5) == []            # sigmoid(0) is not above the threshold
    for bad in (dict(logits=[1.0, 2.0, 3.0], speakers=2), dict(logits=[float("nan")], speakers=1), dict(logits=[1.0], speakers=0),
                dict(logits=[1.0], speakers=1, threshold=1.5), dict(logits=[1.0], speakers=1, frame_seconds=0.0),
                dict(logits=[1.0, 1.0], speakers=1, attention_mask=[True])):
        with pytest.raises(ValueError):
            speaker_segments(**bad)


def test_batched_decode_equals_one_by_one():
    spec = parakeet_tiny()
    model = ParakeetModel.random(spec, seed=15, max_batch=3)
    g = torch.Generator().manual_seed(16)
    rows = [torch.randn(n, spec.decoder_hidden, generator=g).to(torch.bfloat16) for n in (31, 12, 20, 7)]
    valid = [31, 9, 20, 7]
    dec = model.decoder
    together = dec.decode_batch(rows[:3], valid[:3])
    alone = [dec.decode(r, v) for r, v in zip(rows, valid)]
    for a, b in zip(together, alone):
        assert (a.tokens, a.durations, a.frames) == (b.tokens, b.durations, b.frames)
    with pytest.raises(ValueError):
        dec.decode_batch(rows, valid)                       # more utterances than the decoder's batch
    # the model batches by itself
    waves = [0.1 * torch.randn(n, generator=g) for n in (8000, 5000, 9000, 6000)]
    outs = model.decode(waves)
    assert len(outs) == 4 and all(o.tokens[0] == spec.blank for o in outs)


def test_inspect_reports_speech_checkpoints(tmp_path, capsys):
    from flyingfish_b200 import cli
    spec = parakeet_tiny()
    d = tmp_path / "asr"
    _write_model_dir(d, spec, 3)
    assert cli.main(["--model", str(d), "inspect"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["family"] == "speech" and out["architecture"] == "ParakeetForTDT" and out["tensors"] == out["expected_tensors"]
    assert out["spec"]["encoder"]["hidden"] == 128 and out["spec"]["durations"] == [0, 1, 2, 3, 4]


def test_rttm_lines():
    from flyingfish_b200.speech import speaker_segments, to_rttm
    # frames x 2 speakers at 10 ms: speaker 0 on frames 0-1, speaker 1 on frames 1-2, the last frame masked out
    logits = [4.0, -4.0, 4.0, 4.0, -4.0, 4.0, 4.0, 4.0]
    segs = speaker_segments(logits, 2, attention_mask=[True, True, True, False], threshold=0.5, frame_seconds=0.01)
    assert [(s.start, s.end, s.text) for s in segs] == [(0.0, 0.02, "speaker_0"), (0.01, 0.03, "speaker_1")]
    assert to_rttm("clip", segs) == ("SPEAKER clip 1 0.000 0.020 <NA> <NA> speaker_0 <NA> <NA>\n"
                                     "SPEAKER clip 1 0.010 0.020 <NA> <NA> speaker_1 <NA> <NA>\n")
    assert speaker_segments([0.0], 1, frame_seconds=0.01) == []
    with pytest.raises(ValueError):
        to_rttm("two words", segs)
