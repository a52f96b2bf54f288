"""Speaker diarization: configuration files, the encoder and head against a plain FP32 PyTorch model, the speaker
cache policy, the chunked offline and streaming drivers, and the command line."""
import json
import math

import pytest
import torch

from flyingfish_b200.speech import diarization as dz
from flyingfish_b200.speech.audio import write_wav

PUBLISHED_CONFIG = {
    "architectures": ["Nemotron3DiarizationForAudioFrameClassification"],
    "audio_config": {"attention_dropout": 0.0, "hidden_act": "gelu", "hidden_size": 512, "initializer_range": 0.02,
                     "intermediate_size": 2048, "max_position_embeddings": 5000, "model_type": "nemotron3_diarization_audio",
                     "num_attention_heads": 8, "num_hidden_layers": 31, "num_key_value_heads": 8, "num_mel_bins": 128,
                     "partial_rotary_factor": 1.0,
                     "rope_parameters": {"partial_rotary_factor": 1.0, "rope_theta": 10000.0, "rope_type": "default"},
                     "subsampling_factor": 8},
    "chunk_length": 340, "chunk_right_context": 40, "dtype": "float32", "fifo_length": 40,
    "head_config": {"audio_hidden_size": 512, "hidden_size": 192, "model_type": "", "num_speakers": 8, "subsampling_factor": 8},
    "initializer_range": 0.02, "model_type": "nemotron3_diarization", "speaker_cache_update_period": 300,
    "streaming_config": {"fifo_length": 264, "latest_frames_score_boost": 0.05, "min_positive_scores_rate": 0.5, "model_type": "",
                         "num_speakers": 8, "prediction_score_threshold": 0.25, "speaker_cache_length": 264,
                         "speaker_cache_silence_frames_per_speaker": 1, "speaker_cache_update_period": 222,
                         "strong_boost_rate": 0.75, "subsampling_factor": 8, "weak_boost_rate": 1.5},
}
PUBLISHED_PROCESSOR = {
    "feature_extractor": {"feature_extractor_type": "NemotronAsrStreamingFeatureExtractor", "feature_size": 128, "hop_length": 160,
                          "n_fft": 512, "padding_side": "right", "padding_value": 0.0, "preemphasis": 0.97,
                          "return_attention_mask": True, "sampling_rate": 16000, "win_length": 400},
    "processor_class": "Nemotron3DiarizationProcessor", "streaming_mode": "low_latency",
    "streaming_modes": {"low_latency": [9, 4], "ultra_low_latency": [3, 1], "very_low_latency": [6, 2]}, "subsampling_factor": 8,
}


def test_published_configuration():
    spec = dz.DiarizationSpec.from_json(PUBLISHED_CONFIG, PUBLISHED_PROCESSOR)
    assert (spec.hidden, spec.layers, spec.heads, spec.head_dim, spec.head_hidden, spec.speakers, spec.factor) == (512, 31, 8, 64, 192, 8, 8)
    assert spec.offline == dz.ChunkConfig(340, 40, 40, 300)
    assert spec.stream_config() == dz.ChunkConfig(9, 4, 264, 222)
    assert spec.stream_config("ultra_low_latency") == dz.ChunkConfig(3, 1, 264, 222)
    assert spec.cache.budget(8) == 32 and spec.cache.counts(8) == (16, 24, 48)
    assert spec.max_encoder_rows() == 264 + 40 + 340 + 40
    assert spec.frame_seconds == pytest.approx(0.01)
    assert not spec.mel.normalize
    assert len(spec.expected_tensors()) == 417                  # 31 x 13 per layer + 14
    root, processor = spec.to_json()
    again = dz.DiarizationSpec.from_json(root, processor)
    assert again == spec
    with pytest.raises(ValueError):
        spec.stream_config("no_such_mode")
    bad = json.loads(json.dumps(PUBLISHED_CONFIG))
    bad["head_config"]["subsampling_factor"] = 4
    with pytest.raises(ValueError):
        dz.DiarizationSpec.from_json(bad, PUBLISHED_PROCESSOR)
    bad = json.loads(json.dumps(PUBLISHED_CONFIG))
    bad["audio_config"]["max_position_embeddings"] = 600          # the offline window has 684 rows
    with pytest.raises(ValueError):
        dz.DiarizationSpec.from_json(bad, PUBLISHED_PROCESSOR)


def test_checkpoint_layout_is_checked():
    spec = dz.diarization_tiny()
    tensors = dz.random_tensors(spec)
    assert spec.validate(tensors) == len(spec.expected_tensors())
    swapped = dict(tensors)
    swapped["model.upsampler.conv.weight"] = tensors["model.upsampler.conv.weight"].transpose(1, 2).contiguous()
    with pytest.raises(ValueError):
        spec.validate(swapped)
    missing = dict(tensors)
    del missing["silence_embeds"]
    with pytest.raises(ValueError):
        spec.validate(missing)


def test_encoder_and_head_match_plain_model():
    spec = dz.diarization_tiny()
    tensors = dz.random_tensors(spec, 1)
    model = dz.DiarizationModel(spec, tensors)
    g = torch.Generator().manual_seed(3)
    feat = torch.randn(37, spec.mel.mel_bins, generator=g)
    got = model.frame_logits(feat, 30)                          # 10 rows, 8 of them valid
    assert got.shape == (40, spec.speakers)
    rounded = {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
    want = dz.reference_logits(spec, rounded, model.embed(feat).float(), 8)
    assert (got - want).abs().max() < 0.02 * want.abs().max() + 1e-3
    # the mask matters: all keys valid gives other logits
    other = dz.reference_logits(spec, rounded, model.embed(feat).float(), 10)
    assert (other - want).abs().max() > 1e-3


def test_cache_selection_keeps_each_speakers_best_rows():
    spec = dz.diarization_tiny()                                # 4 speakers, 16 cache rows, 1 silence row per speaker
    assert spec.cache.counts(4) == (1, 2, 4)
    frames = 20
    probs = torch.full((frames, 4), 0.02)
    probs[:10, 0] = torch.linspace(0.6, 0.95, 10)              # speaker 0 alone, ever more confident
    probs[10:, 1] = 0.9                                         # speaker 1 alone, flat
    probs[12, 0] = 0.9                                          # one overlapped row: scores lower for both
    pick = dz.select_cache_rows(spec, probs)
    assert len(pick) == 16
    assert pick.count(frames) == 4                              # one silence row per speaker slot
    # grouped by speaker, time order inside a group; the silent speakers' groups are only their silence row
    first_silence = pick.index(frames)
    group0 = pick[:first_silence]
    assert group0 == sorted(group0) and all(r < 10 or r == 12 for r in group0)
    rest = pick[first_silence + 1:]
    group1 = rest[:rest.index(frames)]
    assert group1 == sorted(group1) and all(r >= 10 for r in group1)
    assert rest[rest.index(frames):] == [frames] * 3
    assert len(group0) + len(group1) == 12
    # the least confident rows of speaker 0 are the ones dropped
    assert 9 in group0 and 8 in group0
    # nobody speaks: only silence rows
    assert dz.select_cache_rows(spec, torch.full((frames, 4), 0.1)) == [frames] * 16
    with pytest.raises(ValueError):
        dz.select_cache_rows(spec, torch.zeros(16, 4))


def test_cache_scores_follow_the_formula():
    spec = dz.diarization_tiny()
    cfg = spec.cache
    frames = 17
    probs = torch.full((frames, 4), 0.1)
    probs[3, 2] = 0.8
    pick = dz.select_cache_rows(spec, probs)
    # one scored row for speaker 2 -> it survives, in the third group (after two silence rows)
    assert pick[:3] == [frames, frames, 3]
    assert pick.count(frames) == 15
    # the score itself: log p - log(1 - p) + sum log(1 - p') - log 0.5, probabilities clamped at the threshold
    want = math.log(0.8) - math.log(cfg.threshold) + (math.log(cfg.threshold) + 3 * math.log(0.9)) - math.log(0.5)
    raw = dz.cache_scores(spec, probs, boosts=False)
    assert raw[3, 2].item() == pytest.approx(want, rel=1e-5) and want > 0
    assert torch.isinf(raw).sum() == frames * 4 - 1             # nobody else speaks anywhere
    boosted = dz.cache_scores(spec, probs)
    # row 3 lies inside the old cache (no recency bonus) and is both among the 2 strongest and the 4 best rows
    assert boosted[3, 2].item() == pytest.approx(want + 3 * math.log(2.0), rel=1e-5)
    # an overlapped row scores lower than a row where the speaker is alone, and a speaker with enough positive rows
    # drops the rows that score at or below zero
    probs2 = torch.full((frames, 4), 0.1)
    probs2[0, 0], probs2[1, 0], probs2[1, 1], probs2[2, 0] = 0.9, 0.9, 0.9, 0.55
    raw2 = dz.cache_scores(spec, probs2, boosts=False)
    assert raw2[1, 0] < raw2[0, 0]
    assert raw2[0, 0] > 0 and torch.isinf(raw2[2, 0])           # 0.55 against three 0.9 complements scores below zero
    # rows newer than the old cache get the recency bonus
    probs3 = torch.full((frames, 4), 0.1)
    probs3[16, 3] = 0.8
    assert dz.cache_scores(spec, probs3)[16, 3].item() == pytest.approx(want + cfg.latest_boost + 3 * math.log(2.0), rel=1e-5)


def test_speaker_memory_fills_pops_and_compresses():
    spec = dz.diarization_tiny()
    model = dz.DiarizationModel.random(spec, seed=2)
    cfg = dz.ChunkConfig(frames=5, right=2, fifo=10, update=6)
    state = model.new_state(cfg)
    g = torch.Generator().manual_seed(0)
    sizes = []
    for step in range(9):
        rows = model.embed(torch.randn((cfg.frames + cfg.right) * spec.factor, spec.mel.mel_bins, generator=g))
        logits = model.step(state, rows, [True] * rows.shape[0], cfg.frames)
        assert logits.shape == (cfg.frames * spec.factor, spec.speakers)
        sizes.append((state.cache.shape[0], state.fifo.shape[0]))
        assert state.cache.shape[0] <= spec.cache.frames and state.fifo.shape[0] <= cfg.fifo
        assert state.probs.shape == (state.cache.shape[0], spec.speakers)
    # FIFO fills (5, 10), overflows at 15 -> max(update, 5) = 6 rows move to the cache, and so on
    assert sizes[:4] == [(0, 5), (0, 10), (6, 9), (12, 8)]
    # 12 + 6 = 18 > 16 rows: the cache is compressed to its capacity and stays there
    assert sizes[4] == (16, 7) and state.compressed and state.updates >= 1
    assert all(c == 16 for c, _ in sizes[4:])
    # a window that is too long for the rotary table is refused
    with pytest.raises(ValueError):
        model.encode(torch.zeros(spec.max_encoder_rows() + 1, spec.hidden, dtype=torch.bfloat16), 1)
    # holes in the mask are refused
    rows = model.embed(torch.randn(7 * spec.factor, spec.mel.mel_bins, generator=g))
    with pytest.raises(ValueError):
        model.step(state, rows, [True, False, True, True, True, True, True], 5)


def test_offline_short_clip_equals_one_window_and_long_clip_chunks():
    spec = dz.diarization_tiny()
    model = dz.DiarizationModel.random(spec, seed=4)
    g = torch.Generator().manual_seed(1)
    short = torch.randn(41, spec.mel.mel_bins, generator=g)     # 11 rows <= one chunk of 12
    a = model.offline(short)
    b = model.frame_logits(short)[:41]
    assert a.shape == (41, spec.speakers) and torch.equal(a, b)
    long = torch.randn(50 * spec.factor + 3, spec.mel.mel_bins, generator=g)     # 51 rows: five chunks
    before = model.encoder_calls
    out = model.offline(long)
    assert out.shape == (long.shape[0], spec.speakers) and torch.isfinite(out).all()
    assert model.encoder_calls - before == 5
    assert model.last_state.cache.shape[0] == spec.cache.frames and model.last_state.compressed
    # the first chunk sees only itself and its look-ahead
    first = model.frame_logits(long[: (12 + 3) * spec.factor])[: 12 * spec.factor]
    assert torch.equal(out[: 12 * spec.factor], first)


def test_streaming_emits_every_frame_once():
    spec = dz.diarization_tiny()
    model = dz.DiarizationModel.random(spec, seed=5)
    g = torch.Generator().manual_seed(2)
    wave = torch.randn(spec.mel.hop_length * 131 + 7, generator=g) * 0.1
    feat, lens = model.mel.extract([wave], normalize=False)
    n = int(lens[0])
    st = model.stream()
    pieces = []
    block = spec.mel.hop_length * 9 + 5
    for off in range(0, wave.numel(), block):
        pieces.append(st.push(wave[off:off + block], last=off + block >= wave.numel()))
    logits = torch.cat(pieces, 0)
    assert logits.shape == (n, spec.speakers)
    # the first chunk is a window of chunk + look-ahead rows over the same features
    cfg = st.config
    first = model.frame_logits(feat[0, : (cfg.frames + cfg.right) * spec.factor])[: cfg.frames * spec.factor]
    assert torch.allclose(logits[: cfg.frames * spec.factor], first, atol=2e-2)
    assert st.steps >= n // (cfg.frames * spec.factor)
    with pytest.raises(RuntimeError):
        st.push(wave[:10])
    segs = model.diarize(wave, stream=True)
    again = model.diarize(wave, stream=True)
    assert [(s.start, s.end, s.text) for s in segs] == [(s.start, s.end, s.text) for s in again]
    for s in segs + model.diarize(wave):
        assert s.text.startswith("speaker_") and 0.0 <= s.start <= s.end <= n * spec.frame_seconds + 1e-9


def test_save_load_and_command_line(tmp_path, capsys):
    from flyingfish_b200 import cli
    spec = dz.diarization_tiny()
    tensors = dz.random_tensors(spec, 7)
    # push the output bias so that some frames are active with random weights
    tensors["classifier.out_proj.bias"] = torch.tensor([2.0, -2.0, 0.0, -4.0])
    dz.save_model(tmp_path / "model", spec, tensors)
    model = dz.load_model(tmp_path / "model")
    direct = dz.DiarizationModel(spec, tensors)
    g = torch.Generator().manual_seed(9)
    feat = torch.randn(24, spec.mel.mel_bins, generator=g)
    assert torch.equal(model.frame_logits(feat), direct.frame_logits(feat))
    wave = torch.randn(spec.mel.hop_length * 60, generator=g) * 0.1
    write_wav(tmp_path / "two words.wav", wave, spec.mel.sampling_rate)
    assert cli.main(["--model", str(tmp_path / "model"), "--cpu", "diarize", str(tmp_path / "two words.wav")]) == 0
    out = capsys.readouterr().out
    lines = out.strip().splitlines()
    assert lines and all(ln.startswith("SPEAKER two_words 1 ") and ln.endswith(" <NA> <NA>") for ln in lines)
    assert any(" speaker_0 " in ln for ln in lines)
    assert cli.main(["--model", str(tmp_path / "model"), "--cpu", "diarize", "--stream", "--mode", "ultra_low_latency", "--format", "json",
                     "--output", str(tmp_path / "out.json"), str(tmp_path / "two words.wav")]) == 0
    segs = json.loads((tmp_path / "out.json").read_text())
    assert segs and all(set(s) == {"start", "end", "speaker"} for s in segs)
    with pytest.raises(SystemExit):
        cli.main(["--model", str(tmp_path / "model"), "--cpu", "diarize", "--mode", "low_latency", str(tmp_path / "two words.wav")])
    capsys.readouterr()
    assert cli.main(["--model", str(tmp_path / "model"), "inspect"]) == 0
    info = json.loads(capsys.readouterr().out)
    assert info["architecture"] == "Nemotron3DiarizationForAudioFrameClassification" and info["expected_tensors"] == len(spec.expected_tensors())
    assert info["spec"]["speakers"] == 4 and info["max_encoder_rows"] == spec.max_encoder_rows()


@pytest.mark.gpu
def test_diarization_gpu_matches_cpu():
    spec = dz.diarization_tiny()
    tensors = dz.random_tensors(spec, 11)
    cpu, gpu = dz.DiarizationModel(spec, tensors), dz.DiarizationModel(spec, tensors, "cuda:0")
    g = torch.Generator().manual_seed(5)
    long = torch.randn(50 * spec.factor + 3, spec.mel.mel_bins, generator=g)
    a, b = cpu.offline(long), gpu.offline(long.cuda()).cpu()
    assert a.shape == b.shape
    # the first chunk has no speaker memory behind it: plain numerics of encoder and head
    n0 = spec.offline.frames * spec.factor
    assert (a[:n0] - b[:n0]).abs().max() < 0.03 * a.abs().max() + 2e-3
    # later chunks agree as long as both sides compressed the cache to the same rows
    if torch.equal(cpu.last_state.probs > 0.5, gpu.last_state.probs > 0.5):
        assert (a - b).abs().max() < 0.06 * a.abs().max() + 5e-3
