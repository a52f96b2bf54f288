"""Speaker-attributed streaming recognition: multi-lane transducer streams, speaker kernels, lane gating, word times,
the NeMo archive and the diarizer -> recogniser pipeline."""
import io
import tarfile

import pytest
import torch

from flyingfish_b200.speech import ParakeetModel, StreamingRecognizer, streaming_tiny
from flyingfish_b200.speech import multitalker as mt
from flyingfish_b200.speech.parakeet import random_tensors

YAML = """
sample_rate: 16000
spk_kernel_type: ff
spk_kernel_layers:
- 0
add_bg_spk_kernel: true
model_defaults:
  num_speakers: 3
preprocessor:
  sample_rate: 16000
  normalize: NA
  window_size: 0.025
  window_stride: 0.01
  features: 32
  n_fft: 512
  frame_splicing: 1
  dither: 1.0e-05
  pad_to: 0
encoder:
  feat_in: 32
  n_layers: 2
  d_model: 128
  use_bias: false
  untie_biases: true
  subsampling: dw_striding
  subsampling_factor: 8
  subsampling_conv_channels: 32
  causal_downsampling: true
  ff_expansion_factor: 2
  self_attention_model: rel_pos
  n_heads: 2
  att_context_size:
  - - 9
    - 2
  - - 9
    - 0
  att_context_style: chunked_limited
  xscaling: false
  pos_emb_max_len: 512
  conv_kernel_size: 9
  conv_norm_type: layer_norm
  conv_context_size: causal
decoder:
  vocab_size: 30
  blank_as_pad: true
  prednet:
    pred_hidden: 64
    pred_rnn_layers: 1
joint:
  num_classes: 30
  jointnet:
    joint_hidden: 64
    activation: relu
    encoder_hidden: 128
    pred_hidden: 64
decoding:
  greedy:
    max_symbols: 10
"""


def _tensors(spec: mt.MultitalkerSpec, seed: int, kernel_std: float = 0.05) -> dict[str, torch.Tensor]:
    tensors = random_tensors(spec.asr.expected_tensors(), seed)
    g = torch.Generator().manual_seed(seed + 1)
    h = spec.asr.encoder.hidden
    for name in mt.KERNEL_TENSORS:
        tensors[name + ".weight"] = torch.randn(h, h, generator=g) * kernel_std
        tensors[name + ".bias"] = torch.randn(h, generator=g) * kernel_std
    return tensors


def _wave(seed: int, seconds: float = 1.6) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return 0.2 * torch.randn(int(16000 * seconds), generator=g)


def test_spec_from_yaml():
    spec = mt.MultitalkerSpec.from_yaml(YAML)
    e = spec.asr.encoder
    assert spec.speakers == 3 and (e.chunk_size, e.left_chunks) == (3, 3) and spec.asr.max_symbols == 10
    names = spec.expected_tensors()
    assert names["spk_kernels.0.3.weight"] == ("F32", (128, 128)) and names["bg_spk_kernels.0.0.bias"] == ("F32", (128,))
    with pytest.raises(ValueError, match="speaker-kernel"):
        mt.MultitalkerSpec.from_yaml(YAML.replace("spk_kernel_type: ff", "spk_kernel_type: conv"))
    with pytest.raises(ValueError, match="lacks"):
        mt.MultitalkerSpec.from_yaml(YAML.replace("add_bg_spk_kernel: true\n", ""))
    with pytest.raises(ValueError, match="left context"):
        mt.MultitalkerSpec.from_yaml(YAML.replace("  - - 9\n    - 0\n", "  - - 6\n    - 0\n"))


def test_decoder_lanes_match_single_streams():
    spec = streaming_tiny()
    tensors = random_tensors(spec.expected_tensors(), 3)
    model = ParakeetModel(spec, tensors)
    g = torch.Generator().manual_seed(4)
    rows = [torch.randn(n, spec.decoder_hidden, generator=g).to(torch.bfloat16) for n in (7, 5, 9)]
    dec = model.decoder
    single = []
    for r in rows:
        dec.begin_stream()
        a = dec.extend(r[:3])
        b = dec.extend(r[3:])
        single.append((a.tokens + b.tokens, a.frames + b.frames))
    dec.begin_stream(3)
    first = dec.extend_lanes({0: rows[0][:3], 1: rows[1][:3], 2: rows[2][:3]})
    # lane 1 is parked for a round: its state must not move
    mid = dec.extend_lanes({0: rows[0][3:], 2: rows[2][3:6]})
    last = dec.extend_lanes({1: rows[1][3:], 2: rows[2][6:]})
    got0 = (first[0].tokens + mid[0].tokens, first[0].frames + mid[0].frames)
    got1 = (first[1].tokens + last[1].tokens, first[1].frames + last[1].frames)
    assert got0 == single[0] and got1 == single[1]
    # lane 2 got its rows in three pieces instead of two: the same tokens at the same rows
    got2 = (first[2].tokens + mid[2].tokens + last[2].tokens, first[2].frames + mid[2].frames + last[2].frames)
    keep = lambda tf: [(t, f) for t, f in zip(*tf) if t != spec.blank]
    assert keep(got2) == keep(single[2])
    with pytest.raises(ValueError):
        dec.extend_lanes({3: rows[0]})
    with pytest.raises(ValueError):
        dec.begin_stream(99)


def test_speaker_kernels_follow_the_formula():
    spec = mt.MultitalkerSpec.from_yaml(YAML)
    tensors = _tensors(spec, 5)
    model = mt.MultitalkerModel(spec, tensors)
    g = torch.Generator().manual_seed(6)
    h = torch.randn(6, 128, generator=g).to(torch.bfloat16)
    own = torch.tensor([1.0, 1.0, 0.0, 0.0, 1.0, 0.3])
    others = torch.tensor([0.0, 1.0, 1.0, 0.0, 0.0, 1.0])
    got = model.speaker_kernels(h, own, others).float()
    r = lambda n: tensors[n].to(torch.bfloat16).float()
    x = h.float()
    x = x + torch.relu((x * own[:, None]) @ r("spk_kernels.0.0.weight").t() + r("spk_kernels.0.0.bias")) @ r("spk_kernels.0.3.weight").t() \
        + r("spk_kernels.0.3.bias")
    x = x + torch.relu((x * others[:, None]) @ r("bg_spk_kernels.0.0.weight").t() + r("bg_spk_kernels.0.0.bias")) @ r("bg_spk_kernels.0.3.weight").t() \
        + r("bg_spk_kernels.0.3.bias")
    assert (got - x).abs().max() < 0.05 * x.abs().max()
    # a silent row still gets the kernels' bias path: relu(b1) W2 + b2
    assert (got[3] - h[3].float()).abs().max() > 0


def test_lanes_with_neutral_kernels_equal_the_plain_recogniser():
    spec = mt.MultitalkerSpec.from_yaml(YAML)
    tensors = _tensors(spec, 7, kernel_std=0.0)                 # kernels add exactly zero
    model = mt.MultitalkerModel(spec, tensors)
    wave = _wave(8)
    plain = StreamingRecognizer(ParakeetModel(spec.asr, {n: t for n, t in tensors.items() if n in spec.asr.expected_tensors()}))
    plain.push(wave, last=True)
    want = [(t, f) for t, f in zip(plain.tokens, plain.frames) if t != spec.asr.blank]
    rows = spec.asr.encoder.sub_len(len(wave) // spec.asr.mel.hop_length)
    st = model.stream(torch.ones(rows, 2), gating=True)
    for at in range(0, wave.numel(), 5000):
        st.push(wave[at:at + 5000], last=at + 5000 >= wave.numel())
    for lane in range(2):
        assert list(zip(st.tokens[lane], st.token_rows[lane])) == want
    assert st.lane_steps == [st.steps, st.steps]


def test_masks_steer_lanes_and_gating_parks_them():
    spec = mt.MultitalkerSpec.from_yaml(YAML)
    model = mt.MultitalkerModel(spec, _tensors(spec, 9, kernel_std=0.3))
    wave = _wave(10, 3.2)
    rows = spec.asr.encoder.sub_len(len(wave) // spec.asr.mel.hop_length)
    act = torch.zeros(rows, 3)
    act[:, 0] = 1.0                                             # speaker 0 throughout
    act[rows // 2:, 1] = 1.0                                    # speaker 1 joins half way; speaker 2 never speaks
    st = model.stream(act)
    for at in range(0, wave.numel(), 4000):
        st.push(wave[at:at + 4000], last=at + 4000 >= wave.numel())
    assert st.lane_steps[2] == 0 and st.tokens[2] == [] and st.row_map[2] == []
    assert 0 < st.lane_steps[1] < st.lane_steps[0] == st.steps
    chunk = spec.asr.encoder.chunk_size
    first_live = (rows // 2) // chunk * chunk                   # the chunk that holds speaker 1's first active row
    assert st.row_map[1][0] == first_live and st.row_map[0][0] == 0
    assert all(r >= first_live for r in st.token_rows[1])
    # masks matter: lane 0 hears the overlap in its second half, a lone lane 0 does not
    alone = model.stream(act[:, :1])
    for at in range(0, wave.numel(), 4000):
        alone.push(wave[at:at + 4000], last=at + 4000 >= wave.numel())
    n_first = sum(1 for r in st.token_rows[0] if r < first_live)
    assert list(zip(st.tokens[0], st.token_rows[0]))[:n_first] == list(zip(alone.tokens[0], alone.token_rows[0]))[:n_first]
    # without gating every lane runs every step
    free = model.stream(act, gating=False)
    free.push(wave, last=True)
    assert free.lane_steps == [free.steps] * 3
    # a parked lane resumes on its own row grid: speaker 1 goes quiet, then returns
    act2 = torch.zeros(rows, 2)
    act2[:, 0] = 1.0
    act2[:4, 1] = 1.0
    act2[-6:, 1] = 1.0
    st2 = model.stream(act2)
    st2.push(wave, last=True)
    gaps = [b - a for a, b in zip(st2.row_map[1], st2.row_map[1][1:])]
    assert max(gaps) > 1 and st2.row_map[1] == sorted(st2.row_map[1])
    tr = st2.transcription()
    for sp in tr.speakers:
        assert sp.words and sp.start == sp.words[0].start and sp.end == sp.words[-1].end and sp.start <= sp.end
        assert all(w.end > w.start for w in sp.words)


def test_feature_masking_variant():
    spec = mt.MultitalkerSpec.from_yaml(YAML)
    tensors = _tensors(spec, 7, kernel_std=0.0)
    model = mt.MultitalkerModel(spec, tensors)
    wave = _wave(8, 2.4)
    plain = StreamingRecognizer(ParakeetModel(spec.asr, {n: t for n, t in tensors.items() if n in spec.asr.expected_tensors()}))
    plain.push(wave, last=True)
    want = [(t, f) for t, f in zip(plain.tokens, plain.frames) if t != spec.asr.blank]
    rows = spec.asr.encoder.sub_len(len(wave) // spec.asr.mel.hop_length)
    act = torch.ones(rows, 2)
    act[rows // 3: 2 * rows // 3, 1] = 0.0                       # speaker 1 pauses in the middle third
    st = model.stream(act, gating=False, masked=True)
    for at in range(0, wave.numel(), 5000):
        st.push(wave[at:at + 5000], last=at + 5000 >= wave.numel())
    # a lane whose speaker never pauses sees the unmasked features: the plain recogniser's tokens
    assert list(zip(st.tokens[0], st.token_rows[0])) == want
    # the paused lane heard silence in the middle third: its second layer's attention cache (rows that looked back on
    # the silent stretch) differs from the other lane's, the stem rows of the last chunk (all audible again) do not
    assert not torch.equal(st.lane_streams[1].qkv[1], st.lane_streams[0].qkv[1])
    assert torch.equal(st.lane_streams[1].qkv[0][-2:], st.lane_streams[0].qkv[0][-2:])
    # the mask itself: frames of silent rows are zero, exact zeros take the log floor
    probe = model.stream(act, masked=True)
    frames = torch.ones(8 * rows, spec.asr.mel.mel_bins)
    frames[0, 0] = 0.0
    got = probe.masked_frames(frames, 1)
    lo, hi = 8 * (rows // 3), 8 * (2 * rows // 3)
    assert (got[lo:hi] == 0).all() and (got[hi:] == 1).all() and (got[1:lo] == 1).all()
    assert got[0, 0].item() == pytest.approx(-16.6355, abs=1e-3) and got[0, 1].item() == 1.0


def test_speaker_words():
    pieces = ["<unk>", "▁he", "llo", "▁", "wor", "ld", "▁again", "<EOU>"]
    text, words = mt.speaker_words([1, 2, 3, 4, 5, 7, 6], [2, 3, 9, 9, 11, 12, 20], lambda t: pieces[t], 0.08)
    assert text == "hello world again"
    assert [(w.text, round(w.start, 2), round(w.end, 2)) for w in words] == [("hello", 0.16, 0.32), ("world", 0.72, 0.96), ("again", 1.6, 1.68)]
    with pytest.raises(ValueError):
        mt.speaker_words([1], [], lambda t: "", 0.08)


def _write_nemo(path, spec: mt.MultitalkerSpec, seed: int) -> dict[str, torch.Tensor]:
    canon = _tensors(spec, seed, kernel_std=0.2)
    back = {"decoder.embedding.weight": "decoder.prediction.embed.weight", "decoder.decoder_projector.weight": "joint.pred.weight",
            "decoder.decoder_projector.bias": "joint.pred.bias", "encoder_projector.weight": "joint.enc.weight",
            "encoder_projector.bias": "joint.enc.bias", "joint.head.weight": "joint.joint_net.2.weight", "joint.head.bias": "joint.joint_net.2.bias"}
    for kind in ("weight_ih", "weight_hh", "bias_ih", "bias_hh"):
        back[f"decoder.lstm.{kind}_l0"] = f"decoder.prediction.dec_rnn.lstm.{kind}_l0"
    buf = io.BytesIO()
    torch.save({back.get(n, n): t for n, t in canon.items()}, buf)
    vocab = "\n".join(["<unk>\t0.0"] + [f"{'▁' if i % 2 else ''}p{i}\t-{i}.0" for i in range(1, 30)])
    with tarfile.open(path, "w") as tar:
        for name, data in (("./model_config.yaml", YAML.encode()), ("./model_weights.ckpt", buf.getvalue()),
                           ("./abc_tokenizer.vocab", vocab.encode())):
            info = tarfile.TarInfo(name)
            info.size = len(data)
            tar.addfile(info, io.BytesIO(data))
    return canon


def test_archive_and_pipeline_with_a_diarizer(tmp_path, capsys):
    import json
    from flyingfish_b200 import cli
    from flyingfish_b200.speech import diarization as dz
    from flyingfish_b200.speech.audio import LogMelConfig, write_wav
    spec = mt.MultitalkerSpec.from_yaml(YAML)
    arc = tmp_path / "mt.nemo"
    canon = _write_nemo(arc, spec, 11)
    model = mt.MultitalkerModel.load(arc)
    direct = mt.MultitalkerModel(spec, canon, tokenizer=model.tokenizer)
    wave = _wave(12, 2.4)
    rows = spec.asr.encoder.sub_len(len(wave) // 160)
    act = torch.ones(rows, 2)
    a, b = model.transcribe_speakers(wave, act), direct.transcribe_speakers(wave, act)
    assert a.to_json() == b.to_json()
    # a diarizer at the same 80 ms row grid (hop 160, factor 8) with three output channels
    dspec = dz.DiarizationSpec(hidden=64, intermediate=128, layers=1, heads=2, head_hidden=32, speakers=3, factor=8, max_positions=128,
                               mel=LogMelConfig(sampling_rate=16000, n_fft=512, win_length=400, hop_length=160, mel_bins=16, normalize=False),
                               offline=dz.ChunkConfig(12, 3, 6, 8),
                               cache=dz.SpeakerCacheConfig(frames=15, silence=1, fifo=10, update=6),
                               modes={"low_latency": (5, 2)}, default_mode="low_latency")
    dt = dz.random_tensors(dspec, 13)
    dt["classifier.out_proj.bias"] = torch.tensor([3.0, 3.0, -6.0])           # speakers 0 and 1 always on, 2 never
    dz.save_model(tmp_path / "diar", dspec, dt)
    masks, seconds = dz.speaker_masks(dz.load_model(tmp_path / "diar"), wave)
    assert seconds == pytest.approx(0.08) and masks.shape[1] == 3 and masks[:, :2].all() and not masks[:, 2].any()
    out = mt.transcribe_multitalker(arc, tmp_path / "diar", wave, stream_diarizer=False)
    want = model.transcribe_speakers(wave, masks[:, :3].float())
    assert out.to_json() == want.to_json()
    write_wav(tmp_path / "w.wav", wave, 16000)
    assert cli.main(["--cpu", "--model", str(arc), "transcribe", str(tmp_path / "w.wav"), "--diarization-model", str(tmp_path / "diar"),
                     "--format", "json"]) == 0
    got = json.loads(capsys.readouterr().out)
    assert [s["speaker"] for s in got["speakers"]] == [s.speaker for s in mt.transcribe_multitalker(arc, tmp_path / "diar", wave).speakers]
    capsys.readouterr()
    assert cli.main(["--model", str(arc), "inspect"]) == 0
    info = json.loads(capsys.readouterr().out)
    assert info["architecture"] == "nemo_multitalker_rnnt" and info["speakers"] == 3 and len(info["speaker_kernels"]) == 4
    # a multitalker archive without a diarizer is refused, and so is activity for more lanes than the model serves
    with pytest.raises(SystemExit):
        cli.main(["--cpu", "--model", str(arc), "transcribe", str(tmp_path / "w.wav")])
    model2 = mt.MultitalkerModel(mt.MultitalkerSpec(spec.asr, 2), canon)
    with pytest.raises(ValueError):
        model2.stream(torch.ones(4, 3))
    # a diarizer that hears a speaker on a channel beyond the model's lanes is refused
    dt["classifier.out_proj.bias"] = torch.tensor([3.0, 3.0, 3.0, 3.0])
    dt["classifier.out_proj.weight"] = torch.cat([dt["classifier.out_proj.weight"], torch.zeros(1, 32)], 0)
    from dataclasses import replace
    dz.save_model(tmp_path / "diar4", replace(dspec, speakers=4, cache=dz.SpeakerCacheConfig(frames=16, silence=1, fifo=10, update=6)), dt)
    with pytest.raises(ValueError, match="beyond"):
        mt.transcribe_multitalker(arc, tmp_path / "diar4", wave, stream_diarizer=False)


@pytest.mark.gpu
def test_multitalker_gpu_lanes():
    spec = mt.MultitalkerSpec.from_yaml(YAML)
    tensors = _tensors(spec, 7, kernel_std=0.0)
    model = mt.MultitalkerModel(spec, tensors, "cuda:0")
    wave = _wave(8, 2.4)
    plain = StreamingRecognizer(ParakeetModel(spec.asr, {n: t for n, t in tensors.items() if n in spec.asr.expected_tensors()}, "cuda:0"))
    plain.push(wave, last=True)
    want = [(t, f) for t, f in zip(plain.tokens, plain.frames) if t != spec.asr.blank]
    rows = spec.asr.encoder.sub_len(len(wave) // spec.asr.mel.hop_length)
    act = torch.ones(rows, 3)
    act[: rows // 2, 2] = 0.0                                   # lane 2 starts half way
    st = model.stream(act)
    for at in range(0, wave.numel(), 6000):
        st.push(wave[at:at + 6000], last=at + 6000 >= wave.numel())
    assert list(zip(st.tokens[0], st.token_rows[0])) == want and list(zip(st.tokens[1], st.token_rows[1])) == want
    assert 0 < st.lane_steps[2] < st.lane_steps[0]
    # kernels with weight: the device path follows the host path on the conditioned rows
    tensors = _tensors(spec, 9, kernel_std=0.2)
    cpu, gpu = mt.MultitalkerModel(spec, tensors), mt.MultitalkerModel(spec, tensors, "cuda:0")
    g = torch.Generator().manual_seed(1)
    h = torch.randn(6, 128, generator=g).to(torch.bfloat16)
    own, others = torch.tensor([1.0, 1, 0, 0, 1, 0.3]), torch.tensor([0.0, 1, 1, 0, 0, 1])
    a, b = cpu.speaker_kernels(h, own, others).float(), gpu.speaker_kernels(h.cuda(), own, others).float().cpu()
    assert (a - b).abs().max() < 0.03 * a.abs().max()
