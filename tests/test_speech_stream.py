"""Cache-aware streaming speech recognition: chunk-wise attention context, the incremental front end, encoder stream and
transducer state against their offline counterparts."""
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))

from flyingfish_b200.models.conformer import ConformerEncoder, ConformerStream, random_tensors
from flyingfish_b200.ops import speech_ops
from flyingfish_b200.speech import LogMel, LogMelConfig, ParakeetModel, StreamingLogMel, StreamingRecognizer, streaming_tiny


def _kept(rows, keys, query_offset, kv_offset, valid, chunk=4, left=14, right=0):
    out = []
    for q in range(rows):
        qc = (query_offset + q) // chunk
        out.append(sum(1 for k in range(keys) if k < valid and qc - left <= (kv_offset + k) // chunk <= qc + right))
    return out


def test_chunk_context_counts():
    # the rule itself: key chunk within [query chunk - left, query chunk + right]
    assert _kept(8, 8, 0, 0, 8) == [4, 4, 4, 4, 8, 8, 8, 8]
    assert _kept(8, 8, 0, 0, 5) == [4, 4, 4, 4, 5, 5, 5, 5]
    assert _kept(4, 60, 60, 4, 60) == [60, 60, 60, 60] and _kept(4, 60, 0, 0, 60) == [4, 4, 4, 4]
    # the attention oracle applies it: with constant values the output is the mean over the kept keys, so a value
    # channel that marks key j with j makes the output the mean kept index
    t, d = 12, 8
    q = torch.zeros(t, d).to(torch.bfloat16)
    k = torch.zeros(t, d).to(torch.bfloat16)
    v = torch.arange(t, dtype=torch.float32)[:, None].expand(t, d).to(torch.bfloat16)
    pos = torch.zeros(2 * t - 1, d).to(torch.bfloat16)
    z = torch.zeros(1, d)
    out = speech_ops.relpos_attention(q, k, v, pos, z, z, torch.tensor([11], dtype=torch.int32), 1, 1, left=1, right=0, chunk=4)
    want = []
    for i in range(t):
        ks = [j for j in range(11) if i // 4 - 1 <= j // 4 <= i // 4]
        want.append(sum(ks) / len(ks) if i < 11 else 0.0)
    assert torch.allclose(out[:, 0].float(), torch.tensor(want), atol=0.05)


def test_streaming_front_end_equals_offline():
    cfg = LogMelConfig(mel_bins=32, normalize=False)
    mel = LogMel(cfg)
    g = torch.Generator().manual_seed(3)
    wave = 0.2 * torch.randn(16000 + 77, generator=g)
    want, valid = mel.extract([wave], normalize=False)
    for piece in (5120, 1600, 333):
        s = StreamingLogMel(mel)
        got, at = [], 0
        while at < wave.numel():
            nxt = min(wave.numel(), at + piece)
            got.append(s.push(wave[at:nxt], last=nxt == wave.numel()))
            at = nxt
        got = torch.cat(got)
        assert got.shape[0] == int(valid[0])
        assert (got - want[0, : got.shape[0]]).abs().max() < 1e-4, piece
    with pytest.raises(RuntimeError):
        s.push(wave[:10])


def test_encoder_stream_equals_offline_encode():
    spec = streaming_tiny().encoder
    tensors = random_tensors(spec.expected_tensors(), seed=2)
    enc = ConformerEncoder(spec, tensors)
    g = torch.Generator().manual_seed(4)
    for n_frames in (203, 200, 64):
        feat = torch.randn(1, n_frames, spec.mel_bins, generator=g)
        want, rows = enc.encode(feat, [n_frames])
        for piece in (32, 7, 500):
            stream = ConformerStream(enc)
            got, at = [], 0
            while at < n_frames:
                nxt = min(n_frames, at + piece)
                got.append(stream.push(feat[0, at:nxt], last=nxt == n_frames))
                at = nxt
            got = torch.cat(got)
            assert got.shape[0] == rows[0] == spec.sub_len(n_frames), (n_frames, piece)
            err = (got.float() - want[0, : rows[0]].float()).abs()
            assert err.max() < 0.06 and err.mean() < 0.005, (n_frames, piece, float(err.max()))
    # a query never sees more than left_chunks earlier chunks: changing old frames leaves late rows alone
    feat = torch.randn(1, 800, spec.mel_bins, generator=g)
    base, _ = enc.encode(feat, [800])
    feat2 = feat.clone()
    feat2[0, :40] += 1.0
    moved, _ = enc.encode(feat2, [800])
    assert (base[0, :5].float() - moved[0, :5].float()).abs().max() > 1e-2
    # row r looks back (layers * left_chunks) chunks of 4 rows plus the convolutions' 8 rows per layer and 2 stem rows
    reach = spec.layers * (spec.left_chunks * 4 + 3 + 8) + 2 + 5
    assert (base[0, reach + 5:].float() - moved[0, reach + 5:].float()).abs().max() == 0
    with pytest.raises(ValueError):
        ConformerStream(ConformerEncoder(streaming_tiny().encoder.__class__(layers=1, hidden=128, heads=2, intermediate=128,
                                                                          mel_bins=32, sub_channels=32),
                                         random_tensors(streaming_tiny().encoder.__class__(layers=1, hidden=128, heads=2, intermediate=128,
                                                                                          mel_bins=32, sub_channels=32).expected_tensors(), 0)))


def test_transducer_state_carries_over_pieces():
    spec = streaming_tiny()
    model = ParakeetModel.random(spec, seed=9)
    g = torch.Generator().manual_seed(10)
    rows = torch.randn(37, spec.decoder_hidden, generator=g).to(torch.bfloat16)
    whole = model.decoder.decode(rows, 37)
    dec = model.decoder
    dec.begin_stream()
    tok, dur, frm = [spec.blank], [0], [0]
    for a, b in ((0, 4), (4, 5), (5, 5), (5, 20), (20, 37)):
        part = dec.extend(rows[a:b])
        tok += part.tokens; dur += part.durations; frm += part.frames
    assert (tok, dur, frm) == (whole.tokens, whole.durations, whole.frames)


def test_streaming_recognizer_follows_offline_model():
    spec = streaming_tiny()
    model = ParakeetModel.random(spec, seed=11)
    g = torch.Generator().manual_seed(12)
    wave = 0.2 * torch.randn(24000, generator=g)
    rec = StreamingRecognizer(model)
    seen = 0
    for at in range(0, 24000, 5120):
        nxt = min(24000, at + 5120)
        rec.push(wave[at:nxt], last=nxt == 24000)
        assert len(rec.tokens) >= seen
        seen = len(rec.tokens)
    tr = rec.trajectory()
    rows = spec.encoder.sub_len(24000 // 160)
    assert tr.tokens[0] == spec.blank and tr.frames[-1] < rows and all(d in (0, 1) for d in tr.durations)
    for (f0, d0), f1 in zip(zip(tr.frames[1:], tr.durations[1:]), tr.frames[2:]):
        assert f1 == f0 + d0
    # the encoder rows behind it equal the offline rows
    enc_off, n = model.encode([wave])
    assert n[0] == rows and rec.stream.rows_out == rows
    with pytest.raises(ValueError):
        StreamingRecognizer(ParakeetModel.random(__import__("flyingfish_b200.speech", fromlist=["parakeet_tiny"]).parakeet_tiny(), seed=1))


@pytest.mark.gpu
def test_chunk_context_kernel_and_stream_on_device(cuda):
    g = torch.Generator().manual_seed(5)
    t, d, heads, lens = 150, 64, 2, [150, 90]
    b = len(lens)
    qkv = torch.randn(b * t, 3 * heads * d, generator=g).to(torch.bfloat16)
    pos = torch.randn(2 * t - 1, heads * d, generator=g).to(torch.bfloat16)
    u, v = 0.5 * torch.randn(heads, d, generator=g), 0.5 * torch.randn(heads, d, generator=g)
    ln = torch.tensor(lens, dtype=torch.int32)
    hd = heads * d
    for left, right, chunk in ((14, 0, 4), (2, 1, 16), (0, 0, 7)):
        want = speech_ops.relpos_attention(qkv[:, :hd], qkv[:, hd:2 * hd], qkv[:, 2 * hd:], pos, u, v, ln, b, heads, left, right, chunk)
        qg = qkv.to(cuda)
        got = speech_ops.relpos_attention(qg[:, :hd], qg[:, hd:2 * hd], qg[:, 2 * hd:], pos.to(cuda), u.to(cuda), v.to(cuda),
                                          ln.to(cuda), b, heads, left, right, chunk)
        err = (got.float().cpu() - want.float()).abs()
        assert err.max() < 4e-2, (left, right, chunk, float(err.max()))
    spec = streaming_tiny()
    model = ParakeetModel.random(spec, cuda, seed=11)
    wave = 0.2 * torch.randn(24000, generator=g)
    enc_off, n = model.encode([wave])
    rec = StreamingRecognizer(model)
    got = []
    for at in range(0, 24000, 5120):
        nxt = min(24000, at + 5120)
        frames = rec.front.push(wave[at:nxt], last=nxt == 24000)
        got.append(rec.stream.push(frames, last=nxt == 24000))
    got = torch.cat(got)
    err = (got.float() - enc_off[0, : n[0]].float()).abs()
    assert got.shape[0] == n[0] and err.max() < 0.1 and err.mean() < 0.01, float(err.max())
    rec2 = StreamingRecognizer(model)
    rec2.push(wave[:12000])
    rec2.push(wave[12000:], last=True)
    assert rec2.trajectory().frames[-1] < n[0] and model.decoder.graph_replays > 0


def test_transcribe_stream_command(tmp_path, capsys):
    import json
    from test_speech import _write_model_dir
    from flyingfish_b200 import cli
    from flyingfish_b200.speech import ParakeetSpec, write_wav
    spec = streaming_tiny()
    assert ParakeetSpec.from_json(*spec.to_json()) == spec
    d = tmp_path / "stream"
    _write_model_dir(d, spec, 13)
    g = torch.Generator().manual_seed(14)
    write_wav(tmp_path / "in.wav", 0.2 * torch.randn(20000, generator=g), 16000)
    assert cli.main(["--cpu", "--model", str(d), "transcribe", str(tmp_path / "in.wav"), "--stream", "--format", "json"]) == 0
    io = capsys.readouterr()
    final = json.loads(io.out)
    assert set(final) == {"text", "segments", "words"}
    updates = [json.loads(l) for l in io.err.splitlines() if l.startswith("{")]
    assert all(u["tokens"] and u["seconds"] <= 20000 / 16000 + 1e-9 for u in updates)
    assert [u["seconds"] for u in updates] == sorted(u["seconds"] for u in updates)


NEMO_YAML = """\
token_init_method: constant
sample_rate: 16000
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
  subsampling: dw_striding
  subsampling_factor: 8
  subsampling_conv_channels: 32
  causal_downsampling: true
  ff_expansion_factor: 2
  self_attention_model: rel_pos
  n_heads: 2
  att_context_size:
  - 6
  - 1
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
"""


def _write_nemo(path, spec, seed):
    import io
    import tarfile
    from flyingfish_b200.speech.nemo import canonical_tensors
    canon = random_tensors(spec.expected_tensors(), seed)
    # NeMo spellings of the decoder / joint tensors (the encoder's are carried by the spec)
    back = {"decoder.embedding.weight": "decoder.prediction.embed.weight", "decoder.decoder_projector.weight": "joint.pred.weight",
            "decoder.decoder_projector.bias": "joint.pred.bias", "encoder_projector.weight": "joint.enc.weight",
            "encoder_projector.bias": "joint.enc.bias", "joint.head.weight": "joint.joint_net.2.weight", "joint.head.bias": "joint.joint_net.2.bias"}
    for kind in ("weight_ih", "weight_hh", "bias_ih", "bias_hh"):
        back[f"decoder.lstm.{kind}_l0"] = f"decoder.prediction.dec_rnn.lstm.{kind}_l0"
    nemo = {back.get(n, n): t for n, t in canon.items()}
    assert set(canonical_tensors(spec, nemo)) == set(canon)
    buf = io.BytesIO()
    torch.save(nemo, buf)
    vocab = "\n".join(["<unk>\t0.0"] + [f"{'▁' if i % 2 else ''}p{i}\t-{i}.0" for i in range(1, 28)] + ["<EOU>\t-1.0", "<EOB>\t-1.0"])
    with tarfile.open(path, "w") as tar:
        for name, data in (("./model_config.yaml", NEMO_YAML.encode()), ("./model_weights.ckpt", buf.getvalue()),
                           ("./abc123_tokenizer.vocab", vocab.encode())):
            info = tarfile.TarInfo(name)
            info.size = len(data)
            tar.addfile(info, io.BytesIO(data))
    return canon


def test_nemo_archive_streams_and_cuts_utterances(tmp_path):
    from flyingfish_b200.speech.nemo import UnigramVocab, load_nemo, spec_from_yaml, split_utterances, transcribe_nemo
    spec = spec_from_yaml(NEMO_YAML)
    e = spec.encoder
    assert (e.chunk_size, e.left_chunks, e.right_chunks, e.causal_conv, e.conv_batch_norm) == (2, 3, 0, True, False)
    assert spec.blank == 30 and spec.vocab == 31 and spec.durations == () and not spec.mel.normalize and spec.mel.win_length == 400
    assert "encoder.layers.0.self_attn.linear_pos.weight" in spec.expected_tensors()
    assert "encoder.layers.1.conv.batch_norm.weight" in spec.expected_tensors() and "encoder.pre_encode.out.bias" in spec.expected_tensors()
    with pytest.raises(ValueError, match="architecture variant"):
        spec_from_yaml(NEMO_YAML.replace("chunked_limited", "regular"))
    with pytest.raises(ValueError, match="lacks"):
        spec_from_yaml(NEMO_YAML.replace("  n_heads: 2\n", ""))
    arc = tmp_path / "m.nemo"
    canon = _write_nemo(arc, spec, 21)
    model = load_nemo(arc)
    direct = ParakeetModel(spec, canon)
    g = torch.Generator().manual_seed(22)
    wave = 0.2 * torch.randn(16000, generator=g)
    a, b = StreamingRecognizer(model), StreamingRecognizer(direct)
    a.push(wave, last=True); b.push(wave, last=True)
    assert a.tokens == b.tokens and a.frames == b.frames
    assert UnigramVocab("<unk>\t0.0\n▁hello\t-1.0\n▁world\t-2.0\n▁again\t-3.0").decode([1, 2]) == "hello world"
    # utterances end where the marker is emitted
    utt = split_utterances([30, 5, 6, 28, 30, 7, 28, 9], [0, 1, 1, 3, 3, 6, 8, 9], [0, 0, 0, 0, 1, 0, 0, 0], blank=30, eou=28)
    assert [(u[0], round(u[1], 2), round(u[2], 2)) for u in utt] == [([5, 6], 0.0, 0.24), ([7], 0.24, 0.64), ([9], 0.64, 0.72)]
    res = transcribe_nemo(arc, wave)
    assert isinstance(res.text, str) and all(s.end >= s.start for s in res.segments)
    whole = transcribe_nemo(arc, wave, stream=False)
    assert len(whole.segments) <= 1
    from flyingfish_b200 import cli
    from flyingfish_b200.speech import write_wav
    write_wav(tmp_path / "w.wav", wave, 16000)
    import contextlib, io as _io, json as _json
    buf = _io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert cli.main(["--cpu", "--model", str(arc), "transcribe", str(tmp_path / "w.wav"), "--stream", "--format", "json"]) == 0
    assert _json.loads(buf.getvalue())["text"] == res.text
    buf = _io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert cli.main(["--model", str(arc), "inspect"]) == 0
    info = _json.loads(buf.getvalue())
    assert info["architecture"] == "nemo_rnnt" and info["spec"]["encoder"]["chunk_size"] == 2 and info["tensors"] > 50 and info["bytes"] > 0


def test_prompt_conditioned_rnnt(tmp_path, capsys):
    import json
    from test_speech import _write_model_dir
    from flyingfish_b200 import cli
    from flyingfish_b200.speech import ParakeetSpec, load_model, nemotron_tiny, write_wav
    spec = nemotron_tiny()
    root, processor, generation = spec.to_json()
    assert root["architectures"] == ["Nemotron3_5AsrForRNNT"] and root["durations"] == [] and processor["prompt_dictionary"]["auto"] == 4
    assert ParakeetSpec.from_json(root, processor, generation) == spec
    exp = spec.expected_tensors()
    assert exp["prompt_projector.linear_1.weight"] == ("F32", (96, 128 + 6)) and exp["prompt_projector.linear_2.weight"] == ("F32", (128, 96))
    bad = dict(root, durations=[0, 1])
    with pytest.raises(ValueError):
        ParakeetSpec.from_json(bad, processor, generation)
    # the adapter is the published arithmetic: relu(W1 [row; one-hot] + b1), W2 . + b2, then the joint projection
    tensors = random_tensors(spec.expected_tensors(), 17)
    model = ParakeetModel(spec, tensors)
    g = torch.Generator().manual_seed(18)
    rows = torch.randn(5, 128, generator=g).to(torch.bfloat16)
    r = lambda t: t.to(torch.bfloat16).float()
    for pid in (4, 1):
        model.decoder.prompt_id = pid
        got = model.decoder.project(rows).float()
        onehot = torch.zeros(5, 6); onehot[:, pid] = 1.0
        w1 = r(tensors["prompt_projector.linear_1.weight"])
        u = torch.relu(torch.cat([rows.float(), onehot], 1) @ w1.t() + tensors["prompt_projector.linear_1.bias"])
        c = r(u) @ r(tensors["prompt_projector.linear_2.weight"]).t() + tensors["prompt_projector.linear_2.bias"]
        want = r(c) @ r(tensors["encoder_projector.weight"]).t() + tensors["encoder_projector.bias"]
        assert (got - want).abs().max() < 3e-2, pid
    # through files, the architecture switch, streaming and the prompt dictionary
    d = tmp_path / "nemotron"
    _write_model_dir(d, spec, 17)
    loaded = load_model(d)
    assert loaded.spec == spec and loaded.decoder.adapter is not None
    write_wav(tmp_path / "in.wav", 0.2 * torch.randn(16000, generator=g), 16000)
    assert cli.main(["--cpu", "--model", str(d), "transcribe", str(tmp_path / "in.wav"), "--stream", "--source-lang", "de", "--format", "json"]) == 0
    assert set(json.loads(capsys.readouterr().out)) == {"text", "segments", "words"}
    with pytest.raises(SystemExit, match="prompt dictionary"):
        cli.main(["--cpu", "--model", str(d), "transcribe", str(tmp_path / "in.wav"), "--source-lang", "xx"])
