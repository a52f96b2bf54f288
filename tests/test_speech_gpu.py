"""Speech kernels (csrc/speech.cu) against their CPU oracles, and the whole recognition model on the device against
its CPU run."""
import math

import pytest
import torch

from flyingfish_b200 import ops
from flyingfish_b200.models.conformer import ConformerEncoder, random_tensors
from flyingfish_b200.ops import speech_ops, vision_ops
from flyingfish_b200.ops.speech_ops import TS_ADVANCE, TS_CAP, TS_COUNT, TS_MAXSYM, TS_SYMS, TS_TOKEN, TS_VALID, TS_WORDS
from flyingfish_b200.speech import LogMel, LogMelConfig, ParakeetModel, parakeet_tiny

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _close(got, want, atol, rtol=0.0):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    lim = atol + rtol * want.abs()
    assert (err <= lim).all(), (float(err.max()), float((err - lim).max()))


@pytest.mark.parametrize("cfg", [LogMelConfig(), LogMelConfig(n_fft=256, win_length=200, hop_length=80, mel_bins=40, sampling_rate=8000)])
def test_logmel_kernel(cuda, cfg):
    g = torch.Generator().manual_seed(1)
    ramp = torch.linspace(0.2, 1.0, 12000)
    waves = [0.3 * torch.randn(16000 + 37, generator=g), 0.3 * torch.randn(7000, generator=g), ramp * torch.randn(12000, generator=g)]
    cpu_feat, cpu_valid = LogMel(cfg).extract(waves)
    gpu_feat, gpu_valid = LogMel(cfg, cuda).extract(waves)
    assert gpu_feat.is_cuda and gpu_valid.tolist() == cpu_valid.tolist()
    _close(gpu_feat, cpu_feat, 5e-3)
    # un-normalised values, a pure tone included (most bands then hold only leakage and the guard)
    waves.append(torch.sin(torch.arange(12000) * 0.05))
    raw_c, _ = LogMel(cfg).extract(waves, normalize=False)
    raw_g, _ = LogMel(cfg, cuda).extract(waves, normalize=False)
    _close(raw_g, raw_c, 5e-3, 1e-4)


def test_subsampling_kernels(cuda):
    g = torch.Generator().manual_seed(2)
    b, t, f, c = 3, 61, 32, 32
    feat = torch.randn(b, t, f, generator=g)
    w0, b0 = 0.3 * torch.randn(9, c, generator=g), 0.1 * torch.randn(c, generator=g)
    valid = [61, 40, 7]
    v1 = torch.tensor([speech_ops.conv_out_len(n, 1, 1) for n in valid], dtype=torch.int32)
    want = speech_ops.sub_conv_first(feat, w0, b0, v1, (1, 1))
    got = speech_ops.sub_conv_first(feat.to(cuda), w0.to(cuda), b0.to(cuda), v1.to(cuda), (1, 1))
    _close(got, want, 2e-2, 1e-2)
    w1, b1 = 0.3 * torch.randn(9, c, generator=g), 0.1 * torch.randn(c, generator=g)
    want2 = speech_ops.sub_dwconv(want, w1, b1, v1, (1, 1))
    got2 = speech_ops.sub_dwconv(want.to(cuda), w1.to(cuda), b1.to(cuda), v1.to(cuda), (1, 1))
    _close(got2, want2, 2e-2, 1e-2)
    relu = vision_ops.bias_act_(got2.reshape(-1, c).clone(), b1.to(BF16).to(cuda), "relu")
    assert float(relu.min()) >= 0


@pytest.mark.parametrize("k,xbias,silu", [(9, False, True), (9, True, False), (31, True, True), (5, False, True)])
def test_glu_dwconv1d_kernel(cuda, k, xbias, silu):
    g = torch.Generator().manual_seed(3)
    b, t, h = 3, 45, 192
    x = torch.randn(b * t, 2 * h, generator=g).to(BF16)
    xb = 0.2 * torch.randn(2 * h, generator=g) if xbias else None
    w, bias = 0.3 * torch.randn(k, h, generator=g), 0.1 * torch.randn(h, generator=g)
    lens = torch.tensor([45, 20, 1], dtype=torch.int32)
    want = speech_ops.glu_dwconv1d(x, xb, w, bias, lens, b, k // 2, silu)
    got = speech_ops.glu_dwconv1d(x.to(cuda), xb.to(cuda) if xbias else None, w.to(cuda), bias.to(cuda), lens.to(cuda), b, k // 2, silu)
    _close(got, want, 2e-2, 1e-2)


def test_scale_add_layernorm_kernel(cuda):
    g = torch.Generator().manual_seed(4)
    rows, hidden = 37, 1024
    h = torch.randn(rows, hidden, generator=g).to(BF16)
    d = torch.randn(rows, hidden, generator=g).to(BF16)
    db, w, b = (torch.randn(hidden, generator=g) for _ in range(3))
    h_c, h_g = h.clone(), h.clone().to(cuda)
    want = speech_ops.scale_add_layernorm(h_c, d, db, 0.5, w, b)
    got = speech_ops.scale_add_layernorm(h_g, d.to(cuda), db.to(cuda), 0.5, w.to(cuda), b.to(cuda))
    _close(h_g, h_c, 2e-2, 1e-2)
    _close(got, want, 3e-2, 2e-2)
    plain_w = speech_ops.scale_add_layernorm(h_c, None, None, 0.0, w, None)
    plain_g = speech_ops.scale_add_layernorm(h_g, None, None, 0.0, w.to(cuda), None)
    _close(plain_g, plain_w, 3e-2, 2e-2)


@pytest.mark.parametrize("t,d,lens,left,right", [(150, 128, [150, 64, 1], -1, -1), (70, 64, [70, 33], -1, -1),
                                                 (200, 64, [200, 131], 70, 10), (64, 128, [64], -1, -1)])
def test_relpos_attention_kernel(cuda, t, d, lens, left, right):
    g = torch.Generator().manual_seed(5)
    b, heads = len(lens), 2
    qkv = torch.randn(b * t, 3 * heads * d, generator=g).to(BF16)
    pos = torch.randn(2 * t - 1, heads * d, generator=g).to(BF16)
    u, v = 0.5 * torch.randn(heads, d, generator=g), 0.5 * torch.randn(heads, d, generator=g)
    ln = torch.tensor(lens, dtype=torch.int32)
    hd = heads * d
    want = speech_ops.relpos_attention(qkv[:, :hd], qkv[:, hd:2 * hd], qkv[:, 2 * hd:], pos, u, v, ln, b, heads, left, right)
    qg = qkv.to(cuda)
    got = speech_ops.relpos_attention(qg[:, :hd], qg[:, hd:2 * hd], qg[:, 2 * hd:], pos.to(cuda), u.to(cuda), v.to(cuda),
                                      ln.to(cuda), b, heads, left, right)
    _close(got, want, 3e-2, 2e-2)


def test_decoder_step_kernels(cuda):
    g = torch.Generator().manual_seed(6)
    hd = 640
    gates = torch.randn(4 * hd, generator=g).to(BF16)
    bias = torch.randn(4 * hd, generator=g)
    c0 = torch.randn(hd, generator=g)
    c_c, c_g = c0.clone(), c0.clone().to(cuda)
    hs_c, hn_c = torch.zeros(hd, dtype=BF16), torch.zeros(hd, dtype=BF16)
    hs_g, hn_g = hs_c.to(cuda), hn_c.to(cuda)
    speech_ops.lstm_cell(gates, bias, c_c, hs_c, hn_c, None)
    speech_ops.lstm_cell(gates.to(cuda), bias.to(cuda), c_g, hs_g, hn_g, None)
    _close(c_g, c_c, 1e-4, 1e-4)
    _close(hs_g, hs_c, 1e-2)
    assert torch.equal(hs_g, hn_g)
    # state words gate the update
    st = torch.zeros(TS_WORDS, dtype=torch.int32, device=cuda)
    before = c_g.clone()
    speech_ops.lstm_cell(gates.to(cuda), bias.to(cuda), c_g, hs_g, hn_g, st)
    assert torch.equal(c_g, before)
    # joint input + selection
    frames, j, n_tok = 9, 640, 1025
    enc = torch.randn(frames, j, generator=g).to(BF16)
    pred = torch.randn(1, j, generator=g).to(BF16)
    jb = torch.randn(j, generator=g)
    for frame in (0, 5, 8):
        st_c = torch.zeros(TS_WORDS, dtype=torch.int32)
        st_c[0] = frame
        out_c, out_g = torch.zeros(1, j, dtype=BF16), torch.zeros(1, j, dtype=BF16, device=cuda)
        speech_ops.tdt_joint_in(enc, pred, jb, st_c, out_c)
        speech_ops.tdt_joint_in(enc.to(cuda), pred.to(cuda), jb.to(cuda), st_c.to(cuda), out_g)
        _close(out_g, out_c, 2e-2, 1e-2)
    dur = torch.tensor([0, 1, 2, 3, 4], dtype=torch.int32)
    for trial in range(6):
        logits = torch.randn(1, n_tok + 5 + 2, generator=g).to(BF16)
        ob = 0.1 * torch.randn(n_tok + 5, generator=g)
        res = []
        for dev in ("cpu", cuda):
            st = torch.zeros(TS_WORDS, dtype=torch.int32)
            st[TS_TOKEN], st[TS_COUNT], st[TS_ADVANCE], st[TS_VALID], st[TS_CAP] = n_tok - 1, 1, 1, 50, 40
            st[TS_MAXSYM], st[TS_SYMS] = 2, trial % 2
            st[0] = trial
            st = st.to(dev)
            traj = tuple(torch.zeros(40, dtype=torch.int32, device=dev) for _ in range(3))
            speech_ops.tdt_select(logits.to(dev), ob.to(dev), dur.to(dev), st, traj, n_tok, n_tok - 1, 3)
            res.append((st.cpu().tolist(), [t[:3].cpu().tolist() for t in traj]))
        assert res[0] == res[1]


def test_encoder_on_device_matches_cpu(cuda):
    spec = parakeet_tiny().encoder
    tensors = random_tensors(spec.expected_tensors(), seed=3)
    g = torch.Generator().manual_seed(4)
    feat = torch.randn(2, 300, spec.mel_bins, generator=g)
    valid = [300, 170]
    feat[1, 170:] = 0
    want, rows = ConformerEncoder(spec, tensors).encode(feat, valid)
    got, rows_g = ConformerEncoder(spec, tensors, cuda).encode(feat.to(cuda), valid)
    assert rows == rows_g
    for b, n in enumerate(rows):
        err = (got[b, :n].float().cpu() - want[b, :n].float()).abs()
        assert err.max() < 0.25 and err.mean() < 0.02, (float(err.max()), float(err.mean()))


def test_model_decode_on_device(cuda):
    spec = parakeet_tiny()
    g = torch.Generator().manual_seed(8)
    waves = [0.1 * torch.randn(24000, generator=g), 0.1 * torch.randn(9000, generator=g)]
    before = ops.launch_count()
    dev_model = ParakeetModel.random(spec, cuda, seed=7)
    trajs = dev_model.decode(waves)
    assert ops.launch_count() > before
    assert dev_model.decoder.graph_replays > 0
    for tr, n in zip(trajs, (24000, 9000)):
        rows = spec.encoder.sub_len(n // 160)
        assert tr.tokens[0] == spec.blank and len(tr.tokens) <= tr.capacity and tr.frames[-1] < rows
        assert tr.state_reads <= tr.steps // 32 + 1            # the host looks at the device state once per 32 steps
        for (f0, d0), f1 in zip(zip(tr.frames[1:], tr.durations[1:]), tr.frames[2:]):
            assert f1 == f0 + d0
    # graph replay and eager stepping agree exactly (same kernels, same order)
    eager = ParakeetModel.random(spec, cuda, seed=7)
    eager.decoder.use_graph = False
    again = eager.decode(waves)
    assert [t.tokens for t in again] == [t.tokens for t in trajs] and [t.durations for t in again] == [t.durations for t in trajs]
    # the projection into the joint space agrees with the CPU path numerically
    cpu_model = ParakeetModel.random(spec, "cpu", seed=7)
    enc, rows = dev_model.encode(waves)
    proj = dev_model.decoder.project(enc[0, : rows[0]])
    _close(proj, cpu_model.decoder.project(enc[0, : rows[0]].cpu()), 3e-2, 2e-2)


def test_batched_decode_on_device(cuda):
    spec = parakeet_tiny()
    model = ParakeetModel.random(spec, cuda, seed=15, max_batch=3)
    g = torch.Generator().manual_seed(16)
    rows = [torch.randn(n, spec.decoder_hidden, generator=g).to(BF16).to(cuda) for n in (31, 12, 20)]
    valid = [31, 9, 20]
    dec = model.decoder
    together = dec.decode_batch(rows, valid)
    alone = [dec.decode(r, v) for r, v in zip(rows, valid)]
    for a, b in zip(together, alone):
        assert (a.tokens, a.durations, a.frames) == (b.tokens, b.durations, b.frames)
    assert dec.graph_replays > 0
