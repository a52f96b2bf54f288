"""Looped two-stack decoder: the engine's prefill + decode against a plain full-sequence PyTorch forward with the
prefix mask (prompt rows see the whole prompt, generated rows see everything before them), the YaRN table, whole-prompt
chunking, and the CUDA path against the CPU path."""
import math

import pytest
import torch

from flyingfish_b200 import ops
from flyingfish_b200.api import Model
from flyingfish_b200.config import Settings, named_shape
from flyingfish_b200.models.hrm import yarn_inv_freq
from flyingfish_b200.ops import vision_ops


def _load(device, **kw):
    return Model.load("loop-tiny", Settings(capacity=256, max_batch=4, graph=False, **kw), device=device, seed=0)


def _prompts():
    g = torch.Generator().manual_seed(9)
    return [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (37, 9)]


def _ref_logits(net, ids, prompt_len):
    """FP32 forward over the whole sequence; returns the logits of the last row."""
    w, s = net.w, net.spec
    f32 = lambda t: t.float().cpu()
    rows, h, d, nh = len(ids), s.hidden, 128, s.heads
    norm = lambda x: x * torch.rsqrt((x * x).mean(-1, keepdim=True) + s.rms_eps)
    pos = torch.arange(rows, dtype=torch.float32)
    ang = pos[:, None] * net.inv_freq.cpu()[None, :]
    r = lambda t: t.to(torch.bfloat16).float()
    cs, sn = r(torch.cos(ang) * net.rope_scale)[:, None, :], r(torch.sin(ang) * net.rope_scale)[:, None, :]
    i = torch.arange(rows)[:, None]
    j = torch.arange(rows)[None, :]
    ok = ((i < prompt_len) & (j < prompt_len)) | ((i >= prompt_len) & (j <= i))

    def rope(x):
        x = x.reshape(rows, nh, d)
        a, b = x[..., : d // 2], x[..., d // 2:]
        return torch.cat([a * cs - b * sn, b * cs + a * sn], dim=-1)

    high = f32(w.embed)[torch.tensor(ids)] * net.embedding_scale
    low = f32(net.z_l)[None, :].expand(rows, -1).clone()
    for is_high, _ in net.program:
        target, other = (high, low) if is_high else (low, high)
        x = target + other
        n = norm(x)
        base = net.per if is_high else 0
        for layer in range(net.per):
            lw = w.layers[base + layer]
            p = n @ f32(lw.wqkv).t()
            q, k = rope(p[:, :h]), rope(p[:, h:2 * h])
            v, gate = p[:, 2 * h:3 * h].reshape(rows, nh, d), p[:, 3 * h:]
            sc = torch.einsum("ihd,jhd->hij", q, k) / math.sqrt(d)
            sc = sc.masked_fill(~ok[None], float("-inf"))
            a = torch.einsum("hij,jhd->ihd", torch.softmax(sc, -1), v).reshape(rows, h)
            x = x + (a * torch.sigmoid(gate)) @ f32(lw.wo).t()
            n = norm(x)
            gu = n @ f32(lw.wgu).t()
            f = gu.shape[1] // 2
            x = x + (torch.nn.functional.silu(gu[:, :f]) * gu[:, f:]) @ f32(lw.wdown).t()
            n = norm(x)
        if is_high:
            high = n
        else:
            low = n
    return high[-1] @ f32(w.lm_head).t()


def _check_against_reference(m, prompts, outs, tol=0.05):
    net = m.engine.model
    for p, out in zip(prompts, outs):
        for t, tok in enumerate(out):
            lg = _ref_logits(net, list(p) + list(out[:t]), len(p))
            best = int(lg.argmax())
            if best != tok:
                margin = float(lg[best] - lg[tok])
                assert margin <= tol * float(lg.abs().max()), f"step {t}: {tok} vs {best}, margin {margin}"
                break


def test_program_and_yarn_table():
    spec = named_shape("loopvl-text-shape")
    assert spec.layers == 128 and spec.heads == spec.kv_heads == 12 and abs(spec.extra["hrm"]["embedding_scale"] - 39.191835884530846) < 1e-12
    m = _load("cpu")
    net = m.engine.model
    assert net.program == [(False, 0), (False, 2), (False, 4), (True, 6), (False, 8), (False, 10), (False, 12), (True, 14)]
    assert len(net.w.layers) == 4 and m.engine.kv.k[0].shape[0] > 0 and len(m.engine.kv.k) == 16
    # published geometry: interpolation ramp between the beta_fast and beta_slow rotation counts
    inv = yarn_inv_freq(128, 1e4, 2.0, 4096, 32.0, 1.0)
    base = 1.0 / torch.pow(torch.tensor(1e4), torch.arange(64, dtype=torch.float32) * 2 / 128)
    corr = lambda rot: 128 * math.log(4096 / (rot * 2 * math.pi)) / (2 * math.log(1e4))
    lo, hi = math.floor(corr(32.0)), math.ceil(corr(1.0))
    assert torch.allclose(inv[:lo], base[:lo].to(torch.bfloat16).float())
    assert torch.allclose(inv[hi:], (base[hi:] / 2).to(torch.bfloat16).float())
    assert abs(net.rope_scale - (0.1 * math.log(2.0) + 1.0)) < 1e-12


def test_engine_matches_full_sequence_reference_cpu():
    p = _prompts()
    m = _load("cpu")
    outs = m.generate_batch(p, 6)
    _check_against_reference(m, p, outs, tol=1e-3)
    # the same sequences one at a time give the same tokens (packing does not leak between sequences)
    assert [_load("cpu").generate_batch([q], 6)[0] for q in p] == outs


def test_prompts_are_never_split_over_chunks():
    p = _prompts()
    want = _load("cpu").generate_batch(p, 4)
    # 40-row chunks: the 37-token prompt fills the first chunk, the 9-token prompt waits for the second
    got = _load("cpu", chunk=40).generate_batch(p, 4)
    assert got == want
    with pytest.raises(ValueError, match="does not fit one prefill chunk"):
        _load("cpu", chunk=32).generate_batch(p, 2)


def test_sigmoid_gate_oracle():
    g = torch.Generator().manual_seed(1)
    a, gate = torch.randn(5, 16, generator=g), torch.randn(5, 48, generator=g)
    assert torch.allclose(vision_ops.sigmoid_gate(a, gate[:, 16:32]), a * torch.sigmoid(gate[:, 16:32]))


@pytest.mark.gpu
def test_sigmoid_gate_kernel(cuda):
    g = torch.Generator().manual_seed(2)
    a = torch.randn(77, 256, generator=g).to(torch.bfloat16)
    wide = torch.randn(77, 1024, generator=g).to(torch.bfloat16)
    want = vision_ops.sigmoid_gate(a, wide[:, 768:])
    got = vision_ops.sigmoid_gate(a.to(cuda), wide.to(cuda)[:, 768:])
    assert (got.float().cpu() - want.float()).abs().max() < 2e-2


@pytest.mark.gpu
def test_model_gpu_matches_reference(cuda):
    p = _prompts()
    cpu, gpu = _load("cpu"), _load("cuda")
    got = gpu.generate_batch(p, 6)
    ops.check_status()
    _check_against_reference(cpu, p, got, tol=0.05)
    graphs = Model.load("loop-tiny", Settings(capacity=256, max_batch=4, graph=True), device="cuda", seed=0)
    assert graphs.generate_batch(p, 6) == got and graphs.engine.stats["graph_replays"] > 0
