"""Latent window attention (FP8 ring, per-head sink, blocked soft-max, inverse rotary): CPU oracle
properties and CUDA kernels against the oracle."""
import math

import pytest
import torch

from flyingfish_b200.ops import latent_ops as lo


def _setup(b, heads, d, window, positions, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    codes = torch.zeros(b, window, d, dtype=torch.uint8)
    scales = torch.full((b, window, d // 32), 127, dtype=torch.uint8)
    ring_ids = torch.arange(b, dtype=torch.int32)
    # write every position 0..pos of every sequence
    for i, pos in enumerate(positions):
        rows = (torch.randn(pos + 1, d, generator=g) * 1.5).to(torch.bfloat16)
        lo.ring_write(rows, torch.full((pos + 1,), i, dtype=torch.int32), torch.arange(pos + 1, dtype=torch.int32), codes, scales)
    q = torch.randn(b, heads, d, generator=g).to(torch.bfloat16)
    sink = torch.randn(heads, generator=g)
    pos_t = torch.tensor(positions, dtype=torch.int32)
    return [t.to(device) for t in (q, codes, scales, ring_ids, pos_t, sink)]


def test_quant32_codec_roundtrip_and_scale_rule():
    x = torch.tensor([[0.0] * 32 + [448.0] + [1.0] * 31 + [1e-6] * 32 + [3.0, -1000.0] + [0.5] * 30], dtype=torch.float32)
    codes, scales = lo.quant32_ref(x.to(torch.bfloat16))
    assert scales.tolist()[0][0] == 127 + math.ceil(math.log2(1e-4 / 448))       # all-zero group: floor at 1e-4
    assert scales.tolist()[0][1] == 127                                           # amax 448 -> scale 1
    back = lo.dequant32(codes, scales)
    assert back[0, 32].item() == 448.0 and back[0, 33].item() == 1.0
    assert back[0, 97].item() < -900.0                                            # -1000 survives with a power-of-two scale
    assert (back - x.to(torch.bfloat16).float()).abs().max() <= 64.0              # e4m3 step at 1000 is 64


def test_window_attention_oracle_sink_and_wraparound():
    # window 8, position 11: visible slots are positions 4..11, oldest first
    q, codes, scales, rid, pos, sink = _setup(1, 2, 64, 8, [11], seed=1)
    out = lo.window_attention(q, codes, scales, rid, pos, sink, rope_tail=0, theta=1e4)
    # a huge sink logit takes all the probability mass: output -> 0
    big = lo.window_attention(q, codes, scales, rid, pos, torch.full_like(sink, 80.0), rope_tail=0, theta=1e4)
    assert out.abs().max() > 0.05 and big.abs().max() < 1e-3
    # inverse rotary only touches the tail
    rot = lo.window_attention(q, codes, scales, rid, pos, sink, rope_tail=16, theta=1e4)
    assert torch.equal(rot[..., :48], out[..., :48]) and not torch.equal(rot[..., 48:], out[..., 48:])
    n0 = out[..., 48:].float().reshape(1, 2, 8, 2).norm(dim=-1)
    n1 = rot[..., 48:].float().reshape(1, 2, 8, 2).norm(dim=-1)
    assert torch.allclose(n0, n1, rtol=2e-2, atol=2e-2)                            # a rotation keeps pair norms


@pytest.mark.gpu
@pytest.mark.parametrize("b,heads,d,window,positions,tail", [
    (2, 16, 512, 128, [40, 300], 64), (3, 20, 256, 64, [0, 63, 64], 32), (1, 64, 512, 256, [1000], 64), (2, 8, 64, 200, [199, 77], 0)])
def test_latent_window_attention_cuda_matches_oracle(b, heads, d, window, positions, tail):
    from flyingfish_b200 import ops
    q, codes, scales, rid, pos, sink = _setup(b, heads, d, window, positions, seed=3)
    want = lo.window_attention(q, codes, scales, rid, pos, sink, tail, 1e4)
    got = lo.window_attention(*(t.cuda() for t in (q, codes, scales, rid, pos, sink)), tail, 1e4)
    ops.check_status()
    err = (got.float().cpu() - want.float()).abs()
    assert err.max().item() <= 2e-2 + 2e-2 * want.float().abs().max().item(), err.max().item()


@pytest.mark.gpu
def test_latent_quant_cuda_bit_exact():
    from flyingfish_b200 import ops
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(37, 512, generator=g) * torch.logspace(-3, 3, 37)[:, None]).to(torch.bfloat16)
    x[3, 64:96] = 0
    c_ref, s_ref = lo.quant32_ref(x)
    c, s = lo.act_quant(x.cuda())
    ops.check_status()
    assert torch.equal(s.cpu(), s_ref) and torch.equal(c.cpu(), c_ref)
    codes = torch.zeros(2, 16, 512, dtype=torch.uint8, device="cuda"); scales = torch.zeros(2, 16, 16, dtype=torch.uint8, device="cuda")
    rid = torch.tensor([1, 0, 1], dtype=torch.int32, device="cuda"); pos = torch.tensor([5, 21, 16], dtype=torch.int32, device="cuda")
    lo.ring_write(x[:3].cuda(), rid, pos, codes, scales)
    assert torch.equal(codes[1, 5].cpu(), c_ref[0]) and torch.equal(codes[0, 5].cpu(), c_ref[1]) and torch.equal(codes[1, 0].cpu(), c_ref[2])
