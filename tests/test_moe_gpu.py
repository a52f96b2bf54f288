"""MoE kernels against the FP32 oracle: router variants (ties -> lower id), dispatch + grouped
GEMM + combine, end-to-end MoE decoders on the GPU."""
import pytest
import torch

from flyingfish_b200 import ops
from flyingfish_b200.ops import moe_ops, ref

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(BF16)


@pytest.mark.parametrize("score,E,k,groups,tg", [("softmax", 8, 2, 1, 1), ("softmax", 128, 8, 1, 1),
                                                 ("sigmoid", 64, 4, 1, 1), ("noaux", 256, 8, 8, 4),
                                                 ("noaux", 16, 4, 4, 2)])
def test_route_matches_oracle(score, E, k, groups, tg):
    rows, hidden = 37, 512
    x, w = _rand((rows, hidden), 1), _rand((E, hidden), 2, 0.1)
    bias = (torch.randn(E, generator=torch.Generator().manual_seed(3)) * 0.1) if score == "noaux" else None
    ew, ei = ref.moe_route(x, w, k, score, bias, groups, tg, 2.5 if score == "noaux" else 1.0)
    gw, gi = moe_ops.route(x.cuda(), w.cuda(), k, score, None if bias is None else bias.cuda(), groups, tg,
                           2.5 if score == "noaux" else 1.0)
    ops.check_status()
    # the GPU logits are BF16-rounded from a tensor-core accumulation; compare selections as sets
    # and weights loosely, exact equality where the oracle's margins are not razor thin
    same = (gi.cpu().sort(-1).values == ei.sort(-1).values).all(-1).float().mean().item()
    assert same > 0.9
    m = (gi.cpu() == ei).all(-1)
    assert torch.allclose(gw.cpu()[m], ew[m], rtol=3e-2, atol=3e-3)


def test_route_ties_go_to_lower_id():
    x = torch.zeros(4, 256, dtype=BF16)
    w = _rand((32, 256), 4)
    gw, gi = moe_ops.route(x.cuda(), w.cuda(), 4, "softmax")
    assert gi.cpu().tolist() == [[0, 1, 2, 3]] * 4
    assert torch.allclose(gw.cpu(), torch.full((4, 4), 0.25))


@pytest.mark.parametrize("rows,E,k,h,f", [(5, 8, 2, 256, 128), (300, 16, 4, 512, 256), (64, 32, 8, 1024, 512),
                                          (1000, 4, 2, 256, 192), (2000, 8, 2, 512, 256), (3000, 8, 4, 512, 384)])
def test_experts_forward(rows, E, k, h, f):
    x = _rand((rows, h), 5)
    wgu, wd = _rand((E, 2 * f, h), 6, 0.05), _rand((E, h, f), 7, 0.05)
    g = torch.Generator().manual_seed(8)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(rows)]).to(torch.int32)
    wts = torch.rand(rows, k, generator=g)
    wts = wts / wts.sum(-1, keepdim=True)
    got = moe_ops.experts_forward(x.cuda(), wts.cuda(), ids.cuda(), wgu.cuda(), wd.cuda(), 0)
    torch.cuda.synchronize()
    ops.check_status()
    expect = ref.moe_forward(x, wts, ids, wgu, wd, None, None, 0)
    err = (got.float().cpu() - expect.float()).abs()
    tol = 2e-2 + 3e-2 * expect.float().abs()
    assert (err <= tol).all(), f"max err {err.max().item()}"
    again = moe_ops.experts_forward(x.cuda(), wts.cuda(), ids.cuda(), wgu.cuda(), wd.cuda(), 0)
    assert torch.equal(got, again), "MoE forward must be deterministic"


@pytest.mark.parametrize("name", ["qwen3-moe-tiny"])
def test_moe_model_gpu_matches_cpu(name):
    from flyingfish_b200.api import Model, generate_plain
    from flyingfish_b200.config import Settings
    g = torch.Generator().manual_seed(9)
    ids = torch.randint(0, 2048, (30,), generator=g).tolist()
    m = Model.load(name, Settings(capacity=256, max_batch=4), device="cuda", seed=0)
    a = generate_plain(m, ids, 8, ignore_eos=True, graph=False).ids
    m.reset()
    b = generate_plain(m, ids, 8, ignore_eos=True, graph=True).ids
    assert a == b, "eager and graph decode must agree bitwise"


@pytest.mark.parametrize("rows,E,k,h,f", [(7, 8, 2, 512, 256), (64, 16, 4, 1024, 512), (200, 4, 2, 256, 256)])
def test_experts_forward_nvfp4(rows, E, k, h, f):
    """Packed NVFP4 experts expanded inside the grouped GEMM against the oracle on the dequantised weights."""
    from flyingfish_b200.loaders import quant
    from flyingfish_b200.ops import moe_cuda
    x = _rand((rows, h), 5)
    wgu, wd = _rand((E, 2 * f, h), 6, 0.05), _rand((E, h, f), 7, 0.05)
    g = torch.Generator().manual_seed(8)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(rows)]).to(torch.int32)
    wts = torch.rand(rows, k, generator=g)
    wts = wts / wts.sum(-1, keepdim=True)
    qgu = [quant.quantize_nvfp4(wgu[e].float()) for e in range(E)]
    qd = [quant.quantize_nvfp4(wd[e].float()) for e in range(E)]
    dq_gu = torch.stack([quant.dequantize_nvfp4(*q) for q in qgu])
    dq_d = torch.stack([quant.dequantize_nvfp4(*q) for q in qd])
    st = lambda qs, i: torch.stack([q[i] for q in qs]).cuda()
    gu = moe_cuda.Nvfp4Experts(st(qgu, 0), st(qgu, 1), st(qgu, 2), gate_up=True)
    dn = moe_cuda.Nvfp4Experts(st(qd, 0), st(qd, 1), st(qd, 2))
    assert gu.supported() and dn.supported() and gu.nbytes() * 3 < wgu.numel() * 2
    got = moe_cuda.experts_forward_nvfp4(x.cuda(), wts.cuda(), ids.cuda(), gu, dn)
    torch.cuda.synchronize()
    ops.check_status()
    expect = ref.moe_forward(x, wts, ids, dq_gu, dq_d, None, None, 0)
    err = (got.float().cpu() - expect.float()).abs()
    # the kernel applies the per-expert global scale in FP32, the oracle folds it into BF16-rounded weights
    tol = 4e-2 + 4e-2 * expect.float().abs()
    assert (err <= tol).all(), f"max err {err.max().item()}"
    again = moe_cuda.experts_forward_nvfp4(x.cuda(), wts.cuda(), ids.cuda(), gu, dn)
    assert torch.equal(got, again)


def test_model_with_packed_nvfp4_experts():
    """Decode steps of an NVFP4-expert model run on the packed experts (prefill on their BF16 expansion)."""
    from flyingfish_b200.api import Model, generate_plain
    from flyingfish_b200.config import Settings
    from flyingfish_b200.ops import moe_cuda
    m = Model.load("qwen3-moe-fp4-tiny", Settings(capacity=256, max_batch=4, graph=False), device="cuda", seed=0)
    lw = m.engine.model.w.layers[0]
    gu, dn = lw.extra["experts_fp4"]
    assert gu.codes.shape == (16, 512, 256) and dn.codes.shape == (16, 512, 128)
    # the packed stack reproduces the BF16 experts to FP4 precision
    from flyingfish_b200.ops.quant_ops import dequant_nvfp4
    back = dequant_nvfp4(dn.codes[3], dn.scales[3], dn.global_scale[3])
    rel = (back.float() - lw.experts_down[3].float()).abs().mean() / lw.experts_down[3].float().abs().mean()
    assert rel < 0.15, rel
    calls = {"n": 0}
    orig = moe_cuda.experts_forward_nvfp4

    def spy(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)
    moe_cuda.experts_forward_nvfp4 = spy
    try:
        ids = list(range(3, 40))
        a = generate_plain(m, ids, 6, ignore_eos=True, graph=False).ids
        m.reset()
        b = generate_plain(m, ids, 6, ignore_eos=True, graph=False).ids
    finally:
        moe_cuda.experts_forward_nvfp4 = orig
    assert a == b and calls["n"] >= 2 * 5            # five decode steps x two MoE layers per run, at least
    ops.check_status()


@pytest.mark.parametrize("name", ["qwen3-moe-tiny", "qwen3-moe-fp4-tiny"])
def test_tiered_provider_gpu_half_resident(name):
    """Half of the experts in GPU slots (BF16 slots, or packed NVFP4 slots for an NVFP4-expert model), the rest served
    by the host FFN: decode goes through the device-resolved provider path (one summary copy per layer call, array
    accounting, per-layer copy events) and must produce what the all-resident model produces, up to the first
    near-tie (host FFN arithmetic differs from the tensor-core path in the last bits)."""
    from flyingfish_b200.api import Model, generate_plain
    from flyingfish_b200.config import Settings
    from flyingfish_b200.experts.provider import build_provider_from_weights
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 2048, (24,), generator=g).tolist()
    m = Model.load(name, Settings(capacity=256, max_batch=2, graph=False), device="cuda", seed=0)
    plain = generate_plain(m, ids, 10, ignore_eos=True, graph=False).ids
    m.reset()
    prov = build_provider_from_weights(m.engine.model, resident_fraction=0.5, threads=2, admission_cap=2)
    assert prov.fp4 == (name == "qwen3-moe-fp4-tiny")
    prov.collect_freq = True
    seq = m.engine.add_sequence(ids)
    first = m.engine.prefill([seq])[0]
    prov.collect_freq = False
    prov.begin_request()
    for key in ("hits", "host_misses", "disk_misses"):
        prov.res.stats[key] = 0
    out = [first] + [m.engine.decode([seq])[0] for _ in range(9)]
    torch.cuda.synchronize()
    ops.check_status()
    agree = 0
    for a, b in zip(out, plain):
        if a != b:
            break
        agree += 1
    # an NVFP4 model prefills on the BF16 expansion when all-resident but on FP4-effective weights through the
    # provider, so only the BF16 case is held to (near) token equality
    assert agree >= (6 if name == "qwen3-moe-tiny" else 1), (out, plain)
    st = prov.res.stats
    assert st["tokens"] == 9 and st["hits"] > 0 and st["host_misses"] > 0 and prov.res.hit_rate() > 0.3
    assert prov.stats["d2h_summary_bytes"] > 0 and prov.stats["cpu_rows"] > 0 and prov.stats["gpu_rows"] > 0
    # slots were changed at token boundaries and the next token waited only on its layer's event
    assert prov.stats["h2d_expert_bytes"] > 0
