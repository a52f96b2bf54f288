"""Decode projection chain (one persistent kernel per layer) against the operator-by-operator path and an FP32
reference of the same layer program."""
import pytest
import torch

from flyingfish_b200 import ops
from flyingfish_b200.ops import ref

pytestmark = pytest.mark.gpu

HQ, HKV, D, HIDDEN, FFN = 4, 2, 128, 1024, 1536
EPS = 1e-5


def _weights(seed: int, dev):
    g = torch.Generator().manual_seed(seed)
    def rnd(*shape, std=0.05):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).to(dev)
    wg, wu = rnd(FFN, HIDDEN), rnd(FFN, HIDDEN)
    return {"wo": rnd(HIDDEN, HQ * D), "post_ln": (1 + rnd(HIDDEN, std=0.1)), "wgu": ref.interleave_gate_up(wg, wu),
            "wdown": rnd(HIDDEN, FFN), "next_ln": (1 + rnd(HIDDEN, std=0.1)), "wqkv": rnd((HQ + 2 * HKV) * D, HIDDEN)}


def _unfused(a, res, w, positions, slots, kc, vc, cs, with_qkv):
    o = ops.linear(a, w["wo"])
    n = ops.add_rmsnorm(o, res, w["post_ln"], EPS)
    h = ops.linear_swiglu(n, w["wgu"])
    dn = ops.linear(h, w["wdown"])
    n2 = ops.add_rmsnorm(dn, res, w["next_ln"], EPS)
    qkv = None
    if with_qkv:
        qkv = ops.linear_rope_kv(n2, w["wqkv"], positions, slots, kc, vc, HQ, HKV, D, 5e5, cos_sin=cs)
    return n2, qkv


@pytest.mark.parametrize("m", [1, 8, 64, 128])
@pytest.mark.parametrize("with_qkv", [True, False])
def test_layer_chain_matches_operator_path(m, with_qkv):
    from flyingfish_b200.ops import chain
    dev = torch.device("cuda", 0)
    w = _weights(3, dev)
    g = torch.Generator().manual_seed(10 + m)
    a = torch.randn(m, HQ * D, generator=g).to(torch.bfloat16).to(dev)
    res0 = torch.randn(m, HIDDEN, generator=g).to(torch.bfloat16).to(dev)
    positions = torch.arange(100, 100 + m, dtype=torch.int32, device=dev)
    nb, bs = 8, 64
    slots = (torch.randperm(nb * bs, generator=g)[:m]).to(torch.int32).to(dev)
    cs = ops.rope_table(positions, D, 5e5)
    outs = []
    for path in ("ops", "chain", "chain"):          # the chain runs twice: its counters carry over between launches
        res = res0.clone()
        kc = torch.zeros(nb, HKV, bs, D, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        if path == "ops":
            n2, qkv = _unfused(a, res, w, positions, slots, kc, vc, cs, with_qkv)
        else:
            rope = {"cos_sin": cs, "slots": slots, "kcache": kc, "vcache": vc, "hq": HQ, "hkv": HKV, "rot_dim": D}
            n2, qkv = chain.layer_chain(a, res, w["wo"], w["post_ln"], w["wgu"], w["wdown"], w["next_ln"], EPS,
                                        w["wqkv"] if with_qkv else None, rope if with_qkv else None)
        torch.cuda.synchronize()
        ops.check_status(dev)
        outs.append((n2.float().cpu(), res.float().cpu(), None if qkv is None else qkv.float().cpu(), kc.float().cpu(),
                     vc.float().cpu()))
    # the two chain launches are bit-identical (deterministic reduction order)
    for x, y in zip(outs[1], outs[2]):
        if x is not None:
            assert torch.equal(x, y)
    # chain vs operator path: same rounding points, different split of K in the FP32 sums
    names = ("normed", "residual", "qkv", "kcache", "vcache")
    for name, x, y in zip(names, outs[0], outs[1]):
        if x is None:
            continue
        err = (x - y).abs()
        assert (err <= 3e-2 + 3e-2 * x.abs()).all(), f"{name}: max err {err.max().item()}"
        assert (err > 0).float().mean().item() < 0.2, f"{name}: too many differing elements"


def test_model_decode_chain_equals_operator_path():
    """Greedy decode of the tiny dense decoder through the chain equals the operator-by-operator path, eagerly and
    from a CUDA graph."""
    from flyingfish_b200.api import Model, generate_plain
    from flyingfish_b200.config import Settings
    from flyingfish_b200.ops import chain
    prompt = list(range(5, 45))
    toks = {}
    default = chain.ENABLED
    for name, enabled, graph in (("ops", False, False), ("chain", True, False), ("chain_graph", True, True)):
        chain.ENABLED = enabled
        try:
            m = Model.load("tiny-llama", Settings(capacity=256, max_batch=4, graph=graph), device="cuda:0", seed=0)
            ops.reset_launch_count()
            toks[name] = generate_plain(m, prompt, 12, ignore_eos=True, graph=graph).ids
            torch.cuda.synchronize()
            ops.check_status()
        finally:
            chain.ENABLED = default
    assert toks["chain"] == toks["ops"]
    assert toks["chain_graph"] == toks["chain"]
