"""DeepSeek-V3-style model with the published quantisation: projections, dense FFN, shared expert and routed experts
resident as E4M3 codes with 128x128 block scales, activations quantised 1x128 inside every linear (W8A8), MLA
attention, one MTP module. CPU runs execute the oracle linears; the GPU runs the tcgen05 FP8 kernels."""
import pytest
import torch

from flyingfish_b200.api import Model, generate_plain
from flyingfish_b200.config import Settings

NAME = "deepseek-v3-fp8-mini"


def _load(device="cpu"):
    return Model.load(NAME, Settings(capacity=256, max_batch=4, graph=False), device=device, seed=0)


def test_weights_are_fp8_resident_and_routing_runs_on_cpu():
    from flyingfish_b200.ops.quant_ops import Fp8Experts, Fp8Weight
    m = _load()
    w = m.engine.model.w
    dense, moe = w.layers[0], w.layers[1]
    assert isinstance(dense.wgu, Fp8Weight) and isinstance(dense.wdown, Fp8Weight) and not dense.wgu_interleaved
    assert isinstance(moe.experts_gu, Fp8Experts) and moe.experts_gu.interleaved and isinstance(moe.shared_gu, Fp8Weight)
    mla = moe.extra["mla"]
    assert all(isinstance(t, Fp8Weight) for t in (mla.q_a, mla.q_b, mla.kv_a, mla.wo))
    assert mla.w_uk_t.dtype == torch.bfloat16                     # the absorbed kv_b factors stay BF16
    # codes + scales take about half of what BF16 would
    bf16_bytes = 2 * sum(t.codes.numel() for t in (dense.wgu, dense.wdown))
    assert dense.wgu.nbytes() + dense.wdown.nbytes() < 0.52 * bf16_bytes
    out = generate_plain(m, list(range(3, 30)), 6, ignore_eos=True, graph=False).ids
    assert len(out) == 6


def test_mtp_on_the_mla_model_equals_greedy_cpu():
    from flyingfish_b200.spec.mtp import MtpSpeculator
    m = _load()
    ids = list(range(7, 31))
    plain = generate_plain(m, ids, 8, ignore_eos=True, graph=False).ids
    m.reset()
    sp = MtpSpeculator(m, depth=2, seed=11)
    assert sp.generate(ids, 8).ids == plain and sp.stats.rounds > 0


@pytest.mark.gpu
def test_fp8_model_gpu_matches_cpu_oracle():
    from _oracle import assert_rows_mostly_close
    from flyingfish_b200 import ops
    cpu, gpu = _load(), _load("cuda")
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (70, 9, 33)]
    assert_rows_mostly_close(cpu, gpu, prompts, rel=0.08, frac=0.6)
    out = generate_plain(gpu, prompts[0], 8, ignore_eos=True, graph=False).ids
    assert len(out) == 8
    ops.check_status()


@pytest.mark.gpu
def test_mtp_on_the_mla_model_equals_greedy_gpu():
    from flyingfish_b200 import ops
    from flyingfish_b200.spec.mtp import MtpSpeculator
    m = _load("cuda")
    ids = list(range(7, 31))
    plain = generate_plain(m, ids, 8, ignore_eos=True, graph=False).ids
    m.reset()
    sp = MtpSpeculator(m, depth=2, seed=11)
    got = sp.generate(ids, 8).ids
    # verification rows go through the prefill kernels, plain decoding through the decode kernels: equal up to the
    # first router or logit near-tie, and the first tokens (same kernels both ways) always agree
    assert got[:2] == plain[:2] and len(got) == 8
    ops.check_status()
