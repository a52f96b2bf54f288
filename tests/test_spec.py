"""Speculative decoding: acceptance rules, chain speculation equals plain greedy, transactional
behaviour under injected faults, tree construction."""
import pytest
import torch

from flyingfish_b200.api import Model, generate_plain
from flyingfish_b200.config import Settings
from flyingfish_b200.spec.accept import accept_chain, accept_tree
from flyingfish_b200.spec.chain import ChainSpeculator, Fault, SpecFault


def test_accept_chain_rules():
    a = accept_chain([5, 6, 7], [5, 6, 9, 1])
    assert a.tokens == [5, 6, 9] and a.n_draft_accepted == 2
    a = accept_chain([5, 6, 7], [5, 6, 7, 8])
    assert a.tokens == [5, 6, 7, 8] and a.n_draft_accepted == 3
    a = accept_chain([5], [4, 0])
    assert a.tokens == [4] and a.n_draft_accepted == 0
    a = accept_chain([5, 2, 7], [5, 2, 7, 8], eos_ids=(2,), ignore_eos=False)
    assert a.tokens == [5, 2] and a.hit_eos


def test_accept_tree_follows_matching_child():
    #        0
    #      1   2
    #     3 4   5
    parents = [-1, 0, 0, 1, 1, 2]
    tokens = [0, 10, 11, 20, 21, 22]
    target = [11, 0, 22, 0, 0, 33]
    acc, path = accept_tree(parents, tokens, target)
    assert path == [0, 2, 5] and acc.tokens == [11, 22, 33] and acc.n_draft_accepted == 2
    acc, path = accept_tree(parents, tokens, [99, 0, 0, 0, 0, 0])
    assert path == [0] and acc.tokens == [99]


def _models(k_target="tiny-llama", k_draft="tiny-llama", seed_draft=0):
    st = Settings(capacity=256, max_batch=2, graph=False)
    t = Model.load(k_target, st, device="cpu", seed=0)
    d = Model.load(k_draft, Settings(capacity=256, max_batch=2, graph=False), device="cpu", seed=seed_draft)
    return t, d


@pytest.mark.parametrize("seed_draft,k", [(0, 3), (0, 5), (7, 4)])
def test_chain_speculation_equals_greedy(seed_draft, k):
    """With an identical draft every token is accepted; with a different draft almost none are --
    in both cases the emitted stream must equal plain greedy decoding."""
    t, d = _models(seed_draft=seed_draft)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 2048, (21,), generator=g).tolist()
    plain = generate_plain(t, ids, 17, ignore_eos=True, graph=False).ids
    t.reset()
    spec = ChainSpeculator(t, d, k=k)
    out = spec.generate(ids, 17)
    assert out.ids == plain
    if seed_draft == 0:
        assert spec.stats.acceptance_rate == 1.0 and spec.stats.tokens_per_round > k * 0.9
    else:
        assert spec.stats.acceptance_rate < 0.5


@pytest.mark.parametrize("fault", [Fault.DRAFT, Fault.VERIFY, Fault.COMMIT])
def test_faults_leave_committed_state_intact(fault):
    t, d = _models()
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, 2048, (15,), generator=g).tolist()
    plain = generate_plain(t, ids, 12, ignore_eos=True, graph=False).ids
    t.reset()
    spec = ChainSpeculator(t, d, k=3)
    te, de = t.engine, d.engine
    ts, ds = te.add_sequence(ids), de.add_sequence(ids)
    first = te.prefill([ts])[0]
    de.prefill([ds]); ds.output.clear(); ds.pending = first
    out = [first]
    out += spec._round(ts, ds, 3, (), True)
    lens = (te.kv.seqs[ts.seq_id].length, de.kv.seqs[ds.seq_id].length, list(ts.output))
    spec.fault = fault
    with pytest.raises(SpecFault):
        spec._round(ts, ds, 3, (), True)
    assert (te.kv.seqs[ts.seq_id].length, de.kv.seqs[ds.seq_id].length, list(ts.output)) == lens
    spec.fault = Fault.NONE
    ds.output.clear(); ds.pending = ts.pending
    while len(out) < 12:
        out += spec._round(ts, ds, 3, (), True)
    assert out[:12] == plain


def test_mtp_speculation_equals_greedy():
    from flyingfish_b200.spec.mtp import MtpSpeculator
    t = Model.load("tiny-llama", Settings(capacity=256, max_batch=2, graph=False), device="cpu", seed=0)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 2048, (19,), generator=g).tolist()
    plain = generate_plain(t, ids, 14, ignore_eos=True, graph=False).ids
    t.reset()
    for depth in (1, 3):
        spec = MtpSpeculator(t, depth=depth, seed=11)
        out = spec.generate(ids, 14)
        assert out.ids == plain
        assert spec.stats.rounds > 0 and spec.kv.seqs[0].length <= len(ids) + 14
        t.reset()


def test_mtp_fault_is_transactional():
    from flyingfish_b200.spec.mtp import MtpSpeculator
    t = Model.load("tiny-llama", Settings(capacity=256, max_batch=2, graph=False), device="cpu", seed=0)
    spec = MtpSpeculator(t, depth=2, seed=11)
    ids = list(range(5, 25))
    plain = generate_plain(t, ids, 9, ignore_eos=True, graph=False).ids
    t.reset()
    spec.fault = Fault.VERIFY
    with pytest.raises(SpecFault):
        spec.generate(ids, 9)
    spec.fault = Fault.NONE
    t.reset()
    assert spec.generate(ids, 9).ids == plain


def test_tree_builder_budget_masks_and_order():
    from flyingfish_b200.spec.tree import VerifyCostSchedule, build_tree
    import math

    def children(paths):
        outs = []
        for p in paths:
            base = sum(p) % 7
            outs.append([(100 + base + i, math.log(w)) for i, w in enumerate([0.5, 0.3, 0.15, 0.05])])
        return outs

    for builder in ("waves", "serial"):
        t = build_tree(1, children, 16, builder)
        assert len(t) == 16 and t.parents[0] == -1
        t.check()
        for r in range(1, len(t)):
            assert t.masks[r] & (1 << t.parents[r]) and t.masks[r] & 1        # parent and root visible
            assert bin(t.masks[r]).count("1") == t.depth[r] + 1
        assert t.positions(50)[0] == 50 and max(t.positions(50)) <= 50 + 7
    s = build_tree(1, children, 8, "serial")
    assert all(s.logp[i] >= s.logp[i + 1] - 1e-9 for i in range(1, len(s) - 1)), "serial builder is best-first"
    assert len(build_tree(1, children, 1)) == 1
    sched = VerifyCostSchedule(tau=0.8, miss_cost_ms=0.5, step_ms=1.0, expected_new_experts_per_row=1.0)
    assert sched.select_rows([0.99, 0.98, 0.97, 0.2, 0.9]) <= 5
    assert sched.select_rows([0.1]) == 2
    assert VerifyCostSchedule().select_rows([0.95] * 10) == 8


@pytest.mark.parametrize("seed_draft,builder", [(0, "waves"), (0, "serial"), (5, "waves")])
def test_tree_speculation_equals_greedy(seed_draft, builder):
    from flyingfish_b200.spec.tree_spec import TreeSpeculator
    t, d = _models(seed_draft=seed_draft)
    g = torch.Generator().manual_seed(6)
    ids = torch.randint(0, 2048, (13,), generator=g).tolist()
    plain = generate_plain(t, ids, 12, ignore_eos=True, graph=False).ids
    t.reset()
    spec = TreeSpeculator(t, d, "tree16", builder)
    out = spec.generate(ids, 12)
    assert out.ids == plain
    if seed_draft == 0:
        assert spec.stats.accepted > 0, "an identical draft model must get tokens accepted"
