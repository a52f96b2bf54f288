"""End-to-end engine checks on a GPU: CPU-oracle agreement, eager == graph, chunk invariance."""
import pytest
import torch

from flyingfish_b200.api import Model, generate_plain
from flyingfish_b200.config import Settings

pytestmark = pytest.mark.gpu


def _prompt(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def _load(device, **kw):
    return Model.load("tiny-llama", Settings(capacity=512, max_batch=8, **kw), device=device, seed=0)


def test_logits_match_cpu_oracle():
    """First-token logits of the CUDA path agree with the FP32-math CPU oracle on the same weights."""
    from flyingfish_b200.models.weights import random_decoder_weights
    from flyingfish_b200.models.decoder import DecoderModel
    from flyingfish_b200.engine.engine import Engine
    from flyingfish_b200.config import named_shape
    spec = named_shape("tiny-llama")
    w_cpu = random_decoder_weights(spec, 0, "cpu")
    import copy
    w_gpu = copy.deepcopy(w_cpu)
    for l in w_gpu.layers:
        for k, v in vars(l).items():
            if isinstance(v, torch.Tensor):
                setattr(l, k, v.cuda())
    w_gpu.embed, w_gpu.final_norm, w_gpu.lm_head = w_gpu.embed.cuda(), w_gpu.final_norm.cuda(), w_gpu.lm_head.cuda()
    ids = _prompt(spec.vocab, 77, 1)
    outs = []
    for w, dev in ((w_cpu, "cpu"), (w_gpu, "cuda")):
        eng = Engine(DecoderModel(w), spec, Settings(capacity=512, max_batch=4, graph=False), 32, dev)
        s = eng.add_sequence(ids)
        fb = eng.prefill_batch
        sl = eng.kv.reserve(s.seq_id, len(ids))
        fb.fill(ids=ids, positions=list(range(len(ids))), slots=sl, q_lens=[len(ids)], ctx_lens=[len(ids)],
                block_rows=[eng.kv.seqs[s.seq_id].blocks], logit_rows=[len(ids) - 1], is_decode=False)
        fb.upload()
        outs.append(eng.model.forward(fb, eng.kv, return_logits=True).float().cpu())
    err = (outs[0] - outs[1]).abs().max().item()
    scale = outs[0].abs().max().item()
    assert err < 0.05 * max(scale, 1.0), f"logit error {err} (scale {scale})"


def test_eager_equals_graph_bitwise():
    ids = _prompt(2048, 40, 2)
    m = _load("cuda")
    a = generate_plain(m, ids, 24, ignore_eos=True, graph=False).ids
    m.reset()
    b = generate_plain(m, ids, 24, ignore_eos=True, graph=True).ids
    assert a == b
    assert m.engine.stats["graph_replays"] > 0


def test_chunked_prefill_invariance_and_batching():
    ids = _prompt(2048, 150, 3)
    m = _load("cuda")
    a = generate_plain(m, ids, 8, ignore_eos=True, graph=False).ids
    m.reset()
    m.settings.chunk = 64
    b = generate_plain(m, ids, 8, ignore_eos=True, graph=False).ids
    assert a == b, "results must not depend on the prefill chunking"
    m.reset()
    m.settings.chunk = None
    outs = m.generate_batch([ids, ids[:33], ids[:5]], 8)
    assert outs[0] == a


def test_poisoning_after_injected_failure():
    from flyingfish_b200.engine.engine import EnginePoisoned
    m = _load("cuda")
    m.prefill(_prompt(2048, 10, 4))
    m.engine.fail_next_step = True
    with pytest.raises(RuntimeError):
        m.decode()
    with pytest.raises(EnginePoisoned):
        m.decode()
    m.reset()
    m.prefill(_prompt(2048, 10, 4))
    m.decode()


def test_speculation_on_gpu_equals_greedy():
    """Chain (draft model), MTP and tree speculation through the CUDA kernels (multi-row verify
    via the prefill kernel, tree verify via the masked decode kernel) reproduce plain greedy."""
    from flyingfish_b200.spec.chain import ChainSpeculator
    from flyingfish_b200.spec.mtp import MtpSpeculator
    from flyingfish_b200.spec.tree_spec import TreeSpeculator
    ids = _prompt(2048, 35, 9)
    t = _load("cuda", graph=False)
    d = _load("cuda", graph=False)
    plain = generate_plain(t, ids, 16, ignore_eos=True, graph=False).ids
    t.reset()
    spec = ChainSpeculator(t, d, k=4)
    assert spec.generate(ids, 16).ids == plain
    assert spec.stats.acceptance_rate == 1.0
    t.reset(); d.reset()
    assert MtpSpeculator(t, depth=2, seed=3).generate(ids, 16).ids == plain
    t.reset()
    tree = TreeSpeculator(t, d, "tree32", "waves")
    assert tree.generate(ids, 16).ids == plain
    assert tree.stats.accepted > 0


def test_verification_replays_from_a_cuda_graph():
    """With graphs on, the multi-row verification step of chain / MTP speculation is captured per (bucket, rows) and
    replayed (decode-style attention over the rows); the emitted stream is still plain greedy decoding."""
    from flyingfish_b200.spec.chain import ChainSpeculator
    from flyingfish_b200.spec.mtp import MtpSpeculator
    ids = _prompt(2048, 35, 9)
    t = _load("cuda", graph=True)
    d = _load("cuda", graph=True)
    plain = generate_plain(t, ids, 16, ignore_eos=True, graph=True).ids
    t.reset()
    spec = ChainSpeculator(t, d, k=4)
    assert spec.generate(ids, 16).ids == plain
    assert t.engine.stats.get("verify_graph_replays", 0) > 0 and (1, 5) in t.engine.graphs
    t.reset(); d.reset()
    before = t.engine.stats["verify_graph_replays"]
    assert MtpSpeculator(t, depth=2, seed=3).generate(ids, 16).ids == plain
    assert t.engine.stats["verify_graph_replays"] > before
    # eager verification of the same drafts gives the same tokens
    t.reset()
    e = _load("cuda", graph=False)
    sa, sb = t.engine.add_sequence(ids), e.engine.add_sequence(ids)
    t.engine.prefill([sa]); e.engine.prefill([sb])
    drafts = [plain[1:4]]                              # the true continuation: every row's successor is known
    assert t.engine.verify([sa], drafts) == e.engine.verify([sb], drafts) == [plain[1:5]]
