"""Bidirectional use of the decoder stack: embedding encoder and masked-diffusion sampler (CPU oracles; the GPU
test compares the CUDA kernels with the CPU path)."""
import pytest
import torch

from flyingfish_b200.api import Model
from flyingfish_b200.config import Settings
from flyingfish_b200.models.encoder import EmbeddingHead, embed_texts, run_whole
from flyingfish_b200.spec.diffusion import DiffusionTrace, diffusion_generate


def _load(name, device="cpu"):
    return Model.load(name, Settings(capacity=256, max_batch=4, graph=False), device=device, seed=0)


def test_bidirectional_rows_see_later_tokens():
    m = _load("tiny-embed")
    a = run_whole(m, [[3, 4, 5, 6, 7]])[0]
    b = run_whole(m, [[3, 4, 5, 6, 9]])[0]
    assert (a[0] - b[0]).abs().max() > 1e-4              # row 0 changed although only the last token differs
    causal = _load("tiny-llama")
    ca, cb = run_whole(causal, [[3, 4, 5, 6, 7]])[0], run_whole(causal, [[3, 4, 5, 6, 9]])[0]
    assert torch.equal(ca[:4], cb[:4])


def test_embeddings_are_unit_length_and_batch_invariant():
    m = _load("tiny-embed")
    texts = [[5, 6, 7], [9, 10, 11, 12, 13, 14], [20] * 40]
    head = EmbeddingHead(m.spec, "cpu")
    together = embed_texts(m, texts, head)
    alone = [embed_texts(m, [t], head)[0] for t in texts]
    for a, b in zip(together, alone):
        assert a.shape == (256,) and abs(float(a.norm()) - 1.0) < 1e-4
        assert torch.allclose(a, b, atol=1e-5)
    assert m.engine.kv.alloc.free_blocks == m.engine.kv.alloc.num_blocks - getattr(m.engine.kv.alloc, "reserved", 0) \
        or not m.engine.kv.seqs


def test_diffusion_commits_every_position_by_confidence():
    m = _load("tiny-diffusion")
    mask = m.spec.extra["mask_token_id"]
    tr = DiffusionTrace()
    out = diffusion_generate(m, [11, 12, 13], length=12, steps=4, trace=tr)
    assert len(out) == 12 and mask not in out
    assert tr.passes == 4 and [len(c) for c in tr.committed_per_step] == [3, 3, 3, 3]
    assert sorted(sum(tr.committed_per_step, [])) == list(range(12))
    assert out == diffusion_generate(m, [11, 12, 13], length=12, steps=4)
    # first pass: the three most confident positions of the all-mask canvas
    lg = run_whole(m, [[11, 12, 13] + [mask] * 12], "logits")[0][3:].float()
    lg[:, mask] = -float("inf")
    conf = torch.softmax(lg, -1).max(-1).values
    want = sorted(sorted(range(12), key=lambda i: (-float(conf[i]), i))[:3])
    assert tr.committed_per_step[0] == want
    # block-wise: the first block is fully committed before the second one starts
    tr2 = DiffusionTrace()
    out2 = diffusion_generate(m, [11, 12, 13], length=12, steps=6, block=6, trace=tr2)
    assert mask not in out2 and all(max(c) < 6 for c in tr2.committed_per_step[:3])


@pytest.mark.gpu
def test_bidirectional_gpu():
    """Structural properties of the bidirectional path on the GPU; the numbers are compared with the CPU oracle in
    test_bidirectional_gpu_matches_cpu_oracle."""
    m = _load("tiny-embed", "cuda")
    long = [5, 6, 7, 8, 9, 10, 11] * 11
    a = run_whole(m, [long, [3, 4, 5]])
    b = run_whole(m, [long[:-1] + [99]])
    assert (a[0][0].float() - b[0][0].float()).abs().max() > 1e-3          # row 0 sees the last token
    alone = run_whole(m, [[3, 4, 5]])[0]
    assert torch.allclose(a[1].float(), alone.float(), atol=2e-2)          # packed sequences do not mix
    e = embed_texts(m, [long, [3, 4, 5]])
    assert all(abs(float(v.norm()) - 1.0) < 1e-3 for v in e)
    out = diffusion_generate(_load("tiny-diffusion", "cuda"), [11, 12, 13], length=8, steps=4)
    assert len(out) == 8 and 2046 not in out
    from flyingfish_b200 import ops
    ops.check_status()


@pytest.mark.gpu
def test_bidirectional_gpu_matches_cpu_oracle():
    from _oracle import assert_hidden_close
    long = [5, 6, 7, 8, 9, 10, 11] * 11
    assert_hidden_close(_load("tiny-embed", "cpu"), _load("tiny-embed", "cuda"), [long, [3, 4, 5]])
    ec = embed_texts(_load("tiny-embed", "cpu"), [long, [3, 4, 5]])
    eg = embed_texts(_load("tiny-embed", "cuda"), [long, [3, 4, 5]])
    for a, b in zip(ec, eg):
        assert torch.nn.functional.cosine_similarity(a.float().cpu(), b.float().cpu(), dim=0).item() > 0.995
    assert_hidden_close(_load("tiny-diffusion", "cpu"), _load("tiny-diffusion", "cuda"), [[11, 12, 13, 2046, 2046, 2046]])
