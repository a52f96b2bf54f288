"""MiniCPM-V vision side: position buckets, gather orders, the tower against a plain FP32 PyTorch model, token spans."""
import pytest
import torch

from flyingfish_b200.models import minicpm_vision as mv


def test_position_buckets_and_gather_orders():
    side = 8
    ids = mv.nearest_position_ids([(4, 16), (3, 5)], side)
    want = []
    for h, w in ((4, 16), (3, 5)):
        def bucket(v):
            c = 0
            while c < side and not (torch.tensor((c + 1) / side, dtype=torch.float64).float().item() > v):
                c += 1
            return c
        for r in range(h):
            for c in range(w):
                want.append(bucket(torch.tensor(r / h, dtype=torch.float32).item()) * side + bucket(torch.tensor(c / w, dtype=torch.float32).item()))
    assert ids.tolist() == want
    assert ids[:16].tolist() == [0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5, 6, 6, 7, 7]       # 16 columns over 8 buckets
    assert mv.nearest_position_ids([(8, 8)], side).tolist() == list(range(64))           # the table's own grid: identity
    order = mv.block_order([(2, 4), (2, 2)], 2)
    assert order.tolist() == [0, 1, 4, 5, 2, 3, 6, 7, 8, 9, 10, 11]
    with pytest.raises(ValueError):
        mv.block_order([(3, 4)], 2)


def test_config_and_tensor_list():
    root = {"vision_config": {"hidden_act": "gelu_pytorch_tanh", "hidden_size": 1152, "num_attention_heads": 16, "num_hidden_layers": 27,
                              "intermediate_size": 4304, "patch_size": 14, "image_size": 980, "window_kernel_size": [2, 2]},
            "insert_layer_id": 6, "downsample_mode": "16x", "merge_kernel_size": [2, 2], "text_config": {"hidden_size": 4096}}
    spec = mv.MiniCpmVisionSpec.from_config(root)
    assert (spec.head_dim, spec.position_side, spec.patch_dim, spec.patches_per_token) == (72, 70, 588, 16)
    names = spec.expected_tensors()
    assert names["model.vision_tower.vit_merger.linear_1.weight"] == (4 * 4304, 4 * 1152)
    assert names["model.merger.mlp.0.linear_2.weight"] == (4096, 4 * 1152)
    assert names["model.vision_tower.embeddings.position_embedding.weight"] == (4900, 1152)
    assert len(names) == 5 + 27 * 16 + 8 + 2 + 6 + 6
    bad = dict(root, downsample_mode="4x")
    with pytest.raises(ValueError):
        mv.MiniCpmVisionSpec.from_config(bad)


def test_tower_matches_plain_model():
    spec = mv.minicpm_vision_tiny()
    state = mv.MiniCpmVisionTower.random_state(spec, 3)
    tower = mv.MiniCpmVisionTower(spec, state)
    g = torch.Generator().manual_seed(4)
    grids = [(8, 12), (4, 4)]
    patches = [torch.randn(h * w, spec.patch_dim, generator=g) for h, w in grids]
    got = tower.forward(patches, grids)
    rounded = {k: v.to(torch.bfloat16).float() for k, v in state.items()}
    want = tower.reference_forward([p.to(torch.bfloat16).float() for p in patches], grids, rounded)
    assert [tuple(t.shape) for t in got] == [(6, spec.out_hidden), (1, spec.out_hidden)]
    for a, b in zip(got, want):
        assert (a.float() - b).abs().max() < 0.03 * b.abs().max() + 2e-3
    # views do not see each other: a view alone gives the same rows
    alone = tower.forward(patches[:1], grids[:1])[0]
    assert torch.equal(alone, got[0])
    with pytest.raises(ValueError):
        tower.forward([patches[0][:-1]], grids[:1])
    with pytest.raises(ValueError):
        tower.forward([torch.zeros(6 * 4, spec.patch_dim)], [(6, 4)])
    broken = dict(state)
    broken["model.merger.mlp.0.linear_1.weight"] = broken["model.merger.mlp.0.linear_1.weight"][:, :-1]
    with pytest.raises(ValueError):
        mv.MiniCpmVisionTower(spec, broken)


def test_view_token_spans():
    IMG, S, E, SS, SE, NL = 9, 1, 2, 3, 4, 5
    out = mv.expand_view_tokens([7, IMG, 8], IMG, [(2, 2, 2, 1)], S, E, SS, SE, NL)
    assert out == [7, S, IMG, IMG, E, SS, IMG, SE, SS, IMG, SE, NL, SS, IMG, SE, SS, IMG, SE, 8]
    assert mv.expand_view_tokens([IMG], IMG, [(3, 0, 0, 0)], S, E, SS, SE, NL) == [S, IMG, IMG, IMG, E]
    with pytest.raises(ValueError):
        mv.expand_view_tokens([IMG, IMG], IMG, [(1, 0, 0, 0)], S, E, SS, SE, NL)
    with pytest.raises(ValueError):
        mv.expand_view_tokens([7], IMG, [(1, 0, 0, 0)], S, E, SS, SE, NL)


@pytest.mark.gpu
def test_tower_gpu_matches_cpu():
    spec = mv.minicpm_vision_tiny()
    state = mv.MiniCpmVisionTower.random_state(spec, 5)
    cpu, gpu = mv.MiniCpmVisionTower(spec, state), mv.MiniCpmVisionTower(spec, state, "cuda:0")
    g = torch.Generator().manual_seed(6)
    grids = [(8, 12), (4, 4), (16, 8)]
    patches = [torch.randn(h * w, spec.patch_dim, generator=g) for h, w in grids]
    for a, b in zip(cpu.forward(patches, grids), gpu.forward(patches, grids)):
        assert (a.float() - b.float().cpu()).abs().max() < 0.04 * a.float().abs().max() + 3e-3


def _png(h, w, seed):
    import struct
    import zlib
    import numpy as np
    px = np.random.default_rng(seed).integers(0, 256, (h, w, 3), dtype=np.uint8)
    raw = b"".join(b"\x00" + px[r].tobytes() for r in range(h))
    chunk = lambda t, d: struct.pack(">I", len(d)) + t + d + struct.pack(">I", zlib.crc32(t + d))
    return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0))
            + chunk(b"IDAT", zlib.compress(raw)) + chunk(b"IEND", b""))


def test_sliced_image_prompt_through_the_engine():
    from flyingfish_b200.api import Model
    from flyingfish_b200.config import Settings
    from flyingfish_b200.serve.image import decode_png, slice_plan
    m = Model.load("tiny-minicpm", Settings(capacity=1024, max_batch=2, graph=False), device="cpu", seed=0)
    ex = m.spec.extra
    tok = ex["image_token_id"]
    small, large = decode_png(_png(24, 24, 1)), decode_png(_png(48, 96, 2))
    ids = [5, tok, 6]
    exp, pos, emb = m.encode_images(ids, [small])
    # a small image is shown whole only: start, tokens, end
    assert exp[0] == 5 and exp[1] == ex["image_start_id"] and exp[-2] == ex["image_end_id"] and exp[-1] == 6
    assert len(pos) == emb.shape[0] == len(exp) - 4 and emb.shape[1] == m.spec.hidden
    exp, pos, emb = m.encode_images(ids, [large])
    plan = slice_plan(48, 96, patch=2, max_slices=4, scale=32)
    assert plan.rows * plan.cols >= 2
    per_view = [(g[1] * g[2]) // 16 for g in plan.grids(2)]
    assert emb.shape[0] == sum(per_view) == len(pos)
    assert exp.count(ex["slice_start_id"]) == exp.count(ex["slice_end_id"]) == plan.rows * plan.cols
    assert exp.count(ex["newline_id"]) == plan.rows - 1
    first = m.prefill_multimodal(ids, [large])
    assert first == m.prefill_multimodal(ids, [large])
    assert isinstance(m.decode(), int)
    with pytest.raises(ValueError):
        m.encode_images([5, tok, tok], [large])
