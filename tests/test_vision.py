"""Vision tower and 3-D compute operators: CPU oracles against plain PyTorch restatements, CUDA kernels against the
oracles (reference: kernels/vision_ops.cu, src/sparse.rs, src/convrot.rs)."""
import pytest
import torch

from flyingfish_b200.models.vision import VisionSpec, VisionTower
from flyingfish_b200.ops import vision_ops as vo

BF16 = torch.bfloat16
cuda = pytest.mark.gpu


def _rand(shape, seed, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).to(BF16)


def _tower_inputs(spec, grids, seed=3):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(gh * gw, spec.patch_dim, generator=g) * 0.5).to(BF16) for (_, gh, gw) in grids]


SMALL = VisionSpec(hidden=128, heads=2, depth=2, intermediate=256, out_hidden=64, pos_side=8)
NARROW = VisionSpec(hidden=96, heads=2, depth=1, intermediate=128, out_hidden=64, pos_side=6)     # head_dim 48 -> widened


@pytest.mark.parametrize("spec", [SMALL, NARROW])
def test_tower_cpu_matches_plain_pytorch(spec):
    state = VisionTower.random_state(spec, seed=1, std=0.05)
    tower = VisionTower(spec, state)
    grids = [(1, 8, 12), (1, 4, 4)]
    patches = _tower_inputs(spec, grids)
    got = tower.forward(patches, grids)
    state16 = {k: v.to(BF16).float() for k, v in state.items()}
    state16["pos_embed.weight"] = state["pos_embed.weight"]
    want = tower.reference_forward(patches, grids, state16)
    for a, b, (_, gh, gw) in zip(got, want, grids):
        assert a.shape == (gh * gw // 4, spec.out_hidden)
        err = (a.float() - b).abs().max().item()
        assert err < 0.05 * max(1.0, b.abs().max().item()), err


def test_images_do_not_see_each_other():
    tower = VisionTower.random(SMALL, seed=2)
    grids = [(1, 4, 8), (1, 8, 4)]
    patches = _tower_inputs(SMALL, grids)
    both = tower.forward(patches, grids)
    alone = tower.forward(patches[1:], grids[1:])
    assert torch.equal(both[1], alone[0])


def test_voxel_hash_and_sparse_conv_match_dense_conv():
    g = torch.Generator().manual_seed(5)
    dims, cin, cout = (6, 5, 7), 16, 24
    occ = torch.rand(2, *dims, generator=g) < 0.3
    coords = torch.nonzero(occ).to(torch.int32)                                  # (b, x, y, z)
    feat = _rand((coords.shape[0], cin), 6)
    w = _rand((cout, 27 * cin), 7, 0.1)
    got = vo.sparse_conv3d(feat, coords, w)
    dense = torch.zeros(2, cin, *dims)
    dense[coords[:, 0].long(), :, coords[:, 1].long(), coords[:, 2].long(), coords[:, 3].long()] = feat.float()
    # weight [cout, offsets (x, y, z major to minor), cin] -> conv3d kernel [cout, cin, kx, ky, kz]
    k5 = w.float().reshape(cout, 3, 3, 3, cin).permute(0, 4, 1, 2, 3)
    full = torch.nn.functional.conv3d(dense, k5, padding=1)
    want = full[coords[:, 0].long(), :, coords[:, 1].long(), coords[:, 2].long(), coords[:, 3].long()]
    assert torch.allclose(got.float(), want, rtol=2e-2, atol=2e-2)


def test_voxelize_and_first_mask():
    pts = torch.tensor([[0.1, 0.1, 0.1], [0.4, 0.2, 0.3], [1.6, 0.2, 0.1], [-0.2, 0.0, 0.0], [0.45, 0.3, 0.2]])
    c = vo.voxelize(pts, None, (0.0, 0.0, 0.0), 0.5, (4, 4, 4))
    assert c.tolist() == [[0, 0, 0, 0], [0, 0, 0, 0], [0, 3, 0, 0], [-1, -1, -1, -1], [0, 0, 0, 0]]
    assert vo.VoxelHash(c).first_mask().tolist() == [True, False, True, False, False]


def test_rotated_int8_linear_close_to_bf16_linear():
    x, w = _rand((9, 256), 8), _rand((40, 256), 9, 0.1)
    qw, sw = vo.quantize_weight_rotated(w, 64)
    y = vo.int8_linear(x, qw, sw, 64)
    want = x.float() @ w.float().t()
    assert (y.float() - want).abs().max() < 0.04 * want.abs().max()
    h = vo.hadamard(16)
    assert torch.allclose(h @ h.t(), torch.eye(16), atol=1e-6)


# ---------------------------------------------------------------------------------------------------------------
@cuda
def test_layernorm_bias_act_gpu():
    x, w, b = _rand((77, 1152), 1), _rand((1152,), 2), _rand((1152,), 3)
    got = vo.layernorm(x.cuda(), w.cuda(), b.cuda(), 1e-6).cpu()
    assert torch.allclose(got.float(), vo.layernorm(x, w, b, 1e-6).float(), rtol=2e-2, atol=2e-2)
    for act in vo.ACTS:
        y = _rand((50, 512), 4, 2.0)
        bias = _rand((512,), 5)
        want = vo.bias_act_(y.clone(), bias, act)
        got = vo.bias_act_(y.cuda(), bias.cuda(), act).cpu()
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2), act


@cuda
@pytest.mark.parametrize("spec", [SMALL, NARROW, VisionSpec(hidden=512, heads=4, depth=2, intermediate=1024, out_hidden=256)])
def test_tower_gpu_matches_cpu(spec):
    state = VisionTower.random_state(spec, seed=1, std=0.05)
    grids = [(1, 8, 12), (1, 16, 20), (1, 4, 4)]
    patches = _tower_inputs(spec, grids)
    want = VisionTower(spec, state).forward(patches, grids)
    got = VisionTower(spec, state, "cuda").forward(patches, grids)
    from flyingfish_b200 import ops
    ops.check_status()
    for a, b in zip(got, want):
        err = (a.float().cpu() - b.float()).abs().max().item()
        assert err < 0.06 * max(1.0, b.float().abs().max().item()), err


@cuda
def test_sparse_ops_gpu_match_cpu():
    g = torch.Generator().manual_seed(5)
    occ = torch.rand(2, 20, 17, 23, generator=g) < 0.2
    coords = torch.nonzero(occ).to(torch.int32)
    feat, w = _rand((coords.shape[0], 32), 6), _rand((48, 27 * 32), 7, 0.1)
    off = vo.cube_offsets(3)
    assert torch.equal(vo.VoxelHash(coords.cuda()).neighbor_map(off.cuda()).cpu(), vo.VoxelHash(coords).neighbor_map(off))
    got = vo.sparse_conv3d(feat.cuda(), coords.cuda(), w.cuda()).cpu()
    want = vo.sparse_conv3d(feat, coords, w)
    assert torch.allclose(got.float(), want.float(), rtol=3e-2, atol=3e-2)
    pts = torch.rand(5000, 3, generator=g) * 4 - 0.5
    c_cpu = vo.voxelize(pts, None, (0.0, 0.0, 0.0), 0.25, (12, 12, 12))
    c_gpu = vo.voxelize(pts.cuda(), None, (0.0, 0.0, 0.0), 0.25, (12, 12, 12))
    assert torch.equal(c_gpu.cpu(), c_cpu)
    assert torch.equal(vo.VoxelHash(c_gpu).first_mask().cpu(), vo.VoxelHash(c_cpu).first_mask())


@cuda
def test_rotate_quant_int8_linear_gpu():
    x, w = _rand((33, 1024), 8), _rand((100, 1024), 9, 0.1)
    qw, sw = vo.quantize_weight_rotated(w, 256)
    q_cpu, s_cpu = vo.rotate_quant(x, 256)
    q_gpu, s_gpu = vo.rotate_quant(x.cuda(), 256)
    assert torch.allclose(s_gpu.cpu(), s_cpu, rtol=1e-2)
    assert ((q_gpu.cpu().int() - q_cpu.int()).abs() <= 1).all()
    y = vo.int8_linear(x.cuda(), qw.cuda(), sw.cuda(), 256).cpu()
    want = x.float() @ w.float().t()
    assert (y.float() - want).abs().max() < 0.04 * want.abs().max()


# ---------------------------------------------------------------------------------------------------------------
# multimodal path: image -> processor -> tower -> embedding rows injected into the decoder's prefill
# ---------------------------------------------------------------------------------------------------------------
def _png(h, w, seed):
    import struct
    import zlib
    import numpy as np
    px = np.random.default_rng(seed).integers(0, 256, (h, w, 3), dtype=np.uint8)
    raw = b"".join(b"\x00" + px[r].tobytes() for r in range(h))
    chunk = lambda t, d: struct.pack(">I", len(d)) + t + d + struct.pack(">I", zlib.crc32(t + d))
    return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0))
            + chunk(b"IDAT", zlib.compress(raw)) + chunk(b"IEND", b""))


def _vl_model(device="cpu"):
    from flyingfish_b200.api import Model
    from flyingfish_b200.config import Settings
    return Model.load("tiny-vl", Settings(capacity=512, max_batch=4, graph=False), device=device, seed=0)


def test_multimodal_prefill_uses_tower_rows():
    from flyingfish_b200.serve.image import decode_png
    m = _vl_model()
    tok = m.spec.extra["image_token_id"]
    img_a, img_b = decode_png(_png(64, 96, 1)), decode_png(_png(64, 96, 2))
    ids = [5, 6, tok, 7, 8]
    exp, pos, emb = m.encode_images(ids, [img_a])
    assert len(exp) == 4 + len(pos) and emb.shape == (len(pos), m.spec.hidden) and exp[2] == tok and exp[-1] == 8
    first_a = m.prefill_multimodal(ids, [img_a])
    again = m.prefill_multimodal(ids, [img_a])
    assert first_a == again
    # the image content reaches the logits: a chunked prefill gives the same token, another image may not
    m.engine.settings.chunk = 16
    assert m.prefill_multimodal(ids, [img_a]) == first_a
    m.engine.settings.chunk = 0
    la = _last_logits(m, ids, img_a)
    lb = _last_logits(m, ids, img_b)
    assert (la - lb).abs().max() > 1e-3
    with pytest.raises(ValueError):
        m.encode_images([5, tok, tok], [img_a])


def _last_logits(m, ids, img):
    exp, pos, emb = m.encode_images(ids, [img])
    m.reset()
    seq = m.engine.add_sequence(exp, pos, emb)
    fb = m.engine.prefill_batch
    kvs = m.engine.kv.seqs[seq.seq_id]
    sl = m.engine.kv.reserve(seq.seq_id, len(exp))
    fb.fill(ids=exp, positions=list(range(len(exp))), slots=sl, q_lens=[len(exp)], ctx_lens=[len(exp)],
            block_rows=[list(kvs.blocks)], logit_rows=[len(exp) - 1], is_decode=False)
    fb.upload()
    lg = m.engine.model.forward(fb, m.engine.kv, return_logits=True,
                                inputs_embeds=m.engine._mm_embeds([(seq, len(exp))], fb, len(exp)))
    m.reset()
    return lg.float().cpu()


def test_http_chat_with_image():
    import asyncio
    import base64
    from aiohttp.test_utils import TestClient, TestServer
    from flyingfish_b200.loaders.tokenizer import ByteTokenizer
    from flyingfish_b200.serve.backend import Backend
    from flyingfish_b200.serve.http import Server
    m = _vl_model()
    tok = m.spec.extra["image_token_id"]

    class Tk(ByteTokenizer):
        def encode(self, text):
            out = []
            for i, piece in enumerate(text.split("<|image|>")):
                if i:
                    out.append(tok)
                out += super().encode(piece)
            return out
    template = "{% for m in messages %}{{ m.content }}{% endfor %}"
    url = "data:image/png;base64," + base64.b64encode(_png(64, 64, 3)).decode()

    async def main():
        backend = Backend(m.engine, eos_ids=())
        backend.start()
        srv = Server(backend, Tk(m.spec.vocab), "tiny-vl", template, capacity=512, image_placeholder="<|image|>")
        client = TestClient(TestServer(srv.app()))
        await client.start_server()
        try:
            body = {"messages": [{"role": "user", "content": [{"type": "text", "text": "look "},
                                                               {"type": "image_url", "image_url": {"url": url}}]}],
                    "max_tokens": 4}
            r = await client.post("/v1/chat/completions", json=body)
            js = await r.json()
            assert r.status == 200, js
            assert js["usage"]["completion_tokens"] == 4
            body["messages"][0]["content"][1]["image_url"]["url"] = "data:image/png;base64,AAAA"
            r = await client.post("/v1/chat/completions", json=body)
            assert r.status == 400
        finally:
            await client.close()
            backend.shutdown()
    asyncio.run(main())


@cuda
def test_multimodal_gpu():
    """The decoder's random weights are drawn on the device they live on, so CPU and GPU models differ; what must
    agree is the tower (same host-drawn weights) and the GPU path with itself."""
    from flyingfish_b200.serve.image import decode_png
    img, other = decode_png(_png(96, 64, 4)), decode_png(_png(96, 64, 5))
    tok = 2047
    ids = [5, 6, tok, 7, 8]
    cpu, gpu = _vl_model(), _vl_model("cuda")
    ec, pc, mc = cpu.encode_images(ids, [img])
    eg, pg, mg = gpu.encode_images(ids, [img])
    assert ec == eg and pc == pg
    cos = torch.nn.functional.cosine_similarity(mc.float().flatten(), mg.float().cpu().flatten(), dim=0).item()
    assert cos > 0.999, cos
    first = gpu.prefill_multimodal(ids, [img])
    rest = [gpu.decode() for _ in range(3)]
    gpu.engine.settings.chunk = 16
    assert gpu.prefill_multimodal(ids, [img]) == first and [gpu.decode() for _ in range(3)] == rest
    gpu.engine.settings.chunk = 0
    la, lb = _last_logits(gpu, ids, img), _last_logits(gpu, ids, other)
    assert (la - lb).abs().max() > 1e-3
    from flyingfish_b200 import ops
    ops.check_status()


def test_group_norm_and_conv3d_oracles():
    from flyingfish_b200.ops import vision_ops
    g = torch.Generator().manual_seed(41)
    x = torch.randn(2, 50, 32, generator=g).to(torch.bfloat16)
    w, b = 1 + 0.1 * torch.randn(32, generator=g), 0.1 * torch.randn(32, generator=g)
    got = vision_ops.group_norm(x, w, b, groups=4, act="silu").float()
    ref = torch.nn.functional.silu(torch.nn.functional.group_norm(x.float().transpose(1, 2), 4, w, b, 1e-5).transpose(1, 2))
    assert (got - ref).abs().max() < 3e-2
    v = torch.randn(1, 5, 6, 7, 16, generator=g).to(torch.bfloat16)
    wt = 0.1 * torch.randn(24, 16, 3, 3, 3, generator=g)
    bias = 0.1 * torch.randn(24, generator=g)
    got = vision_ops.conv3d(v, wt, bias, act="relu").float()
    ref = torch.relu(torch.nn.functional.conv3d(v.float().permute(0, 4, 1, 2, 3), wt, bias, padding=1).permute(0, 2, 3, 4, 1))
    assert got.shape == (1, 5, 6, 7, 24) and (got - ref).abs().max() < 5e-2


@pytest.mark.gpu
def test_group_norm_and_conv3d_kernels(cuda):
    from flyingfish_b200.ops import vision_ops
    g = torch.Generator().manual_seed(42)
    for n, positions, c, groups in ((2, 777, 64, 8), (1, 4096, 128, 32), (3, 10, 16, 2)):
        x = torch.randn(n, positions, c, generator=g).to(torch.bfloat16)
        w, b = 1 + 0.1 * torch.randn(c, generator=g), 0.1 * torch.randn(c, generator=g)
        for act in ("none", "silu"):
            want = vision_ops.group_norm(x, w, b, groups, act=act).float()
            got = vision_ops.group_norm(x.to(cuda), w.to(cuda), b.to(cuda), groups, act=act).float().cpu()
            assert (got - want).abs().max() < 4e-2, (n, positions, c, groups, act)
    v = torch.randn(2, 6, 7, 9, 32, generator=g).to(torch.bfloat16)
    wt = 0.05 * torch.randn(40, 32, 3, 3, 3, generator=g)
    bias = 0.1 * torch.randn(40, generator=g)
    want = vision_ops.conv3d(v, wt, bias, act="silu").float()
    got = vision_ops.conv3d(v.to(cuda), wt.to(cuda), bias.to(cuda), act="silu").float().cpu()
    assert got.shape == want.shape and (got - want).abs().max() < 6e-2


def test_neighborhood_attention_window_rule():
    from flyingfish_b200.ops import vision_ops
    g = torch.Generator().manual_seed(43)
    q, k, v = (torch.randn(1, 5, 6, 2, 32, generator=g).to(torch.bfloat16) for _ in range(3))
    out = vision_ops.neighborhood_attention(q, k, v, 3).float()
    # corner query: the window is shifted inwards and still holds 9 keys
    kk, vv = k.float()[0, :3, :3].reshape(9, 2, 32), v.float()[0, :3, :3].reshape(9, 2, 32)
    sc = torch.einsum("hd,khd->hk", q.float()[0, 0, 0], kk) / 32 ** 0.5
    assert (out[0, 0, 0] - torch.einsum("hk,khd->hd", torch.softmax(sc, -1), vv)).abs().max() < 2e-2
    # a full-size window is plain attention over the grid
    full = vision_ops.neighborhood_attention(q[:, :5, :5].contiguous(), k[:, :5, :5].contiguous(), v[:, :5, :5].contiguous(), 5).float()
    kk, vv = k.float()[0, :5, :5].reshape(25, 2, 32), v.float()[0, :5, :5].reshape(25, 2, 32)
    sc = torch.einsum("ijhd,khd->ijhk", q.float()[0, :5, :5], kk) / 32 ** 0.5
    assert (full[0] - torch.einsum("ijhk,khd->ijhd", torch.softmax(sc, -1), vv)).abs().max() < 2e-2


@pytest.mark.gpu
def test_neighborhood_attention_kernel(cuda):
    from flyingfish_b200.ops import vision_ops
    g = torch.Generator().manual_seed(44)
    for shape, ks in (((2, 9, 11, 3, 64), 7), ((1, 8, 8, 2, 128), 3), ((1, 5, 5, 1, 32), 5)):
        q, k, v = (torch.randn(*shape, generator=g).to(torch.bfloat16) for _ in range(3))
        want = vision_ops.neighborhood_attention(q, k, v, ks).float()
        got = vision_ops.neighborhood_attention(q.to(cuda), k.to(cuda), v.to(cuda), ks).float().cpu()
        assert (got - want).abs().max() < 3e-2, (shape, ks)
