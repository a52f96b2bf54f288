"""Layout, blending and sampling operators of the media / 3-D decoders against index-by-index restatements."""
import math

import pytest
import torch

from flyingfish_b200.ops import media_ops as mo


def test_embeddings():
    t, fr = torch.tensor([0.0, 0.5, 2.0]), torch.tensor([1.0, 0.1])
    e = mo.sinusoidal_embed(t, fr)
    assert e.shape == (3, 4) and torch.allclose(e[1], torch.tensor([math.cos(0.5), math.cos(0.05), math.sin(0.5), math.sin(0.05)]))
    assert torch.allclose(mo.sinusoidal_embed(t, fr, two_pi=True)[1, 2], torch.tensor(math.sin(math.pi)), atol=1e-6)
    pts = torch.tensor([[0.25, -0.5, 1.0]])
    p = mo.point_position_embed(pts, torch.tensor([1.0, 2.0]), 16, version=2)
    assert p.shape == (1, 16) and (p[0, 12:] == 0).all()
    want_x = [math.sin(0.25 * math.pi), math.sin(0.5 * math.pi), math.cos(0.25 * math.pi), math.cos(0.5 * math.pi)]
    assert torch.allclose(p[0, :4], torch.tensor(want_x), atol=1e-6)
    assert torch.allclose(mo.point_position_embed(pts, torch.tensor([1.0, 2.0]), 12, version=1)[0, 0], torch.tensor(math.sin(0.5 * math.pi)))
    with pytest.raises(ValueError):
        mo.point_position_embed(pts, torch.tensor([1.0, 2.0]), 8)


def test_pixel_shuffle_3d_and_unpatchify():
    side, c = 2, 3
    x = torch.arange(side ** 3 * c * 8, dtype=torch.float32).reshape(side ** 3, c * 8)
    y = mo.pixel_shuffle_3d(x, side)
    out = 2 * side
    for i in range(out ** 3 * c):
        ch, p = i % c, i // c
        ix, iy, iz = p % out, (p // out) % out, p // (out * out)
        parent = (iz // 2 * side + iy // 2) * side + ix // 2
        child = (iz % 2) * 4 + (iy % 2) * 2 + ix % 2
        assert y.reshape(-1)[i] == x.reshape(-1)[(parent * c + ch) * 8 + child]
    frames, h, w, ch, pt, p = 2, 2, 3, 2, 2, 2
    rows = torch.arange(frames * h * w * ch * pt * p * p, dtype=torch.float32).reshape(frames * h * w, ch * pt * p * p)
    px = mo.unpatchify(rows, frames, h, w, ch, pt, p)
    assert px.shape == (ch, frames * pt, h * p, w * p)
    flat = px.reshape(-1)
    ot, oh, ow = frames * pt, h * p, w * p
    for i in range(0, flat.numel(), 7):
        x_, y_, t_, c_ = i % ow, (i // ow) % oh, (i // (ow * oh)) % ot, i // (ow * oh * ot)
        token = ((t_ // pt) * h + y_ // p) * w + x_ // p
        col = ((c_ * pt + t_ % pt) * p + y_ % p) * p + x_ % p
        assert flat[i] == rows[token, col]
    with pytest.raises(ValueError):
        mo.unpatchify(rows, frames, h, w, ch, pt, 3)


def test_frame_blend_and_tile_stitch():
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(2, 5, 3, generator=g), torch.randn(2, 6, 3, generator=g)
    out = mo.frame_blend(a, b, 3, 2, 1)
    for k in range(3):
        w = torch.tensor(float(k)) * (1.0 / torch.tensor(3.0))
        assert torch.allclose(out[:, k], a[:, 2 + k] * (1.0 - w) + b[:, 1 + k] * w)
    assert torch.equal(out[:, 0], a[:, 2])
    with pytest.raises(ValueError):
        mo.frame_blend(a, b, 4, 2, 1)
    # a 2 x 2 grid of 4 x 5 tiles with one overlapping row and two overlapping columns -> a 7 x 8 canvas
    tiles = torch.randn(4, 2, 4, 5, generator=g)
    rs, ro, cs, co = [0, 3], [1], [0, 3], [2]
    canvas = mo.tile_stitch(tiles, rs, ro, cs, co, 7, 8)
    assert canvas.shape == (2, 7, 8)
    blend = lambda p, q, k, n: p * (1.0 - torch.tensor(float(k)) * (1.0 / torch.tensor(float(n)))) + q * (torch.tensor(float(k)) * (1.0 / torch.tensor(float(n))))
    for Y in range(7):
        for X in range(8):
            r, c = (1 if Y >= 3 else 0), (1 if X >= 3 else 0)
            y, x = Y - rs[r], X - cs[c]
            v = tiles[r * 2 + c, :, y, x]
            if r > 0 and y < 1:
                v = blend(tiles[c, :, y + 4 - 1, x], v, y, 1)
            if c > 0 and x < 2:
                v = blend(tiles[r * 2, :, y, x + 5 - 2], v, x, 2)
            assert torch.allclose(canvas[:, Y, X], v, atol=1e-6), (Y, X)
    with pytest.raises(ValueError):
        mo.tile_stitch(tiles, rs, ro, cs, co, 9, 8)                          # rows 7, 8 lie below the last tile


def test_gaussian_posterior():
    g = torch.Generator().manual_seed(1)
    moments, eps = torch.randn(6, 4, 5, generator=g), torch.randn(3, 4, 5, generator=g)
    moments[3, 0, 0], moments[4, 0, 0] = 50.0, -50.0                       # clamped log-variances
    lm, ls = torch.tensor([0.1, -0.2, 0.3]), torch.tensor([1.5, 0.5, 2.0])
    mean, std, lat = mo.gaussian_posterior(moments, eps, lm, ls)
    assert torch.equal(mean, moments[:3]) and std[0, 0, 0] == pytest.approx(math.exp(10.0), rel=1e-6) and std[1, 0, 0] == pytest.approx(math.exp(-15.0), rel=1e-6)
    want = ((moments[1, 2, 3] + std[1, 2, 3] * eps[1, 2, 3]).half().float() - lm[1]) / ls[1]
    assert lat[1, 2, 3] == want
    assert mo.gaussian_posterior(moments, eps, lm, ls, crop=(2, 3))[2].shape == (3, 2, 3)
    with pytest.raises(ValueError):
        mo.gaussian_posterior(moments[:5], eps, lm, ls)


def test_projection_samples_the_feature_map():
    assert mo.perspective_focal(math.pi / 2, 64.0) == pytest.approx(32.0)
    with pytest.raises(ValueError):
        mo.perspective_focal(math.pi, 64.0)
    h = w = 8
    g = torch.Generator().manual_seed(2)
    feats = torch.randn(h, w, 3, generator=g)
    # camera two units in front of the origin looking down -z: world-to-camera = translation by (0, 0, -2)
    cam = torch.tensor([1.0, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, -2.0, mo.perspective_focal(0.8, 8.0), 1.0, 8.0])
    side = 3
    out = mo.project_bilinear(feats, cam, side)
    assert out.shape == (27, 3)
    # the centre of the lattice projects to image coordinate resolution / 2, which is the centre of pixel (4, 4)
    centre = (1 * side + 1) * side + 1
    assert torch.allclose(out[centre], feats[4, 4], atol=1e-5)
    # index-by-index restatement for every lattice point
    for row in range(27):
        ix, iy, iz = row // 9, (row // 3) % 3, row % 3
        u = lambda j: ((j * 1.0 - 1.0) if j < side // 2 else (-(side - 1 - j) * 1.0 + 1.0)) / 1.0 / 2.0
        a, b, d = u(ix), -u(iz), u(iy)
        x, y, z = a, b, d - 2.0
        denom = -z + 1e-8
        def pix(cc, size):
            pr = float(cam[12]) * cc / denom + 4.0
            nm = (pr + 0.5) / 8.0 * 2.0 - 1.0
            return min(max(((nm + 1.0) * size - 1.0) / 2.0, 0.0), size - 1.0)
        px, py = pix(x, w), pix(-y, h)
        x0, y0 = int(px), int(py)
        x1, y1 = min(x0 + 1, w - 1), min(y0 + 1, h - 1)
        dx, dy = px - x0, py - y0
        want = feats[y0, x0] * (1 - dx) * (1 - dy) + feats[y0, x1] * dx * (1 - dy) + feats[y1, x0] * (1 - dx) * dy + feats[y1, x1] * dx * dy
        assert torch.allclose(out[row], want, atol=1e-4), row
    sub = mo.project_bilinear(feats, cam, side, torch.tensor([[1, 1, 1], [0, 2, 1]]))
    assert torch.allclose(sub[0], out[centre]) and torch.allclose(sub[1], out[(0 * 3 + 2) * 3 + 1])
    with pytest.raises(ValueError):
        mo.project_bilinear(feats, cam, side, torch.tensor([[3, 0, 0]]))


def test_spatial_rotary():
    h, w, heads, dim = 3, 4, 2, 8
    table = mo.axial_rotary_table(h, w, dim)
    assert table.shape == (12, 8)
    # pixel (0, 0) is the identity; a pixel in row 0 only turns the column frequencies
    assert torch.allclose(table[0], torch.tensor([1.0, 1, 1, 1, 0, 0, 0, 0]))
    assert torch.allclose(table[2, :2], torch.ones(2)) and not torch.allclose(table[2, 2:4], torch.ones(2))
    g = torch.Generator().manual_seed(3)
    x = torch.randn(12, heads, dim, generator=g)
    y = mo.rotary_spatial(x, table)
    for p in (0, 5, 11):
        for hd in range(heads):
            for d in range(4):
                c, s = table[p, d], table[p, 4 + d]
                assert y[p, hd, d] == pytest.approx(float(x[p, hd, d] * c - x[p, hd, 4 + d] * s), abs=1e-6)
                assert y[p, hd, 4 + d] == pytest.approx(float(x[p, hd, 4 + d] * c + x[p, hd, d] * s), abs=1e-6)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)           # a rotation
    with pytest.raises(ValueError):
        mo.rotary_spatial(x[..., :6], table[:, :6])
