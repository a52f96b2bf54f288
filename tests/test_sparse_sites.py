"""Sparse site bookkeeping: unique sites, shared corners, parent / child grids, re-quantisation."""
import pytest
import torch

from flyingfish_b200.ops import mesh_ops, sparse_sites as ss


def _sites(rows):
    return torch.tensor(rows, dtype=torch.int32)


def test_deduplicate_and_checks():
    c = _sites([[0, 2, 1, 1], [0, 1, 5, 0], [0, 2, 1, 1], [1, 0, 0, 0], [0, 1, 5, 0]])
    uniq, inv = ss.deduplicate(c)
    assert uniq.tolist() == [[0, 1, 5, 0], [0, 2, 1, 1], [1, 0, 0, 0]] and inv.tolist() == [1, 0, 1, 2, 0]
    with pytest.raises(ValueError, match="duplicate"):
        ss.check_sites(_sites([[0, 2, 1, 1], [0, 1, 5, 0], [0, 2, 1, 1]]))
    with pytest.raises(ValueError, match="batch"):
        ss.check_sites(_sites([[1, 0, 0, 0], [0, 0, 0, 0]]))
    with pytest.raises(ValueError):
        ss.check_sites(_sites([[0, -1, 0, 0]]))


def test_cube_corners_feed_the_surface_extraction():
    c = _sites([[0, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0]])
    corners, cubes, offsets, contributors = ss.cube_corners(c)
    assert corners.shape[0] == 16 and cubes.shape == (3, 8)                  # 3 cubes x 8 corners, 8 of them shared
    for cube in range(3):
        for k in range(8):
            want = [0, c[cube, 1] + (k & 1), c[cube, 2] + ((k >> 1) & 1), c[cube, 3] + ((k >> 2) & 1)]
            assert corners[cubes[cube, k]].tolist() == [int(v) for v in want]
    assert offsets[-1] == 24 and offsets.shape[0] == 17
    for k in range(16):
        slots = contributors[offsets[k]:offsets[k + 1]].tolist()
        assert slots == sorted(slots) and all(cubes.reshape(-1)[s] == k for s in slots) and len(slots) >= 1
    shared = corners.tolist().index([0, 1, 1, 0])                             # the edge all three cubes meet at
    assert offsets[shared + 1] - offsets[shared] == 3
    # a sphere over sparse sites, extracted through the shared corners
    g = 8
    idx = torch.stack(torch.meshgrid(torch.arange(g), torch.arange(g), torch.arange(g), indexing="ij"), -1).reshape(-1, 3)
    sites = torch.cat([torch.zeros(idx.shape[0], 1, dtype=torch.long), idx], 1).to(torch.int32)
    corners, cubes, _, _ = ss.cube_corners(sites)
    positions = corners[:, 1:].float()
    scalar = (positions - torch.tensor([3.9, 4.1, 4.05])).norm(dim=1) - 2.7
    v, f = mesh_ops.dual_contour_mesh(sites, cubes, positions, scalar)
    e = torch.cat([f[:, [0, 1]], f[:, [1, 2]], f[:, [2, 0]]]).long()
    und = torch.minimum(e[:, 0], e[:, 1]) * v.shape[0] + torch.maximum(e[:, 0], e[:, 1])
    assert f.shape[0] > 100 and (und.unique(return_counts=True)[1] == 2).all()


def test_parents_children_and_rescaling():
    c = _sites([[0, 5, 2, 7], [0, 4, 3, 6], [0, 1, 1, 1], [1, 5, 2, 7]])
    parents, inv = ss.downsample(c, 2)
    assert parents.tolist() == [[0, 0, 0, 0], [0, 2, 1, 3], [1, 2, 1, 3]] and inv.tolist() == [1, 1, 0, 2]
    active = torch.zeros(3, 8, dtype=torch.bool)
    active[0, [0, 7]] = True
    active[2, 3] = True
    kids, src = ss.subdivide(parents, active, capacity=8)
    assert kids.tolist() == [[0, 0, 0, 0], [0, 1, 1, 1], [1, 5, 3, 6]] and src.tolist() == [[0, 0], [0, 7], [2, 3]]
    assert ss.downsample(kids, 2)[0].tolist() == [[0, 0, 0, 0], [1, 2, 1, 3]]
    with pytest.raises(ValueError):
        ss.subdivide(parents, active, capacity=2)
    with pytest.raises(ValueError):
        ss.subdivide(parents, torch.zeros(3, 8, dtype=torch.bool), capacity=8)
    sc = ss.scaled_coordinates(_sites([[0, 0, 1, 3]]), 4, 9)
    assert torch.allclose(sc, torch.tensor([[1.0, 3.0, 7.0]]))
    # ties round to even: (1 + 0.5) / 4 * 4 = 1.5 -> 2, (0 + 0.5) / 4 * 4 = 0.5 -> 0
    assert ss.round_unique(_sites([[0, 0, 1, 3], [0, 0, 1, 2]]), 4, 5).tolist() == [[0, 0, 2, 2], [0, 0, 2, 4]]
    assert ss.round_unique(_sites([[0, 0, 0, 0], [0, 1, 0, 0]]), 8, 3).tolist() == [[0, 0, 0, 0]]      # two cells merge
    with pytest.raises(ValueError):
        ss.scaled_coordinates(_sites([[0, 4, 0, 0]]), 4, 9)
    with pytest.raises(ValueError):
        ss.downsample(c, 0)


def test_serialized_windows():
    c = _sites([[0, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1], [0, 3, 2, 1], [1, 1, 1, 1], [1, 0, 0, 0]])
    k = ss.morton_keys(c)
    # depth 2 (largest coordinate 3): x y z bits interleaved, x most significant inside a triple
    assert k[:4].tolist() == [0, 4, 2, 1]
    assert k[4].item() == ((1 << 5) | (1 << 4)) | ((1 << 2) | (1 << 0))        # x = 0b11, y = 0b10, z = 0b01
    assert k[5].item() == (1 << 6) | 7 and k[6].item() == (1 << 6)
    assert ss.morton_keys(c, swap_xy=True)[:3].tolist() == [0, 2, 4]
    w = ss.serialized_windows(c, window=2)
    assert w["order"][0].tolist() == [0, 3, 2, 1, 4, 6, 5] and w["order"][1].tolist() == [0, 3, 1, 2, 4, 6, 5]
    for o, inv in zip(w["order"], w["inverse"]):
        assert inv[o.long()].tolist() == list(range(7))
    # sample 0 has 5 rows -> 6 slots (the odd row's window is filled from the last full window), sample 1 has 2
    assert w["pad"].tolist() == [0, 1, 2, 3, 4, 3, 5, 6] and w["unpad"].tolist() == [0, 1, 2, 3, 4, 6, 7]
    assert w["offsets"].tolist() == [0, 2, 4, 6, 8]
    small = ss.serialized_windows(c, window=8)                                  # samples shorter than a window are not padded
    assert small["pad"].tolist() == list(range(7)) and small["offsets"].tolist() == [0, 5, 7]
    with pytest.raises(ValueError):
        ss.serialized_windows(c, 0)
    with pytest.raises(ValueError):
        ss.morton_keys(_sites([[0, 1 << 17, 0, 0]]))


def test_unit_ball_frame_and_adaptive_pool():
    c = _sites([[2, 0, 0, 0], [2, 4, 0, 0], [2, 2, 6, 2]])
    f = ss.unit_ball_frame(c)
    centre = torch.tensor([2.0, 2.0, 2.0 / 3.0])
    pts = torch.cat([c[:, 1:].float(), torch.ones(3, 1)], 1) @ f.t()
    assert torch.allclose(pts[:, :3].mean(0), torch.zeros(3), atol=1e-6) and pts[:, 3].tolist() == [1.0, 1.0, 1.0]
    assert pts[:, :3].norm(dim=1).max().item() == pytest.approx(1.0, abs=1e-6)
    assert torch.allclose(f[:3, 3] / f[0, 0], -centre, atol=1e-6)
    with pytest.raises(ValueError):
        ss.unit_ball_frame(_sites([[0, 0, 0, 0], [1, 1, 1, 1]]))
    from flyingfish_b200.ops import media_ops
    x = torch.arange(5 * 7 * 2, dtype=torch.float32).reshape(5, 7, 2)
    y = media_ops.adaptive_avg_pool2d(x, 2, 3)
    for oy in range(2):
        for ox in range(3):
            y0, y1 = oy * 5 // 2, ((oy + 1) * 5 + 1) // 2
            x0, x1 = ox * 7 // 3, ((ox + 1) * 7 + 2) // 3
            assert torch.allclose(y[oy, ox], x[y0:y1, x0:x1].reshape(-1, 2).mean(0))
