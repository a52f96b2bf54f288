"""Mesh post-processing: components, normalisation, the native quadric-error simplifier, hole filling."""
import pytest
import torch

from flyingfish_b200.ops import mesh_ops as mo
from flyingfish_b200.utils import mesh_post as mp


def _sphere(g=10, r=3.4, centre=(4.9, 5.1, 5.05)):
    idx = torch.stack(torch.meshgrid(torch.arange(g), torch.arange(g), torch.arange(g), indexing="ij"), -1).reshape(-1, 3)
    coords = torch.cat([torch.zeros(idx.shape[0], 1, dtype=torch.long), idx], 1).to(torch.int32)
    s = g + 1
    corner = lambda x, y, z: x + s * (y + s * z)
    cubes = torch.stack([corner(idx[:, 0] + (c & 1), idx[:, 1] + ((c >> 1) & 1), idx[:, 2] + ((c >> 2) & 1)) for c in range(8)], 1)
    lat = torch.stack(torch.meshgrid(torch.arange(s), torch.arange(s), torch.arange(s), indexing="ij"), -1).reshape(-1, 3)
    positions = torch.zeros(s ** 3, 3)
    positions[corner(lat[:, 0], lat[:, 1], lat[:, 2])] = lat.float()
    scalar = (positions - torch.tensor(centre)).norm(dim=1) - r
    return mo.dual_contour_mesh(coords, cubes, positions, scalar)


def _closed(v, f):
    e = torch.cat([f[:, [0, 1]], f[:, [1, 2]], f[:, [2, 0]]]).long()
    und = torch.minimum(e[:, 0], e[:, 1]) * v.shape[0] + torch.maximum(e[:, 0], e[:, 1])
    directed = e[:, 0] * v.shape[0] + e[:, 1]
    return bool((und.unique(return_counts=True)[1] == 2).all()) and directed.unique().numel() == directed.numel()


def _volume(v, f):
    p = v[f.long()]
    return float((p[:, 0] * torch.cross(p[:, 1], p[:, 2], dim=1)).sum() / 6.0)


def test_simplify_keeps_a_closed_oriented_surface():
    v, f = _sphere()
    assert _closed(v, f) and f.shape[0] > 400
    target = 150
    sv, sf, fmap, vmap = mp.simplify(v, f, target)
    assert sf.shape[0] <= target and sf.shape[0] >= target - 2 and sv.shape[0] < v.shape[0]
    assert _closed(sv, sf)
    assert int(sf.max()) == sv.shape[0] - 1 and int(sf.min()) == 0
    # ancestry indexes the input, every output face descends from a distinct input face
    assert fmap.shape[0] == sf.shape[0] and fmap.unique().numel() == fmap.numel() and int(fmap.max()) < f.shape[0]
    assert vmap.shape[0] == sv.shape[0] and vmap.unique().numel() == vmap.numel() and int(vmap.max()) < v.shape[0]
    # the shape survives: same orientation, volume within a few percent, vertices near the sphere
    assert abs(_volume(sv, sf) - _volume(v, f)) < 0.06 * _volume(v, f)
    assert ((sv - torch.tensor([4.9, 5.1, 5.05])).norm(dim=1) - 3.4).abs().max() < 0.8
    # deterministic, and a target above the face count is the identity
    again = mp.simplify(v, f, target)
    assert torch.equal(again[0], sv) and torch.equal(again[1], sf)
    same = mp.simplify(v, f, f.shape[0] + 5)
    assert torch.equal(same[1], f) and torch.equal(same[2], torch.arange(f.shape[0]))
    # a flat sheet collapses without moving its plane
    n = 9
    gx, gy = torch.meshgrid(torch.arange(n), torch.arange(n), indexing="ij")
    pv = torch.stack([gx.reshape(-1).float(), gy.reshape(-1).float(), torch.full((n * n,), 2.5)], 1)
    quads = [(i * n + j, (i + 1) * n + j, (i + 1) * n + j + 1, i * n + j + 1) for i in range(n - 1) for j in range(n - 1)]
    pf = torch.tensor([t for a, b, c, d in quads for t in ((a, b, c), (a, c, d))], dtype=torch.int32)
    fv, ff, _, _ = mp.simplify(pv, pf, 40)
    assert ff.shape[0] <= 40 and (fv[:, 2] - 2.5).abs().max() < 1e-5
    with pytest.raises(ValueError):
        mp.simplify(v, f, 0)
    with pytest.raises(ValueError):
        mp.simplify(v, f + v.shape[0], 10)


def test_components_and_normalisation():
    v1, f1 = _sphere(g=8, r=2.6, centre=(3.9, 4.1, 4.05))
    v2, f2 = _sphere(g=6, r=1.4, centre=(2.9, 3.1, 3.05))
    v = torch.cat([v1, v2 + 20.0])
    f = torch.cat([f1, f2 + v1.shape[0]])
    share = f2.shape[0] / f.shape[0]
    kv, kf, faces_kept, verts_kept = mp.filter_components(v, f, share + 0.01)
    assert kf.shape[0] == f1.shape[0] and kv.shape[0] == v1.shape[0] and torch.equal(faces_kept, torch.arange(f1.shape[0]))
    assert torch.equal(kv, v1) and torch.equal(kf, f1) and torch.equal(verts_kept, torch.arange(v1.shape[0]))
    both = mp.filter_components(v, f, share - 0.01)
    assert both[1].shape[0] == f.shape[0]
    # the largest component stays even under ratio 1
    assert mp.filter_components(v, f, 1.0)[1].shape[0] == f1.shape[0]
    # a face hanging on by a vertex only is its own component
    lone = torch.cat([f1, torch.tensor([[0, v1.shape[0], v1.shape[0] + 1]], dtype=torch.int32)])
    vv = torch.cat([v1, torch.tensor([[50.0, 0, 0], [50.0, 1, 0]])])
    assert mp.filter_components(vv, lone, 0.5)[1].shape[0] == f1.shape[0]
    with pytest.raises(ValueError):
        mp.filter_components(v, f, 1.5)
    nv = mp.normalize(v1)
    assert nv.mean(dim=0).abs().max() < 1e-6 and nv.norm(dim=1).max().item() == pytest.approx(1.0, abs=1e-6)
    with pytest.raises(ValueError):
        mp.normalize(torch.ones(4, 3))


def test_holes_are_found_and_closed():
    v, f = _sphere(g=8, r=2.6, centre=(3.9, 4.1, 4.05))
    # remove the fan around one vertex and one separate face: two holes
    hub = int(f[0, 0])
    around = (f == hub).any(dim=1)
    far = int(torch.nonzero(~around & ~torch.isin(f, f[around].unique()).any(dim=1))[0])
    keep = ~around
    keep[far] = False
    open_f = f[keep]
    loops = mp.boundary_loops(open_f)
    assert sorted(len(l) for l in loops) == sorted([3, int(around.sum())])
    filled, closed = mp.fill_holes(v, open_f, capacity=16)
    assert closed == 2 and _closed(v, filled)
    assert abs(_volume(v, filled) - _volume(v, f)) < 0.05 * abs(_volume(v, f))           # same orientation as the surface
    small_only, n = mp.fill_holes(v, open_f, capacity=3)
    assert n == 1 and small_only.shape[0] == open_f.shape[0] + 1
    assert mp.fill_holes(v, f, 8)[1] == 0
    with pytest.raises(ValueError):
        mp.fill_holes(v, f, 2)


def test_to_3d_command_runs_the_decode_tail(tmp_path, capsys):
    import json
    from flyingfish_b200 import cli
    from flyingfish_b200.loaders.safetensors_io import save_safetensors
    from flyingfish_b200.utils import media
    # a corner field of a sphere with a small stray blob, saved as the shape decoder would leave it
    g = 10
    idx = torch.stack(torch.meshgrid(torch.arange(g), torch.arange(g), torch.arange(g), indexing="ij"), -1).reshape(-1, 3)
    coords = torch.cat([torch.zeros(idx.shape[0], 1, dtype=torch.long), idx], 1).to(torch.int32)
    s = g + 1
    corner = lambda x, y, z: x + s * (y + s * z)
    cubes = torch.stack([corner(idx[:, 0] + (c & 1), idx[:, 1] + ((c >> 1) & 1), idx[:, 2] + ((c >> 2) & 1)) for c in range(8)], 1)
    lat = torch.stack(torch.meshgrid(torch.arange(s), torch.arange(s), torch.arange(s), indexing="ij"), -1).reshape(-1, 3)
    positions = torch.zeros(s ** 3, 3)
    positions[corner(lat[:, 0], lat[:, 1], lat[:, 2])] = lat.float()
    big = (positions - torch.tensor([4.4, 4.6, 4.5])).norm(dim=1) - 3.1
    blob = (positions - torch.tensor([8.6, 8.5, 8.4])).norm(dim=1) - 0.8
    scalar = torch.minimum(big, blob)
    src = tmp_path / "decoder.safetensors"
    save_safetensors(src, {"coords": coords, "cubes": cubes.to(torch.int32), "positions": positions, "scalar": scalar})
    out = tmp_path / "shape.ply"
    assert cli.main(["--cpu", "to-3d", str(src), "--output", str(out), "--min-component", "0.2", "--faces", "120", "--unit-ball"]) == 0
    report = json.loads(capsys.readouterr().out)
    assert report["surface"] == "dual_contour" and report["output"]["faces"] <= 120
    assert report["components"]["faces_kept"] < report["input"]["faces"]                # the blob is gone
    mesh = media.read_mesh(out.read_bytes(), "ply")
    assert mesh.triangles.shape[0] == report["output"]["faces"] and _closed(mesh.positions, mesh.triangles)
    assert mesh.positions.norm(dim=1).max().item() == pytest.approx(1.0, abs=1e-5)
    # dual-grid fields go the other way in, OBJ comes out; existing outputs are not overwritten
    fields = torch.randn(coords.shape[0], 7, generator=torch.Generator().manual_seed(0))
    src2 = tmp_path / "fields.safetensors"
    save_safetensors(src2, {"coords": coords, "fields": fields})
    assert cli.main(["--cpu", "to-3d", str(src2), "--output", str(tmp_path / "grid.obj"), "--resolution", "10"]) == 0
    assert json.loads(capsys.readouterr().out)["surface"] == "dual_grid" and (tmp_path / "grid.obj").read_text().startswith("v ")
    # a corner field without explicit cubes: values in the order of the shared corner lattice
    from flyingfish_b200.ops import sparse_sites
    corners, _, _, _ = sparse_sites.cube_corners(coords)
    field = (corners[:, 1:].float() - torch.tensor([4.4, 4.6, 4.5])).norm(dim=1) - 3.1
    src3 = tmp_path / "corners.safetensors"
    save_safetensors(src3, {"coords": coords, "scalar": field})
    assert cli.main(["--cpu", "to-3d", str(src3), "--output", str(tmp_path / "ball.ply")]) == 0
    rep = json.loads(capsys.readouterr().out)
    ball = media.read_mesh((tmp_path / "ball.ply").read_bytes(), "ply")
    assert rep["surface"] == "dual_contour" and _closed(ball.positions, ball.triangles)
    save_safetensors(tmp_path / "short.safetensors", {"coords": coords, "scalar": field[:-1]})
    with pytest.raises(SystemExit):
        cli.main(["--cpu", "to-3d", str(tmp_path / "short.safetensors"), "--output", str(tmp_path / "y.ply")])
    with pytest.raises(SystemExit):
        cli.main(["--cpu", "to-3d", str(src2), "--output", str(out), "--resolution", "10"])
    with pytest.raises(SystemExit):
        cli.main(["--cpu", "to-3d", str(src2), "--output", str(tmp_path / "x.ply")])                  # no --resolution
    with pytest.raises(SystemExit):
        cli.main(["--cpu", "to-3d", str(src2), "--output", str(tmp_path / "x.stl"), "--resolution", "10"])
