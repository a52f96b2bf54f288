"""Surface extraction from sparse voxel grids: cube topology, the per-voxel dual grid and dual contouring of a corner field."""
import io

import pytest
import torch

from flyingfish_b200.ops import mesh_ops as mo


def test_cube_topology_table():
    t = mo.cube_topology()
    assert t.shape == (256, 14) and t.dtype == torch.int8
    assert t[0, 12] == 0 and t[255, 12] == 0 and (t[0, :12] == -1).all()
    # one corner inside: its three edges form one component
    row = t[1]
    assert row[12] == 1 and sorted(e for e in range(12) if row[e] == 0) == [0, 4, 8]
    assert int(t[:, 12].max()) == 4 and int(t[0b01101001, 12]) == 4           # four isolated corners
    # an edge is labelled exactly when its end points differ in sign
    for mask in (0b00010111, 0b10000001, 0b00111100):
        for e in range(12):
            a, b = mo._edge_corners(e)
            assert (t[mask, e] >= 0) == (((mask >> a) ^ (mask >> b)) & 1 == 1)
    # two opposite corners of the bottom face: separate here, joined in the complement -> the face is marked there
    mask = 0b00001001
    assert t[mask, 12] == 2 and t[mask ^ 255, 12] == 1
    assert t[mask ^ 255, 13] & (1 << 4) and not t[mask, 13] & (1 << 4)        # face z = 0 is 2 * 2 + 0
    # edge numbering: 4 * axis + lower corner without the axis bit
    assert [mo._edge_corners(e) for e in (0, 3, 4, 7, 8, 11)] == [(0, 1), (6, 7), (0, 2), (5, 7), (0, 4), (3, 7)]


def _sparse_coords(g: int, keep: float, seed: int) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    grid = torch.stack(torch.meshgrid(torch.arange(g), torch.arange(g), torch.arange(g), indexing="ij"), -1).reshape(-1, 3)
    grid = grid[torch.rand(grid.shape[0], generator=gen) < keep]
    grid = grid[torch.randperm(grid.shape[0], generator=gen)]
    return torch.cat([torch.zeros(grid.shape[0], 1, dtype=torch.long), grid], 1).to(torch.int32)


def test_dual_grid_mesh_matches_the_per_voxel_restatement():
    coords = _sparse_coords(6, 0.7, 0)
    gen = torch.Generator().manual_seed(1)
    fields = torch.randn(coords.shape[0], 7, generator=gen) * 2.0
    fields[0, 6] = 25.0                                                        # the large-argument branch of softplus
    v, f = mo.dual_grid_mesh(coords, fields, 6)
    rv, rf = mo.dual_grid_mesh_reference(coords, fields, 6)
    assert torch.allclose(v, rv, atol=1e-6) and torch.equal(f, rf) and f.shape[0] > 20 and f.shape[0] % 2 == 0
    # vertices stay inside their voxel stretched by half a cell, in [-0.5, 0.5) world units
    cell = (v - (-0.5)) * 6 - coords[:, 1:].float()
    assert (cell > -0.5).all() and (cell < 1.5).all()
    # no flagged edge, no face; a lone voxel has no quad
    quiet = fields.clone()
    quiet[:, 3:6] = -1.0
    assert mo.dual_grid_mesh(coords, quiet, 6)[1].shape == (0, 3)
    assert mo.dual_grid_mesh(coords[:1], fields[:1].abs(), 6)[1].shape == (0, 3)
    with pytest.raises(ValueError):
        mo.dual_grid_mesh(coords, fields[:, :6], 6)
    with pytest.raises(ValueError):
        mo.dual_grid_mesh(coords, fields, 5)                                   # a voxel outside the grid


def _dense_block(g: int):
    """All cubes of a g^3 block with shared corners on the (g + 1)^3 lattice (corner c: x = bit 0)."""
    idx = torch.stack(torch.meshgrid(torch.arange(g), torch.arange(g), torch.arange(g), indexing="ij"), -1).reshape(-1, 3)
    coords = torch.cat([torch.zeros(idx.shape[0], 1, dtype=torch.long), idx], 1).to(torch.int32)
    s = g + 1
    corner = lambda x, y, z: x + s * (y + s * z)
    cubes = torch.stack([corner(idx[:, 0] + (c & 1), idx[:, 1] + ((c >> 1) & 1), idx[:, 2] + ((c >> 2) & 1)) for c in range(8)], 1)
    lat = torch.stack(torch.meshgrid(torch.arange(s), torch.arange(s), torch.arange(s), indexing="ij"), -1).reshape(-1, 3)
    positions = torch.zeros(s ** 3, 3)
    positions[corner(lat[:, 0], lat[:, 1], lat[:, 2])] = lat.float()
    return coords, cubes, positions


def test_dual_contouring_of_a_sphere_is_closed_and_on_the_surface():
    g, r = 8, 2.7
    coords, cubes, positions = _dense_block(g)
    centre = torch.tensor([3.9, 4.1, 4.05])
    scalar = (positions - centre).norm(dim=1) - r
    v, f = mo.dual_contour_mesh(coords, cubes, positions, scalar)
    rv, rf = mo.dual_contour_mesh_reference(coords, cubes, positions, scalar)
    assert torch.allclose(v, rv, atol=1e-5) and torch.equal(f, rf) and f.shape[0] > 100
    # every vertex is a mean of crossings of the sphere: within a cell diagonal of the surface
    assert ((v - centre).norm(dim=1) - r).abs().max() < 0.9
    # the surface is closed: every undirected edge belongs to exactly two triangles, every directed edge to one
    e = torch.cat([f[:, [0, 1]], f[:, [1, 2]], f[:, [2, 0]]]).long()
    directed = e[:, 0] * v.shape[0] + e[:, 1]
    assert directed.unique().numel() == directed.numel()
    undirected = torch.minimum(e[:, 0], e[:, 1]) * v.shape[0] + torch.maximum(e[:, 0], e[:, 1])
    assert (undirected.unique(return_counts=True)[1] == 2).all()
    # outward orientation: the signed volume is positive and close to the sphere's
    p = v[f.long()]
    volume = (p[:, 0] * torch.cross(p[:, 1], p[:, 2], dim=1)).sum() / 6.0
    sphere = 4.0 / 3.0 * 3.14159265 * r ** 3
    assert 0.8 * sphere < float(volume) < sphere                                # chords of a coarse grid lie inside the sphere
    # a shuffled cube order gives the same surface up to numbering
    perm = torch.randperm(coords.shape[0], generator=torch.Generator().manual_seed(2))
    v2, f2 = mo.dual_contour_mesh(coords[perm], cubes[perm], positions, scalar)
    assert v2.shape == v.shape and f2.shape == f.shape
    with pytest.raises(ValueError):
        mo.cube_sign_masks(torch.tensor([float("nan")]), torch.zeros(1, 8, dtype=torch.long))


def test_ambiguous_faces_are_resolved_consistently():
    # random fields produce ambiguous faces; the two builders must still agree, and masks with up to four components occur
    g = 5
    coords, cubes, positions = _dense_block(g)
    gen = torch.Generator().manual_seed(3)
    scalar = torch.randn(positions.shape[0], generator=gen)
    masks = mo.cube_sign_masks(scalar, cubes)
    resolved, counts = mo.resolve_components(coords, masks)
    assert int(counts.max()) >= 2 and bool((resolved != masks).any())
    v, f = mo.dual_contour_mesh(coords, cubes, positions, scalar)
    rv, rf = mo.dual_contour_mesh_reference(coords, cubes, positions, scalar)
    assert v.shape[0] == int(counts.sum()) and torch.allclose(v, rv, atol=1e-5) and torch.equal(f, rf)
    # a sparse subset of the cubes: quads need all four cubes around an edge
    keep = torch.rand(coords.shape[0], generator=gen) < 0.6
    v3, f3 = mo.dual_contour_mesh(coords[keep], cubes[keep], positions, scalar)
    rv3, rf3 = mo.dual_contour_mesh_reference(coords[keep], cubes[keep], positions, scalar)
    assert torch.allclose(v3, rv3, atol=1e-5) and torch.equal(f3, rf3) and f3.shape[0] < f.shape[0]


def test_mesh_goes_out_as_ply():
    from flyingfish_b200.utils import media
    coords = _sparse_coords(4, 0.9, 5)
    fields = torch.randn(coords.shape[0], 7, generator=torch.Generator().manual_seed(6))
    v, f = mo.dual_grid_mesh(coords, fields, 4)
    buf = io.BytesIO()
    media.write_ply(buf, media.Mesh(v, f))
    back = media.read_mesh(buf.getvalue(), "ply")
    assert torch.equal(back.positions, v) and torch.equal(back.triangles, f)


@pytest.mark.gpu
def test_mesh_builders_on_the_device():
    coords = _sparse_coords(8, 0.7, 7)
    fields = torch.randn(coords.shape[0], 7, generator=torch.Generator().manual_seed(8)) * 2.0
    v, f = mo.dual_grid_mesh(coords.cuda(), fields.cuda(), 8)
    rv, rf = mo.dual_grid_mesh_reference(coords, fields, 8)
    assert torch.allclose(v.cpu(), rv, atol=1e-5) and torch.equal(f.cpu(), rf)
    g = 8
    coords, cubes, positions = _dense_block(g)
    scalar = (positions - torch.tensor([3.9, 4.1, 4.05])).norm(dim=1) - 2.7
    v, f = mo.dual_contour_mesh(coords.cuda(), cubes.cuda(), positions.cuda(), scalar.cuda())
    rv, rf = mo.dual_contour_mesh_reference(coords, cubes, positions, scalar)
    assert torch.allclose(v.cpu(), rv, atol=1e-4) and torch.equal(f.cpu(), rf)
    cells, owners = mo.triangle_voxels(v, f, g)
    rc, ro = mo.triangle_voxels(v.cpu(), f.cpu(), g)
    # touching cases may differ in the last bit between devices: compare the bulk
    assert abs(cells.shape[0] - rc.shape[0]) <= 0.01 * rc.shape[0] + 2


def test_triangle_voxels():
    # a triangle in the plane z = 0.5 over a 4 x 4 x 4 grid: exactly the cells of layer z = 0 its area touches
    v = torch.tensor([[0.2, 0.2, 0.5], [3.7, 0.2, 0.5], [0.2, 3.7, 0.5]])
    f = torch.tensor([[0, 1, 2]])
    cells, owners = mo.triangle_voxels(v, f, 4)
    assert (cells[:, 2] == 0).all() and (owners == 0).all()
    got = {tuple(c) for c in cells[:, :2].tolist()}
    assert got == {(x, y) for x in range(4) for y in range(4) if x + y <= 3}
    # random triangles, some partly outside the grid: the batched test equals the per-cell restatement, order included
    gen = torch.Generator().manual_seed(4)
    v = torch.rand(30, 3, generator=gen) * 8.0 - 1.0
    f = torch.randint(0, 30, (25, 3), generator=gen)
    cells, owners = mo.triangle_voxels(v, f, 6)
    rc, ro = mo.triangle_voxels_reference(v, f, 6)
    assert torch.equal(cells, rc) and torch.equal(owners, ro) and cells.shape[0] > 50
    assert (cells >= 0).all() and (cells < 6).all()
    # a triangle outside the grid gives nothing
    out = mo.triangle_voxels(torch.tensor([[9.0, 9, 9], [10, 9, 9], [9, 10, 9]]), f[:1] * 0 + torch.tensor([[0, 1, 2]]), 4)
    assert out[0].shape == (0, 3)
    # the voxels of an extracted sphere contain every vertex of its mesh
    coords, cubes, positions = _dense_block(8)
    scalar = (positions - torch.tensor([3.9, 4.1, 4.05])).norm(dim=1) - 2.7
    mv, mf = mo.dual_contour_mesh(coords, cubes, positions, scalar)
    cells, _ = mo.triangle_voxels(mv, mf, 8)
    occ = mo.occupied_voxels(cells, 8)
    assert occ.shape[1] == 4 and occ.shape[0] == len({tuple(c) for c in cells.tolist()})
    have = {tuple(c[1:]) for c in occ.tolist()}
    assert all(tuple(int(t) for t in p.floor().tolist()) in have for p in mv)
    with pytest.raises(ValueError):
        mo.triangle_voxels(v, f, 0)
