"""Surface extraction from sparse voxel grids: the two mesh builders of the image-to-3D decoders.

* ``dual_grid_mesh``: every occupied voxel carries one vertex (an offset inside the voxel) and three edge flags; a
  flagged edge whose four surrounding voxels exist becomes a quad, split along the diagonal the vertices' split weights
  prefer (kernels/vision_ops.cu ``dual_grid_head_f32`` / ``sparse_cube_edge_ids`` / ``quad_diagonal_f32`` /
  ``sparse_face_compact`` and src/backend/cuda/sparse.rs:723-930 of the reference).
* ``dual_contour_mesh``: a scalar field on the voxel corners; every cube gets one vertex per connected component of its
  sign-changing edges (up to four, from a 256-row topology table; ambiguous faces are resolved against the neighbour), a
  vertex sits at the mean of its component's edge crossings, and every sign-changing grid edge with four cubes around it
  becomes a quad (``cube_sign_masks_f32`` / ``cube_resolved_components_u8`` / ``cube_dual_vertices_f32`` /
  ``sparse_cube_component_edge_ids``; topology table src/sparse.rs:1120-1240).

B200 mapping: neighbour look-ups go through the voxel hash kernels (``vision_ops.VoxelHash``); everything else is
whole-array arithmetic over all voxels, edges or components at once on the tensors' device: offsets by prefix sums and
compaction by masks replace the reference's count / scan / emit kernel triples, with the same stable order (edge id =
3 * voxel row + axis). ``*_reference`` are plain per-voxel restatements used as oracles by the tests."""
from __future__ import annotations

import functools
import math

import torch

from .vision_ops import VoxelHash


# ------------------------------------------------------------------------------------------------
# cube topology
# ------------------------------------------------------------------------------------------------
def _edge_corners(edge: int) -> tuple[int, int]:
    """Edge = 4 * axis + (lower corner with the axis bit squeezed out); corners use x = bit 0."""
    axis, packed = divmod(edge, 4)
    lower = (packed & ((1 << axis) - 1)) | ((packed >> axis) << (axis + 1))
    return lower, lower | (1 << axis)


def _face_edges(axis: int, side: int) -> list[int]:
    """The four edges around the face ``axis = side`` in rim order."""
    o = [a for a in range(3) if a != axis]
    base = side << axis
    corners = [base, base | (1 << o[0]), base | (1 << o[0]) | (1 << o[1]), base | (1 << o[1])]
    out = []
    for i in range(4):
        a, b = corners[i], corners[(i + 1) % 4]
        d = (a ^ b).bit_length() - 1
        lower = min(a, b)
        out.append(4 * d + (lower & ((1 << d) - 1)) + ((lower >> (d + 1)) << d))
    return out


def _components(mask: int) -> list[int]:
    crossing = [((mask >> a) ^ (mask >> b)) & 1 == 1 for a, b in map(_edge_corners, range(12))]
    adj: list[set[int]] = [set() for _ in range(12)]
    for axis in range(3):
        for side in range(2):
            rim = _face_edges(axis, side)
            sel = [e for e in rim if crossing[e]]
            if len(sel) == 2:
                adj[sel[0]].add(sel[1]); adj[sel[1]].add(sel[0])
            elif len(sel) == 4:
                # an ambiguous face: edges are joined around the corners that are inside
                for i in range(4):
                    prev, cur = rim[(i + 3) % 4], rim[i]
                    corner = next(c for c in _edge_corners(cur) if c in _edge_corners(prev))
                    if mask & (1 << corner):
                        adj[prev].add(cur); adj[cur].add(prev)
            elif sel:
                raise AssertionError("cube face crossing parity")
    labels = [-1] * 12
    comp = 0
    for edge in sorted(range(12), key=_edge_corners):
        if not crossing[edge] or labels[edge] >= 0:
            continue
        todo = [edge]
        while todo:
            e = todo.pop()
            if labels[e] < 0:
                labels[e] = comp
                todo += list(adj[e])
        comp += 1
    if comp > 4:
        raise AssertionError("more than four dual vertices in a cube")
    return labels


@functools.lru_cache(maxsize=1)
def cube_topology() -> torch.Tensor:
    """int8 [256, 14]: per corner sign mask the component id of each of the 12 edges (-1: no crossing), the number of
    components, and six bits (face = 2 * axis + side) marking faces whose four edges are crossed and joined into one
    component here but not in the complementary mask -- the faces where two cubes may disagree."""
    table = [[-1] * 14 for _ in range(256)]
    for mask in range(256):
        lab = _components(mask)
        table[mask][:12] = lab
        table[mask][12] = max(lab) + 1
        table[mask][13] = 0
    for mask in range(256):
        for axis in range(3):
            for side in range(2):
                rim = _face_edges(axis, side)
                if all(table[mask][e] >= 0 for e in rim):
                    own, opp = table[mask][rim[0]], table[mask ^ 255][rim[0]]
                    if all(table[mask][e] == own for e in rim) and any(table[mask ^ 255][e] != opp for e in rim):
                        table[mask][13] |= 1 << (2 * axis + side)
    return torch.tensor(table, dtype=torch.int8)


# ------------------------------------------------------------------------------------------------
# shared: quads -> triangles
# ------------------------------------------------------------------------------------------------
def split_quads(quads: torch.Tensor, diagonal: torch.Tensor) -> torch.Tensor:
    """quads [m, 4] (vertex ids in the order base, +second, +first, +both) -> triangles [2 m, 3]; ``diagonal`` picks
    the split: (0 1 3)(0 3 2) when set, (0 1 2)(2 1 3) otherwise. Winding, duplicates and degenerate faces are kept."""
    q = quads.long()
    d = diagonal.bool()[:, None]
    first = torch.where(d, q[:, [0, 1, 3]], q[:, [0, 1, 2]])
    second = torch.where(d, q[:, [0, 3, 2]], q[:, [2, 1, 3]])
    return torch.stack([first, second], dim=1).reshape(-1, 3).to(torch.int32)


def _unit(axis: int) -> list[int]:
    return [1 if a == axis else 0 for a in range(3)]


# ------------------------------------------------------------------------------------------------
# dual grid: one vertex per voxel
# ------------------------------------------------------------------------------------------------
def dual_grid_mesh(coords: torch.Tensor, fields: torch.Tensor, resolution: int, origin: float = -0.5
                   ) -> tuple[torch.Tensor, torch.Tensor]:
    """coords [n, 4] int32 (batch, x, y, z; unique), fields [n, 7] FP32 = (vertex offset logits x y z, edge logits x y
    z, split logit). Returns (vertices [n, 3] FP32 in world units, triangles [f, 3] int32)."""
    n = coords.shape[0]
    if fields.shape != (n, 7) or resolution <= 0 or not math.isfinite(origin):
        raise ValueError("invalid dual grid fields")
    f = fields.float()
    if not torch.isfinite(f).all():
        raise ValueError("non-finite dual grid field")
    xyz = coords[:, 1:].to(f.device)
    if bool(((xyz < 0) | (xyz >= resolution)).any()):
        raise ValueError("voxel outside the grid")
    dual = 2.0 * torch.sigmoid(f[:, :3]) - 0.5
    vertices = (xyz.float() + dual) / float(resolution) + origin
    flags = f[:, 3:6] > 0.0
    weight = torch.where(f[:, 6] > 20.0, f[:, 6], torch.log1p(torch.exp(f[:, 6].clamp(max=20.0))))        # softplus
    offs = []
    for axis in range(3):
        a, b = (axis + 1) % 3, (axis + 2) % 3
        ua, ub = _unit(a), _unit(b)
        offs += [ub, ua, [x + y for x, y in zip(ua, ub)]]
    nbr = VoxelHash(coords.contiguous()).neighbor_map(torch.tensor(offs, dtype=torch.int32, device=coords.device)).long()   # [9, n]
    rows = torch.arange(n, device=coords.device)
    quads = torch.stack([torch.stack([rows, nbr[3 * ax], nbr[3 * ax + 1], nbr[3 * ax + 2]], dim=1) for ax in range(3)], dim=1)   # [n, 3, 4]
    keep = flags.to(coords.device) & (quads.min(dim=2).values >= 0)
    q = quads[keep]                                                     # edge order: 3 * row + axis
    w = weight.to(q.device)
    diagonal = w[q[:, 0]] * w[q[:, 3]] > w[q[:, 1]] * w[q[:, 2]]
    return vertices, split_quads(q, diagonal)


def dual_grid_mesh_reference(coords: torch.Tensor, fields: torch.Tensor, resolution: int, origin: float = -0.5):
    """Per-voxel restatement (dictionary look-ups, scalar arithmetic in FP32)."""
    c = coords.cpu().tolist()
    f = fields.float().cpu()
    index = {tuple(p): i for i, p in enumerate(c)}
    dual = 2.0 * torch.sigmoid(f[:, :3]) - 0.5
    verts = (torch.tensor([p[1:] for p in c], dtype=torch.float32) + dual) / float(resolution) + origin
    w = torch.nn.functional.softplus(f[:, 6], threshold=20.0)
    faces = []
    for row, p in enumerate(c):
        for axis in range(3):
            if not f[row, 3 + axis] > 0:
                continue
            a, b = (axis + 1) % 3 + 1, (axis + 2) % 3 + 1
            q = [row]
            for da, db in ((0, 1), (1, 0), (1, 1)):
                t = list(p)
                t[a] += da
                t[b] += db
                q.append(index.get(tuple(t), -1))
            if min(q) < 0:
                continue
            if float(w[q[0]] * w[q[3]]) > float(w[q[1]] * w[q[2]]):
                faces += [[q[0], q[1], q[3]], [q[0], q[3], q[2]]]
            else:
                faces += [[q[0], q[1], q[2]], [q[2], q[1], q[3]]]
    return verts, torch.tensor(faces, dtype=torch.int32).reshape(-1, 3)


# ------------------------------------------------------------------------------------------------
# dual contouring of a corner field: one vertex per edge component of a cube
# ------------------------------------------------------------------------------------------------
def cube_sign_masks(scalar: torch.Tensor, cubes: torch.Tensor) -> torch.Tensor:
    """scalar [corners] FP32, cubes [n, 8] corner ids (corner c of a cube has x = bit 0) -> uint8 sign masks (bit c set
    where the field is negative)."""
    if not torch.isfinite(scalar).all():
        raise ValueError("non-finite scalar field")
    if cubes.numel() and (int(cubes.min()) < 0 or int(cubes.max()) >= scalar.numel()):
        raise ValueError("cube corner outside the corner arrays")
    neg = (scalar[cubes.long()] < 0).to(torch.int32)
    weights = (1 << torch.arange(8, device=neg.device, dtype=torch.int32))
    return (neg * weights).sum(dim=1).to(torch.uint8)


def resolve_components(coords: torch.Tensor, masks: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """A cube takes the complementary mask's components when one of its ambiguous faces meets a neighbour whose facing
    face is ambiguous too. Returns (resolved masks uint8 [n], dual vertices per cube int64 [n])."""
    table = cube_topology().to(masks.device)
    crit = table[masks.long(), 13].to(torch.int32)
    offs = [[(-1 if side == 0 else 1) * u for u in _unit(axis)] for axis in range(3) for side in range(2)]
    nbr = VoxelHash(coords.contiguous()).neighbor_map(torch.tensor(offs, dtype=torch.int32, device=coords.device)).long()   # [6, n]
    split = torch.zeros_like(masks, dtype=torch.bool)
    for axis in range(3):
        for side in range(2):
            k = 2 * axis + side
            other = nbr[k]
            facing = torch.where(other >= 0, crit[other.clamp(min=0)], torch.zeros_like(crit))
            split |= ((crit >> k) & 1).bool() & (other >= 0) & ((facing >> (2 * axis + 1 - side)) & 1).bool()
    resolved = torch.where(split, masks ^ 255, masks)
    return resolved, table[resolved.long(), 12].long()


def dual_contour_mesh(coords: torch.Tensor, cubes: torch.Tensor, positions: torch.Tensor, scalar: torch.Tensor
                      ) -> tuple[torch.Tensor, torch.Tensor]:
    """coords [n, 4] int32 (unique cubes), cubes [n, 8] corner ids, positions [corners, 3] and scalar [corners] FP32.
    Returns (vertices [v, 3] FP32, triangles [f, 3] int32); the vertices of cube r are rows offsets[r] .. of the output
    in component order."""
    n = coords.shape[0]
    dev = scalar.device
    table = cube_topology().to(dev)
    masks = cube_sign_masks(scalar, cubes)
    resolved, counts = resolve_components(coords, masks)
    offsets = torch.cumsum(counts, 0) - counts                          # exclusive scan
    total = int(counts.sum())
    comp = table[resolved.long(), :12].long()                           # [n, 12]
    # crossing point of every edge of every cube
    lower = torch.tensor([_edge_corners(e)[0] for e in range(12)], device=dev)
    upper = torch.tensor([_edge_corners(e)[1] for e in range(12)], device=dev)
    ca, cb = cubes.long()[:, lower], cubes.long()[:, upper]           # [n, 12]
    sa, sb = scalar[ca], scalar[cb]
    live = comp >= 0
    denom = torch.where(live, sa - sb, torch.ones_like(sa))
    if bool((live & (((sa < 0) == (sb < 0)) | (denom == 0))).any()):
        raise ValueError("component edge without a sign change")
    t = sa / denom
    pa, pb = positions[ca], positions[cb]                               # [n, 12, 3]
    point = pa + t[..., None] * (pb - pa)
    # mean per component, accumulated relative to the component's first point as the scalar kernel does
    vertices = torch.zeros(total, 3, dtype=torch.float32, device=dev)
    for g in range(4):
        sel = comp == g                                                 # [n, 12]
        has = sel.any(dim=1)
        if not bool(has.any()):
            continue
        first = sel.float().argmax(dim=1)                               # first edge of the component
        base = point[torch.arange(n, device=dev), first]                # [n, 3]
        s = ((point - base[:, None, :]) * sel[..., None]).sum(dim=1)
        cnt = sel.sum(dim=1).clamp(min=1).float()[:, None]
        v = base + s / cnt
        vertices[(offsets + g)[has]] = v[has]
    if not torch.isfinite(vertices).all():
        raise ValueError("non-finite dual vertex")
    # quads around the sign-changing edge along `axis` at the cube's far corner
    nbr_table = VoxelHash(coords.contiguous())
    quads, diags = [], []
    rows = torch.arange(n, device=coords.device)
    for axis in range(3):
        b, c = (axis + 1) % 3, (axis + 2) % 3
        lo = (1 << b) | (1 << c)
        start, stop = scalar[cubes.long()[:, lo]], scalar[cubes.long()[:, lo | (1 << axis)]]
        ub, uc = _unit(b), _unit(c)
        offs = torch.tensor([ub, [x + y for x, y in zip(ub, uc)], uc], dtype=torch.int32, device=coords.device)
        nb = nbr_table.neighbor_map(offs).long()                        # [3, n]
        adjacent = torch.stack([rows, nb[0], nb[1], nb[2]], dim=1)      # [n, 4]
        ok = ((start < 0) != (stop < 0)).to(coords.device) & (adjacent.min(dim=1).values >= 0)
        cyc = []
        for j in range(4):
            local = ((1 << b) if j in (0, 3) else 0) | ((1 << c) if j < 2 else 0)
            packed = (local & ((1 << axis) - 1)) | ((local >> (axis + 1)) << axis)
            other = adjacent[:, j].clamp(min=0)
            component = table[resolved.long()[other], axis * 4 + packed].long()
            if bool((ok & (component < 0)).any()):
                raise ValueError("quad corner without a dual vertex")
            cyc.append(offsets[other] + component)
        cyc = torch.stack(cyc, dim=1)
        flip = (start > 0)[:, None].to(cyc.device)
        cyc = torch.where(flip, cyc.flip(1), cyc)
        q = torch.stack([cyc[:, 0], cyc[:, 1], cyc[:, 3], cyc[:, 2]], dim=1)
        quads.append(torch.where(ok[:, None], q, torch.full_like(q, -1)))
        diags.append(torch.full((n,), axis != 1, dtype=torch.bool, device=coords.device))
    quads = torch.stack(quads, dim=1).reshape(-1, 4)                    # edge order: 3 * row + axis
    diags = torch.stack(diags, dim=1).reshape(-1)
    keep = quads[:, 0] >= 0
    return vertices, split_quads(quads[keep], diags[keep])


def dual_contour_mesh_reference(coords: torch.Tensor, cubes: torch.Tensor, positions: torch.Tensor, scalar: torch.Tensor):
    """Per-cube restatement of :func:`dual_contour_mesh` with dictionary look-ups and scalar loops."""
    table = cube_topology().tolist()
    c = coords.cpu().tolist()
    cu = cubes.cpu().tolist()
    sc = scalar.float().cpu().tolist()
    pos = positions.float().cpu()
    index = {tuple(p): i for i, p in enumerate(c)}
    n = len(c)
    masks = [sum((1 << k) for k in range(8) if sc[cu[r][k]] < 0) for r in range(n)]
    resolved = []
    for r in range(n):
        crit, split = table[masks[r]][13], False
        for axis in range(3):
            for side in range(2):
                if not crit & (1 << (2 * axis + side)):
                    continue
                t = list(c[r])
                t[axis + 1] += 1 if side else -1
                o = index.get(tuple(t), -1)
                if o >= 0 and table[masks[o]][13] & (1 << (2 * axis + 1 - side)):
                    split = True
        resolved.append(masks[r] ^ 255 if split else masks[r])
    offsets, verts = [0], []
    for r in range(n):
        row = table[resolved[r]]
        for g in range(row[12]):
            pts = []
            for e in range(12):
                if row[e] != g:
                    continue
                lo, hi = _edge_corners(e)
                a, b = cu[r][lo], cu[r][hi]
                t = torch.tensor(sc[a], dtype=torch.float32) / (torch.tensor(sc[a], dtype=torch.float32) - torch.tensor(sc[b], dtype=torch.float32))
                pts.append(pos[a] + t * (pos[b] - pos[a]))
            base = pts[0]
            acc = torch.zeros(3)
            for p in pts:
                acc = acc + (p - base)
            verts.append(base + acc / float(len(pts)))
        offsets.append(offsets[-1] + row[12])
    faces = []
    for r in range(n):
        for axis in range(3):
            b, cc = (axis + 1) % 3, (axis + 2) % 3
            lo = (1 << b) | (1 << cc)
            start, stop = sc[cu[r][lo]], sc[cu[r][lo | (1 << axis)]]
            if (start < 0) == (stop < 0):
                continue
            adj = [r]
            for db, dc in ((1, 0), (1, 1), (0, 1)):
                t = list(c[r])
                t[b + 1] += db
                t[cc + 1] += dc
                adj.append(index.get(tuple(t), -1))
            if min(adj) < 0:
                continue
            cyc = []
            for j in range(4):
                local = ((1 << b) if j in (0, 3) else 0) | ((1 << cc) if j < 2 else 0)
                packed = (local & ((1 << axis) - 1)) | ((local >> (axis + 1)) << axis)
                cyc.append(offsets[adj[j]] + table[resolved[adj[j]]][axis * 4 + packed])
            if start > 0:
                cyc = cyc[::-1]
            q = [cyc[0], cyc[1], cyc[3], cyc[2]]
            if axis != 1:
                faces += [[q[0], q[1], q[3]], [q[0], q[3], q[2]]]
            else:
                faces += [[q[0], q[1], q[2]], [q[2], q[1], q[3]]]
    v = torch.stack(verts) if verts else torch.zeros(0, 3)
    return v, torch.tensor(faces, dtype=torch.int32).reshape(-1, 3)


# ------------------------------------------------------------------------------------------------
# triangles -> voxels
# ------------------------------------------------------------------------------------------------
def _dot3(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    # the summation order of the scalar kernel: fma(a2, b2, fma(a0, b0, a1 * b1))
    return a[..., 2] * b[..., 2] + (a[..., 0] * b[..., 0] + a[..., 1] * b[..., 1])


def triangle_voxels(vertices: torch.Tensor, faces: torch.Tensor, resolution: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Every (voxel, triangle) pair that overlaps, for triangles given in voxel units over the grid ``[0, resolution)^3``
    (kernels/vision_ops.cu ``triangle_box_count`` / ``triangle_box_emit`` of the reference: the separating-axis test of a
    triangle against a unit cube -- three box axes, nine edge cross products, the triangle's plane). Returns
    (voxels [m, 3] int32, owners [m] int32), triangles in order and the voxels of a triangle in x, y, z order. All
    candidate cells of all triangles are tested at once."""
    if vertices.dim() != 2 or vertices.shape[1] != 3 or faces.dim() != 2 or faces.shape[1] != 3 or resolution <= 0:
        raise ValueError("triangle_voxels: vertices [n, 3], faces [f, 3], positive resolution")
    if not torch.isfinite(vertices).all():
        raise ValueError("non-finite vertex")
    dev = vertices.device
    pts = vertices.float()[faces.long()]                                 # [f, 3 vertices, 3 axes]
    lower = torch.floor(pts.min(dim=1).values).clamp(min=0).long()
    upper = torch.floor(pts.max(dim=1).values).clamp(max=resolution - 1).long()
    size = (upper - lower + 1).clamp(min=0)
    count = size.prod(dim=1)
    total = int(count.sum())
    if total == 0:
        return torch.zeros(0, 3, dtype=torch.int32, device=dev), torch.zeros(0, dtype=torch.int32, device=dev)
    owner = torch.repeat_interleave(torch.arange(faces.shape[0], device=dev), count)
    local = torch.arange(total, device=dev) - torch.repeat_interleave(torch.cumsum(count, 0) - count, count)
    sz = size[owner]
    z = local % sz[:, 2]
    y = (local // sz[:, 2]) % sz[:, 1]
    x = local // (sz[:, 2] * sz[:, 1])
    cell = torch.stack([x, y, z], dim=1) + lower[owner]
    p = pts[owner] - (cell.float() + 0.5)[:, None, :]                    # triangle relative to the cell centre
    edges = p[:, [1, 2, 0]] - p
    ok = ~((p.min(dim=1).values > 0.5) | (p.max(dim=1).values < -0.5)).any(dim=1)
    for e in range(3):
        for a in range(3):
            axis = torch.zeros_like(p[:, 0])
            axis[:, (a + 1) % 3] = edges[:, e, (a + 2) % 3]
            axis[:, (a + 2) % 3] = -edges[:, e, (a + 1) % 3]
            proj = torch.stack([_dot3(p[:, v], axis) for v in range(3)], dim=1)
            radius = 0.5 * ((axis[:, 0].abs() + axis[:, 1].abs()) + axis[:, 2].abs())
            ok &= (proj.min(dim=1).values <= radius) & (proj.max(dim=1).values >= -radius)
    normal = torch.stack([edges[:, 0, (a + 1) % 3] * edges[:, 1, (a + 2) % 3] - edges[:, 0, (a + 2) % 3] * edges[:, 1, (a + 1) % 3]
                          for a in range(3)], dim=1)
    radius = 0.5 * ((normal[:, 0].abs() + normal[:, 1].abs()) + normal[:, 2].abs())
    ok &= _dot3(p[:, 0], normal).abs() <= radius
    return cell[ok].to(torch.int32), owner[ok].to(torch.int32)


def triangle_voxels_reference(vertices: torch.Tensor, faces: torch.Tensor, resolution: int):
    """Per-triangle, per-cell restatement of :func:`triangle_voxels`."""
    v = vertices.float().cpu()
    cells, owners = [], []
    f32 = lambda t: torch.tensor(t, dtype=torch.float32)
    for fi, face in enumerate(faces.cpu().tolist()):
        tri = v[face]
        lo = [max(0, int(math.floor(float(tri[:, a].min())))) for a in range(3)]
        hi = [min(resolution - 1, int(math.floor(float(tri[:, a].max())))) for a in range(3)]
        for x in range(lo[0], hi[0] + 1):
            for y in range(lo[1], hi[1] + 1):
                for z in range(lo[2], hi[2] + 1):
                    p = tri - (f32([x, y, z]) + 0.5)
                    e = p[[1, 2, 0]] - p
                    hit = not any(float(p[:, a].min()) > 0.5 or float(p[:, a].max()) < -0.5 for a in range(3))
                    for k in range(3):
                        for a in range(3):
                            ax = torch.zeros(3)
                            ax[(a + 1) % 3] = e[k, (a + 2) % 3]
                            ax[(a + 2) % 3] = -e[k, (a + 1) % 3]
                            proj = _dot3(p, ax[None, :])
                            rad = 0.5 * ((ax[0].abs() + ax[1].abs()) + ax[2].abs())
                            hit = hit and bool(proj.min() <= rad) and bool(proj.max() >= -rad)
                    n = torch.stack([e[0, (a + 1) % 3] * e[1, (a + 2) % 3] - e[0, (a + 2) % 3] * e[1, (a + 1) % 3] for a in range(3)])
                    rad = 0.5 * ((n[0].abs() + n[1].abs()) + n[2].abs())
                    hit = hit and bool(_dot3(p[0], n).abs() <= rad)
                    if hit:
                        cells.append([x, y, z])
                        owners.append(fi)
    return torch.tensor(cells, dtype=torch.int32).reshape(-1, 3), torch.tensor(owners, dtype=torch.int32)


def occupied_voxels(voxels: torch.Tensor, resolution: int) -> torch.Tensor:
    """Unique voxels of a (voxel, triangle) list in x, y, z order, as sparse coordinates [m, 4] int32 of batch 0."""
    key = (voxels[:, 0].long() * resolution + voxels[:, 1].long()) * resolution + voxels[:, 2].long()
    u = torch.unique(key)
    xyz = torch.stack([u // (resolution * resolution), (u // resolution) % resolution, u % resolution], dim=1)
    return torch.cat([torch.zeros(u.shape[0], 1, dtype=torch.long, device=u.device), xyz], dim=1).to(torch.int32)
