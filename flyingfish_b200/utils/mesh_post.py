"""Host-side mesh post-processing of the image-to-3D pipeline: drop small components, normalise, simplify, close holes.

The reference does these on the host too (src/sparse.rs ``filter_components`` :29-141, ``normalize`` :144-156,
``simplify`` :159-173 with the decimator behind it, ``fill_holes`` :175-270). Component labelling runs as one sparse
connected-components call over the face adjacency, the simplifier is the native quadric-error decimator of
``native/mesh_simplify.cpp``, hole filling walks the boundary loops."""
from __future__ import annotations

import ctypes

import numpy as np
import torch


def _check(vertices: torch.Tensor, faces: torch.Tensor) -> tuple[np.ndarray, np.ndarray]:
    v = vertices.detach().float().cpu().numpy().reshape(-1, 3)
    f = faces.detach().cpu().numpy().astype(np.int64).reshape(-1, 3)
    if v.shape[0] == 0 or f.shape[0] == 0 or not np.isfinite(v).all() or f.min() < 0 or f.max() >= v.shape[0]:
        raise ValueError("invalid mesh buffers")
    return v, f


def _compact(v: np.ndarray, f: np.ndarray, keep_faces: np.ndarray) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    sel = f[keep_faces]
    used = np.unique(sel)
    remap = np.full(v.shape[0], -1, dtype=np.int64)
    remap[used] = np.arange(used.shape[0])
    return (torch.from_numpy(v[used].astype(np.float32)), torch.from_numpy(remap[sel].astype(np.int32)),
            torch.from_numpy(np.nonzero(keep_faces)[0]), torch.from_numpy(used))


def filter_components(vertices: torch.Tensor, faces: torch.Tensor, minimum_face_ratio: float):
    """Keeps the largest face component and every component holding at least ``minimum_face_ratio`` of the faces. Two
    faces are connected when they share an edge that exactly two faces use. Returns (vertices, faces, kept face ids,
    kept vertex ids) with the ids indexing the input."""
    from scipy.sparse import coo_matrix
    from scipy.sparse.csgraph import connected_components
    v, f = _check(vertices, faces)
    if not (0.0 <= minimum_face_ratio <= 1.0):
        raise ValueError("invalid component face ratio")
    if (v == v[0]).all():
        raise ValueError("mesh must have non-zero extent")
    m = f.shape[0]
    a, b = f[:, [0, 1, 2]].reshape(-1), f[:, [1, 2, 0]].reshape(-1)
    key = np.minimum(a, b) * v.shape[0] + np.maximum(a, b)
    face = np.repeat(np.arange(m), 3)
    order = np.argsort(key, kind="stable")
    key, face = key[order], face[order]
    start = np.flatnonzero(np.r_[True, key[1:] != key[:-1]])
    size = np.diff(np.r_[start, key.shape[0]])
    pair = start[size == 2]
    fa, fb = face[pair], face[pair + 1]
    ok = fa != fb
    graph = coo_matrix((np.ones(int(ok.sum())), (fa[ok], fb[ok])), shape=(m, m))
    count, label = connected_components(graph, directed=False)
    sizes = np.bincount(label, minlength=count)
    # ties for the largest go to the component met first in edge order (isolated faces after all edges)
    first = np.full(count, key.shape[0] + m, dtype=np.int64)
    np.minimum.at(first, label[fa[ok]], pair[ok])
    np.minimum.at(first, label[fb[ok]], pair[ok])
    np.minimum.at(first, label, key.shape[0] + np.arange(m))
    largest = max(range(count), key=lambda c: (sizes[c], -first[c]))
    keep = (label == largest) | (sizes[label] / float(m) >= minimum_face_ratio)
    return _compact(v, f, keep)


def normalize(vertices: torch.Tensor) -> torch.Tensor:
    """Centres the vertices on their mean and scales the farthest one to radius 1 (FP64 arithmetic, FP32 result)."""
    v = vertices.detach().double().cpu().reshape(-1, 3)
    if v.shape[0] == 0 or not torch.isfinite(v).all():
        raise ValueError("invalid mesh buffers")
    v = v - v.mean(dim=0, keepdim=True)
    r = v.norm(dim=1).max()
    if not r > 0:
        raise ValueError("mesh must have non-zero extent")
    return (v / r).float()


def simplify(vertices: torch.Tensor, faces: torch.Tensor, target_faces: int):
    """Quadric-error edge collapses until at most ``target_faces`` faces remain (or no collapse is allowed any more).
    Returns (vertices, faces, face ancestry, vertex ancestry): for every output face / vertex the input face / vertex it
    descends from."""
    from ..ops import lib as oplib
    v, f = _check(vertices, faces)
    if target_faces <= 0:
        raise ValueError("simplification target must be positive")
    n, m = v.shape[0], f.shape[0]
    if m <= target_faces:
        return (torch.from_numpy(v.copy()), torch.from_numpy(f.astype(np.int32)), torch.arange(m), torch.arange(n))
    vin = np.ascontiguousarray(v, dtype=np.float32)
    fin = np.ascontiguousarray(f, dtype=np.int32)
    ov, of = np.zeros((n, 3), np.float32), np.zeros((m, 3), np.int32)
    fmap, vmap, counts = np.zeros(m, np.int32), np.zeros(n, np.int32), np.zeros(3, np.int32)
    p = lambda arr: arr.ctypes.data_as(ctypes.c_void_p)
    rc = oplib.host().ff_mesh_simplify(p(vin), n, p(fin), m, int(target_faces), p(ov), p(of), p(fmap), p(vmap), p(counts))
    if rc != 0:
        raise ValueError("mesh simplification refused its input")
    nv, nf = int(counts[0]), int(counts[1])
    return (torch.from_numpy(ov[:nv].copy()), torch.from_numpy(of[:nf].copy()), torch.from_numpy(fmap[:nf].astype(np.int64)),
            torch.from_numpy(vmap[:nv].astype(np.int64)))


def boundary_loops(faces: torch.Tensor) -> list[list[int]]:
    """Closed loops of boundary edges (directed edges whose reverse no face has), each as a vertex cycle in the
    direction opposite to the faces' winding along it (so that a fan over the loop continues the surface's orientation)."""
    f = faces.detach().cpu().numpy().astype(np.int64).reshape(-1, 3)
    directed = {(int(a), int(b)) for t in f for a, b in ((t[0], t[1]), (t[1], t[2]), (t[2], t[0]))}
    nxt: dict[int, list[int]] = {}
    for a, b in directed:
        if (b, a) not in directed:
            nxt.setdefault(b, []).append(a)                          # walk against the winding
    loops, used = [], set()
    for start in sorted(nxt):
        for first in nxt[start]:
            if (start, first) in used:
                continue
            loop, cur, prev = [start], first, start
            used.add((start, first))
            ok = True
            while cur != start:
                loop.append(cur)
                cand = [c for c in nxt.get(cur, []) if (cur, c) not in used]
                if not cand:
                    ok = False
                    break
                prev, cur = cur, cand[0]
                used.add((prev, cur))
            if ok and len(loop) >= 3:
                loops.append(loop)
    return loops


def fill_holes(vertices: torch.Tensor, faces: torch.Tensor, capacity: int) -> tuple[torch.Tensor, int]:
    """Closes every boundary loop of at most ``capacity`` edges with a triangle fan from the loop's first vertex.
    Returns (faces with the new triangles appended, number of loops closed)."""
    _check(vertices, faces)
    if capacity < 3:
        raise ValueError("hole capacity below a triangle")
    new, closed = [], 0
    for loop in boundary_loops(faces):
        if len(loop) > capacity:
            continue
        for i in range(1, len(loop) - 1):
            new.append([loop[0], loop[i], loop[i + 1]])
        closed += 1
    if not new:
        return faces.to(torch.int32), 0
    return torch.cat([faces.to(torch.int32).cpu(), torch.tensor(new, dtype=torch.int32)], dim=0), closed


def finish_mesh(vertices: torch.Tensor, faces: torch.Tensor, minimum_face_ratio: float = 0.0, hole_capacity: int = 0,
                target_faces: int = 0, unit_ball: bool = False) -> tuple[torch.Tensor, torch.Tensor, dict]:
    """The tail of the image-to-3D pipeline on an extracted mesh, each stage optional: drop small components, close
    small holes, simplify to a face budget, normalise into the unit ball. Returns (vertices, faces, what each stage did)."""
    report: dict = {"input": {"vertices": int(vertices.shape[0]), "faces": int(faces.shape[0])}}
    v, f = vertices.detach().float().cpu(), faces.detach().to(torch.int32).cpu()
    if f.shape[0] == 0:
        raise ValueError("the extracted surface has no faces")
    if minimum_face_ratio > 0.0:
        v, f, kept_faces, _ = filter_components(v, f, minimum_face_ratio)
        report["components"] = {"faces_kept": int(kept_faces.shape[0])}
    if hole_capacity >= 3:
        f, closed = fill_holes(v, f, hole_capacity)
        report["holes"] = {"closed": closed}
    if target_faces > 0:
        v, f, _, _ = simplify(v, f, target_faces)
        report["simplify"] = {"faces": int(f.shape[0])}
    if unit_ball:
        v = normalize(v)
    report["output"] = {"vertices": int(v.shape[0]), "faces": int(f.shape[0])}
    return v, f, report
