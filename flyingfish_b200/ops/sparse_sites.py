"""Coordinate bookkeeping of sparse voxel cascades: unique sites, shared cube corners, parent / child grids, rescaling.

Sites are rows ``(batch, x, y, z)`` of an int32 tensor. The reference keeps them in host vectors with a sorted index
(src/sparse.rs ``SparseSites``: ``deduplicate`` :1352, ``cube_corners`` :1303, ``downsample`` :1504, ``subdivide`` :1555,
``scaled_coordinates`` / ``round_unique`` :1606-1655); here every helper is a few whole-tensor operations on the
coordinates' device (lexicographic keys, ``unique`` with inverse indices, prefix sums), so a cascade stage never leaves the
GPU between its network passes."""
from __future__ import annotations

import torch

_BITS = 20                                    # per spatial axis in a key; batch takes the rest


def _keys(coords: torch.Tensor) -> torch.Tensor:
    c = coords.long()
    if coords.dim() != 2 or coords.shape[1] != 4 or coords.shape[0] == 0:
        raise ValueError("sparse sites are [n, 4] (batch, x, y, z) with n > 0")
    if bool((c < 0).any()) or bool((c[:, 1:] >= (1 << _BITS)).any()):
        raise ValueError("sparse coordinate negative or beyond the key range")
    return ((c[:, 0] << (3 * _BITS)) | (c[:, 1] << (2 * _BITS)) | (c[:, 2] << _BITS) | c[:, 3])


def _from_keys(keys: torch.Tensor) -> torch.Tensor:
    m = (1 << _BITS) - 1
    return torch.stack([keys >> (3 * _BITS), (keys >> (2 * _BITS)) & m, (keys >> _BITS) & m, keys & m], dim=1).to(torch.int32)


def check_sites(coords: torch.Tensor) -> None:
    """Sites must be non-negative, unique, and ordered by batch (rows of one sample contiguous)."""
    k = _keys(coords)
    if bool((coords[1:, 0] < coords[:-1, 0]).any()):
        raise ValueError("sparse sample rows must be contiguous and batch ordered")
    if torch.unique(k).numel() != k.numel():
        raise ValueError("duplicate sparse coordinate")


def deduplicate(coords: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """-> (unique sites in lexicographic order, index of every input row among them)."""
    uniq, inverse = torch.unique(_keys(coords), sorted=True, return_inverse=True)
    return _from_keys(uniq), inverse.to(torch.int32)


def cube_corners(coords: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """The corner lattice the cubes share. Returns (corner sites [c, 4], cubes [n, 8] corner ids with x = bit 0,
    contributor offsets [c + 1], contributors [8 n]): ``contributors[offsets[k]:offsets[k + 1]]`` are the flattened
    ``cube * 8 + corner`` slots that touch corner k, in increasing order."""
    check_sites(coords)
    n = coords.shape[0]
    bits = torch.arange(8, device=coords.device)
    delta = torch.stack([torch.zeros_like(bits), bits & 1, (bits >> 1) & 1, (bits >> 2) & 1], dim=1).to(torch.int32)
    expanded = (coords[:, None, :].to(torch.int32) + delta[None]).reshape(n * 8, 4)
    corners, inverse = deduplicate(expanded)
    counts = torch.bincount(inverse.long(), minlength=corners.shape[0])
    offsets = torch.cat([torch.zeros(1, dtype=torch.long, device=coords.device), torch.cumsum(counts, 0)])
    contributors = torch.sort(inverse.long(), stable=True).indices.to(torch.int32)
    return corners, inverse.reshape(n, 8), offsets, contributors


def downsample(coords: torch.Tensor, factor: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Parent grid: coordinates divided by ``factor``. -> (unique parents in lexicographic order, parent row of every site)."""
    if factor <= 0:
        raise ValueError("invalid sparse downsample factor")
    parents = coords.clone().to(torch.int32)
    parents[:, 1:] = torch.div(parents[:, 1:], factor, rounding_mode="floor")
    return deduplicate(parents)


def subdivide(coords: torch.Tensor, active: torch.Tensor, capacity: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Children of the sites: ``active`` [n, 8] bool picks which of the 8 children (child c sits at offset
    (c & 1, c >> 1 & 1, c >> 2 & 1)) exist on the twice finer grid. -> (child sites [m, 4] parent-major,
    source [m, 2] = (parent row, child index))."""
    check_sites(coords)
    if active.shape != (coords.shape[0], 8):
        raise ValueError("subdivision mask / site count mismatch")
    rows, child = torch.nonzero(active.bool(), as_tuple=True)
    if rows.numel() == 0 or rows.numel() > capacity:
        raise ValueError("subdivision exceeds capacity or has no active child")
    out = coords[rows].clone().to(torch.int32)
    for axis in range(3):
        out[:, axis + 1] = out[:, axis + 1] * 2 + ((child >> axis) & 1).to(torch.int32)
    return out, torch.stack([rows, child], dim=1).to(torch.int32)


def scaled_coordinates(coords: torch.Tensor, source_grid: int, target_grid: int) -> torch.Tensor:
    """Voxel centres of a ``source_grid`` lattice in the continuous coordinates of a ``target_grid`` lattice:
    ``(x + 0.5) / source_grid * (target_grid - 1)`` as FP32 [n, 3]."""
    if source_grid <= 0 or target_grid <= 1:
        raise ValueError("invalid cascade grids")
    xyz = coords[:, 1:]
    if bool(((xyz < 0) | (xyz >= source_grid)).any()):
        raise ValueError("cascade coordinate outside source grid")
    return ((xyz.float() + 0.5) / float(source_grid)) * float(target_grid - 1)


def round_unique(coords: torch.Tensor, source_grid: int, target_grid: int) -> torch.Tensor:
    """Sites re-quantised onto another grid (ties to even), duplicates merged, lexicographic order."""
    scaled = torch.round(scaled_coordinates(coords, source_grid, target_grid)).to(torch.int32)
    return deduplicate(torch.cat([coords[:, :1].to(torch.int32), scaled], dim=1))[0]


def morton_keys(coords: torch.Tensor, swap_xy: bool = False) -> torch.Tensor:
    """Z-order keys [n] int64: the bits of (x, y, z) -- or (y, x, z) -- interleaved with the first axis most significant
    inside every triple, the batch index above them."""
    c = coords.long()
    top = int(c[:, 1:].max())
    depth = max(top.bit_length(), 0)
    batches = int(c[:, 0].max()) + 1
    if depth > 16 or 3 * depth + batches.bit_length() > 63:
        raise ValueError("serialized coordinate or batch exceeds Morton capacity")
    axes = [c[:, 2], c[:, 1], c[:, 3]] if swap_xy else [c[:, 1], c[:, 2], c[:, 3]]
    key = c[:, 0] << (3 * depth)
    for bit in range(depth):
        for axis, value in enumerate(axes):
            key = key | (((value >> bit) & 1) << (3 * bit + 2 - axis))
    return key


def serialized_windows(coords: torch.Tensor, window: int) -> dict[str, torch.Tensor | list[torch.Tensor]]:
    """Orders for windowed attention over sparse sites (src/sparse.rs:1411-1502 of the reference): two space-filling
    orders (z-order over x y z and over y x z) with their inverse permutations, and a padding plan that makes every
    sample's row count a multiple of ``window`` by repeating rows of its last full window: ``pad`` lists the source row
    of every padded slot, ``unpad`` the slot of every real row, ``offsets`` the window boundaries (cumulative)."""
    check_sites(coords)
    if window <= 0:
        raise ValueError("invalid serialized window size")
    n = coords.shape[0]
    keys = [morton_keys(coords, False), morton_keys(coords, True)]
    order = [torch.sort(k, stable=True).indices for k in keys]
    inverse = []
    for o in order:
        inv = torch.empty_like(o)
        inv[o] = torch.arange(n, device=o.device)
        inverse.append(inv)
    counts = torch.bincount(coords[:, 0].long()).tolist()
    pad, unpad, offsets, first = [], [], [0], 0
    for count in counts:
        if count == 0:
            continue
        padded = -(-count // window) * window if count > window else count
        base = len(pad)
        unpad += list(range(base, base + count))
        pad += list(range(first, first + count))
        if padded > count:
            tail = count % window
            pad += list(range(first + count - window, first + count - tail))
        for start in range(base, base + padded, window):
            offsets.append(start + min(window, base + padded - start))
        first += count
    dev = coords.device
    as_t = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    return {"keys": keys, "order": [o.to(torch.int32) for o in order], "inverse": [i.to(torch.int32) for i in inverse],
            "pad": as_t(pad), "unpad": as_t(unpad), "offsets": as_t(offsets)}


def unit_ball_frame(coords: torch.Tensor) -> torch.Tensor:
    """4 x 4 affine frame (FP32) that moves the sites' centroid to the origin and the farthest site to radius 1
    (src/sparse.rs:1265-1301 of the reference); the sites must belong to one sample."""
    if bool((coords[:, 0] != coords[0, 0]).any()):
        raise ValueError("unit-ball frame requires one sample")
    xyz = coords[:, 1:].long()
    center = xyz.sum(dim=0).float() * (1.0 / float(coords.shape[0]))
    d = xyz.float() - center
    radius = float(torch.sqrt((d[:, 0] * d[:, 0] + d[:, 2] * d[:, 2]) + d[:, 1] * d[:, 1]).max()) + 1e-8
    if not (radius > 0.0 and radius < float("inf")):
        raise ValueError("invalid unit-ball radius")
    frame = torch.zeros(4, 4)
    for a in range(3):
        frame[a, a] = 1.0 / radius
        frame[a, 3] = -float(center[a]) / radius
    frame[3, 3] = 1.0
    return frame
