"""Layout, blending and sampling operators around the media and 3-D decoders (kernels/vision_ops.cu of the reference:
``sinusoidal_embed_f32``, ``pcd_pos_embed_f32``, ``pixel_shuffle_3d_f16``, ``unpatchify_bf16``, ``frame_blend_bf16``,
``tile_stitch_*``, ``gaussian_posterior_*``, ``perspective_focal_f32``, ``project_bilinear_*``).

The reference has one flat-index kernel per operator. Here each is a handful of whole-tensor operations on the input's
device (reshapes and permutes for the layout operators, gathers for the sampling ones), with the arithmetic of the
blends and the posterior in the reference's order of rounding."""
from __future__ import annotations

import math

import torch


def sinusoidal_embed(t: torch.Tensor, freqs: torch.Tensor, two_pi: bool = False) -> torch.Tensor:
    """t [b], freqs [half] -> [b, 2 half] = (cos(t f), sin(t f)), the argument scaled by 2 pi when ``two_pi``."""
    arg = t.float()[:, None] * freqs.float()[None, :]
    if two_pi:
        arg = (arg * 2.0) * math.pi
    return torch.cat([torch.cos(arg), torch.sin(arg)], dim=1)


def point_position_embed(points: torch.Tensor, freqs: torch.Tensor, channels: int, version: int = 2) -> torch.Tensor:
    """points [n, 3], freqs [f] -> [n, channels]: per axis ``sin(x f pi k)`` then ``cos(...)`` (k = 2 for version 1, 1 for
    version 2), the three axes one after the other, zero in the remaining channels."""
    f = freqs.numel()
    if version not in (1, 2) or 6 * f > channels:
        raise ValueError("point embedding: version 1 or 2, 6 * frequencies <= channels")
    ang = points.float()[:, :, None] * freqs.float()[None, None, :]
    ang = (ang * 2.0) * math.pi if version == 1 else ang * math.pi
    emb = torch.cat([torch.sin(ang), torch.cos(ang)], dim=2).reshape(points.shape[0], 6 * f)
    return torch.nn.functional.pad(emb, (0, channels - 6 * f))


def pixel_shuffle_3d(x: torch.Tensor, side: int) -> torch.Tensor:
    """x [side^3, channels * 8] (voxels z-major, the 8 children of a voxel innermost as z y x bits) ->
    [(2 side)^3, channels]: every voxel becomes its 2 x 2 x 2 children."""
    c8 = x.shape[1]
    if x.shape[0] != side ** 3 or c8 % 8:
        raise ValueError("pixel_shuffle_3d: [side^3, 8 c]")
    c = c8 // 8
    y = x.reshape(side, side, side, c, 2, 2, 2).permute(0, 4, 1, 5, 2, 6, 3)          # z dz y dy x dx c
    return y.reshape((2 * side) ** 3, c)


def unpatchify(rows: torch.Tensor, frames: int, height: int, width: int, channels: int, pt: int, p: int) -> torch.Tensor:
    """Token rows [frames * height * width, channels * pt * p * p] -> pixels [channels, frames * pt, height * p, width * p]."""
    if rows.shape != (frames * height * width, channels * pt * p * p):
        raise ValueError("unpatchify: row extent")
    x = rows.reshape(frames, height, width, channels, pt, p, p).permute(3, 0, 4, 1, 5, 2, 6)
    return x.reshape(channels, frames * pt, height * p, width * p)


def _blend(a: torch.Tensor, b: torch.Tensor, position: torch.Tensor, extent) -> torch.Tensor:
    """a (1 - w) + b w with w = position / extent, every operation rounded in FP32."""
    w = position.float() * (1.0 / torch.as_tensor(extent, dtype=torch.float32, device=position.device))
    return a.float() * (1.0 - w) + b.float() * w


def frame_blend(a: torch.Tensor, b: torch.Tensor, extent: int, a_first: int, b_first: int) -> torch.Tensor:
    """Cross-fade of ``extent`` frames: frame k of the result goes linearly from ``a[:, a_first + k]`` (k = 0) towards
    ``b[:, b_first + k]``; a, b are [channels, frames, ...]."""
    if extent <= 0 or a_first + extent > a.shape[1] or b_first + extent > b.shape[1]:
        raise ValueError("frame_blend: window outside the clips")
    k = torch.arange(extent, device=a.device).reshape(1, extent, *([1] * (a.dim() - 2)))
    return _blend(a[:, a_first:a_first + extent], b[:, b_first:b_first + extent], k, extent).to(a.dtype)


def tile_stitch(tiles: torch.Tensor, row_start: list[int], row_overlap: list[int], col_start: list[int], col_overlap: list[int],
                canvas_h: int, canvas_w: int) -> torch.Tensor:
    """Raw tiles [rows * cols, planes, tile_h, tile_w] -> canvas [planes, canvas_h, canvas_w]. A canvas pixel belongs to
    the last tile that starts at or before it; within the first ``overlap`` rows (columns) of a tile it is blended
    linearly with the raw tile above (then with the raw tile to the left)."""
    rows, cols = len(row_start), len(col_start)
    n, planes, th, tw = tiles.shape
    if n != rows * cols or len(row_overlap) != rows - 1 or len(col_overlap) != cols - 1:
        raise ValueError("tile_stitch: grid extents")
    dev = tiles.device
    Y, X = torch.arange(canvas_h, device=dev), torch.arange(canvas_w, device=dev)
    rs, cs = torch.tensor(row_start, device=dev), torch.tensor(col_start, device=dev)
    r = (torch.bucketize(Y, rs, right=True) - 1).clamp(min=0)
    c = (torch.bucketize(X, cs, right=True) - 1).clamp(min=0)
    y, x = Y - rs[r], X - cs[c]
    if bool((y >= th).any()) or bool((x >= tw).any()):
        raise ValueError("tile_stitch: the tiles do not cover the canvas")
    ro = torch.tensor([0] + list(row_overlap), device=dev)[r]            # overlap with the tile above (0 for the first row)
    co = torch.tensor([0] + list(col_overlap), device=dev)[c]
    t = tiles.float()
    tile = (r[:, None] * cols + c[None, :])                               # [H, W]
    yy, xx = y[:, None].expand(canvas_h, canvas_w), x[None, :].expand(canvas_h, canvas_w)
    v = t[tile, :, yy, xx]                                                # [H, W, planes]
    up = (r[:, None] > 0) & (yy < ro[:, None])
    above = t[(tile - cols).clamp(min=0), :, (yy + th - ro[:, None]).clamp(max=th - 1), xx]
    v = torch.where(up[..., None], _blend(above, v, yy[..., None], ro[:, None, None].clamp(min=1)), v)
    left_ok = (c[None, :] > 0) & (xx < co[None, :])
    left = t[(tile - 1).clamp(min=0), :, yy, (xx + tw - co[None, :]).clamp(max=tw - 1)]
    v = torch.where(left_ok[..., None], _blend(left, v, xx[..., None], co[None, :, None].clamp(min=1)), v)
    return v.permute(2, 0, 1).to(tiles.dtype).contiguous()


def gaussian_posterior(moments: torch.Tensor, eps: torch.Tensor, latents_mean: torch.Tensor, latents_std: torch.Tensor,
                       crop: tuple[int, int] | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """moments [2 c, h, w] (mean, then log-variance), eps [c, h, w] -> (mean, std, latents) with
    std = exp(0.5 clamp(logvar, -30, 20)) and latents = (fp16(mean + std eps) - latents_mean[c]) / latents_std[c],
    optionally cropped to the top-left ``crop`` = (height, width)."""
    c = eps.shape[0]
    if moments.shape[0] != 2 * c or moments.shape[1:] != eps.shape[1:]:
        raise ValueError("gaussian_posterior: moments [2 c, ...], eps [c, ...]")
    mean = moments[:c].float()
    std = torch.exp(0.5 * moments[c:].float().clamp(-30.0, 20.0))
    sample = (mean + std * eps.float()).to(torch.float16).float()
    shape = (c,) + (1,) * (eps.dim() - 1)
    lat = (sample - latents_mean.float().reshape(shape)) / latents_std.float().reshape(shape)
    if crop is not None:
        lat = lat[:, : crop[0], : crop[1]].contiguous()
    return mean, std, lat


def perspective_focal(fov: float, resolution: float) -> float:
    """Focal length in pixels of a camera with vertical field of view ``fov`` (radians) rendering ``resolution`` pixels."""
    if not (0.0 < fov < math.pi) or not resolution > 0:
        raise ValueError("field of view in (0, pi), positive resolution")
    return 16.0 / math.tan(0.5 * fov) * resolution / 32.0


def project_bilinear(features: torch.Tensor, camera: torch.Tensor, grid_side: int, coordinates: torch.Tensor | None = None
                     ) -> torch.Tensor:
    """Samples an image feature map at the projections of grid points. ``features`` [height, width, channels];
    ``camera`` = 12 values of a row-major 3 x 4 world-to-camera matrix, the focal length in pixels, the mesh scale and the
    image resolution. Grid points are the ``grid_side^3`` lattice over [-1, 1]^3 (x-major) or the listed integer
    ``coordinates`` [n, 3]; a point (ix, iy, iz) sits at world (u(ix), -u(iz), u(iy)) / (2 scale). Bilinear sampling with
    border clamping (pixel centres at half-integers). Returns [n, channels]."""
    h, w, ch = features.shape
    cam = camera.float()
    if cam.numel() != 15 or grid_side < 2:
        raise ValueError("project_bilinear: 15 camera values, grid_side >= 2")
    dev = features.device
    if coordinates is None:
        idx = torch.arange(grid_side ** 3, device=dev)
        ijk = torch.stack([idx // (grid_side * grid_side), (idx // grid_side) % grid_side, idx % grid_side], dim=1)
    else:
        ijk = coordinates.to(dev).long()
        if bool(((ijk < 0) | (ijk >= grid_side)).any()):
            raise ValueError("grid coordinate outside the lattice")
    step = 2.0 / float(grid_side - 1)
    j = ijk.float()
    v = torch.where(ijk < grid_side // 2, j * step - 1.0, -(float(grid_side - 1) - j) * step + 1.0)
    u = (v / cam[13]) / 2.0
    a, b, d = u[:, 0], -u[:, 2], u[:, 1]
    m = cam[:12].reshape(3, 4).to(dev)
    xyz = [((a * m[r, 0] + b * m[r, 1]) + d * m[r, 2]) + m[r, 3] for r in range(3)]
    focal, res = cam[12], cam[14]
    denom = -xyz[2] + 1.0e-8

    def pixel(coord: torch.Tensor, size: int) -> torch.Tensor:
        projected = (focal * coord) / denom + res / 2.0
        normalized = ((projected + 0.5) / res) * 2.0 - 1.0
        return ((((normalized + 1.0) * float(size)) - 1.0) / 2.0).clamp(0.0, float(size - 1))
    px, py = pixel(xyz[0], w), pixel(-xyz[1], h)
    x0, y0 = px.long(), py.long()
    x1, y1 = (x0 + 1).clamp(max=w - 1), (y0 + 1).clamp(max=h - 1)
    dx, dy = (px - x0.float())[:, None], (py - y0.float())[:, None]
    f = features.float()
    val = f[y0, x0] * ((1.0 - dx) * (1.0 - dy))
    val = val + f[y0, x1] * (dx * (1.0 - dy))
    val = val + f[y1, x0] * ((1.0 - dx) * dy)
    return val + f[y1, x1] * (dx * dy)


def adaptive_avg_pool2d(x: torch.Tensor, out_h: int, out_w: int) -> torch.Tensor:
    """Channels-last adaptive average pooling [h, w, c] -> [out_h, out_w, c]: output cell (y, x) averages rows
    ``floor(y h / out_h) .. ceil((y + 1) h / out_h)`` and the matching columns (the windows of PyTorch's operator)."""
    h, w, c = x.shape
    if out_h <= 0 or out_w <= 0:
        raise ValueError("adaptive pooling needs a positive output size")
    return torch.nn.functional.adaptive_avg_pool2d(x.float().permute(2, 0, 1)[None], (out_h, out_w))[0].permute(1, 2, 0).contiguous()


def axial_rotary_table(height: int, width: int, dim: int, theta: float = 10000.0) -> torch.Tensor:
    """[height * width, dim] table for :func:`rotary_spatial`: cos in the first half, sin in the second; the first
    quarter of the frequencies turns with the row index, the second with the column index."""
    if dim % 4:
        raise ValueError("axial rotary needs a head width that is a multiple of 4")
    q = dim // 4
    inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), torch.arange(q, dtype=torch.float32) / q)
    ys, xs = torch.meshgrid(torch.arange(height, dtype=torch.float32), torch.arange(width, dtype=torch.float32), indexing="ij")
    ang = torch.cat([ys.reshape(-1, 1) * inv[None], xs.reshape(-1, 1) * inv[None]], dim=1)          # [pixels, dim / 2]
    return torch.cat([torch.cos(ang), torch.sin(ang)], dim=1)


def rotary_spatial(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Split-half rotary embedding of channels-last activations: x [pixels, heads, dim] with a per-pixel table
    [pixels, dim] (cos | sin); pairs are (d, d + dim / 2)."""
    pixels, heads, dim = x.shape
    if dim % 4 or table.shape != (pixels, dim):
        raise ValueError("rotary_spatial: x [pixels, heads, dim], table [pixels, dim], dim a multiple of 4")
    half = dim // 2
    c, s = table[:, None, :half].float(), table[:, None, half:].float()
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)
