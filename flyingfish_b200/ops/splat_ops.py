"""Gaussian-splat parameters from decoder features, and their PLY form.

A splat decoder emits, per anchor point, a feature row holding ``g`` Gaussians' raw parameters in blocks
``[offset 3g | colour 3g | scale 3g | rotation 4g | opacity g | offset scale g]``. The head turns them into world-space
Gaussians (src/backend/cuda/engine_vision.rs ``to_representation`` of the reference, which loops over anchors on the host):

* position = anchor + tanh(raw * lr + perturbation) * perturbe_size / 2 * softplus(offset scale + base) - 0.5
* scale = sqrt(softplus(raw * lr + inverse-softplus(scaling_bias))^2 + filter_kernel^2)
* rotation = normalise(raw * lr + (1, 0, 0, 0)); opacity = sigmoid(raw * lr + logit(opacity_bias)); colour = raw * lr

Here the head is whole-array arithmetic on the features' device. The PLY rows (17 floats: position with y and z swapped
and z negated, three zero normals, colour, opacity as a logit, log scales, rotation pre-multiplied by the quarter turn
about x that matches the axis swap) follow the usual splat-viewer layout."""
from __future__ import annotations

import math
from dataclasses import dataclass
from pathlib import Path

import torch


@dataclass(frozen=True)
class SplatConfig:
    per_anchor: int = 32
    lr_xyz: float = 1.0
    lr_features_dc: float = 1.0
    lr_scaling: float = 1.0
    lr_rotation: float = 1.0
    lr_opacity: float = 1.0
    perturbe_size: float = 1.0
    filter_kernel_size: float = 0.0
    scaling_bias: float = 0.01
    opacity_bias: float = 0.1

    @property
    def feature_width(self) -> int:
        return 15 * self.per_anchor

    def check(self) -> None:
        if self.per_anchor <= 0 or not (0.0 < self.opacity_bias < 1.0) or self.scaling_bias <= 0.0 or self.filter_kernel_size < 0.0:
            raise ValueError("invalid splat representation settings")


@dataclass
class Splats:
    xyz: torch.Tensor           # [n, 3]
    features_dc: torch.Tensor   # [n, 3]
    scaling: torch.Tensor       # [n, 3]
    rotation: torch.Tensor      # [n, 4] unit quaternions (w, x, y, z)
    opacity: torch.Tensor       # [n]


def _softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 20.0, x, torch.log1p(torch.exp(x.clamp(max=20.0))))


def splat_parameters(points: torch.Tensor, features: torch.Tensor, offset_perturbation: torch.Tensor, base_offset_scale: float,
                     cfg: SplatConfig) -> Splats:
    """points [a, 3], features [a, 15 g], offset_perturbation [g, 3] -> ``a * g`` Gaussians (anchor-major)."""
    cfg.check()
    a, g = points.shape[0], cfg.per_anchor
    if points.shape != (a, 3) or features.shape != (a, cfg.feature_width) or offset_perturbation.shape != (g, 3):
        raise ValueError("splat head: points [a, 3], features [a, 15 g], perturbation [g, 3]")
    f = features.float()
    if not (torch.isfinite(f).all() and torch.isfinite(points).all()):
        raise ValueError("non-finite splat input")
    p = points.float()
    blk = lambda lo, width: f[:, lo * g: lo * g + width * g].reshape(a, g, width)
    raw_off, raw_dc, raw_s, raw_r = blk(0, 3), blk(3, 3), blk(6, 3), f[:, 9 * g: 13 * g].reshape(a, g, 4)
    raw_op, raw_os = f[:, 13 * g: 14 * g], f[:, 14 * g: 15 * g]
    off_scale = _softplus(raw_os + base_offset_scale)                                   # [a, g]
    off = torch.tanh(raw_off * cfg.lr_xyz + offset_perturbation.to(f.device).float()[None]) * (0.5 * cfg.perturbe_size) * off_scale[..., None]
    xyz = (off + p[:, None, :]) - 0.5
    scaling_offset = cfg.scaling_bias + math.log(-math.expm1(-cfg.scaling_bias))         # softplus^-1(scaling_bias)
    sp = _softplus(raw_s * cfg.lr_scaling + scaling_offset)
    scaling = torch.sqrt(sp * sp + cfg.filter_kernel_size ** 2)
    rot = raw_r * cfg.lr_rotation
    rot = torch.cat([rot[..., :1] + 1.0, rot[..., 1:]], dim=-1)
    rot = rot / rot.norm(dim=-1, keepdim=True).clamp(min=1e-12)
    opacity = torch.sigmoid(raw_op * cfg.lr_opacity + math.log(cfg.opacity_bias / (1.0 - cfg.opacity_bias)))
    n = a * g
    return Splats(xyz.reshape(n, 3), (raw_dc * cfg.lr_features_dc).reshape(n, 3), scaling.reshape(n, 3), rot.reshape(n, 4),
                  opacity.reshape(n))


def splat_parameters_reference(points, features, offset_perturbation, base_offset_scale, cfg: SplatConfig) -> Splats:
    """Per-anchor, per-Gaussian restatement in scalar FP32."""
    g = cfg.per_anchor
    f32 = lambda v: torch.tensor(v, dtype=torch.float32)
    sp = lambda x: x if float(x) > 20.0 else torch.log1p(torch.exp(x))
    s_off = f32(cfg.scaling_bias + math.log(-math.expm1(-cfg.scaling_bias)))
    o_off = f32(math.log(cfg.opacity_bias / (1.0 - cfg.opacity_bias)))
    out = {k: [] for k in ("xyz", "dc", "s", "r", "o")}
    for a in range(points.shape[0]):
        row = features[a].float()
        for k in range(g):
            scale = sp(row[14 * g + k] + f32(base_offset_scale))
            raw = row[k * 3: k * 3 + 3] * cfg.lr_xyz + offset_perturbation[k].float()
            out["xyz"].append((torch.tanh(raw) * f32(0.5 * cfg.perturbe_size) * scale + points[a].float()) - 0.5)
            out["dc"].append(row[3 * g + k * 3: 3 * g + k * 3 + 3] * cfg.lr_features_dc)
            s = torch.stack([sp(v + s_off) for v in row[6 * g + k * 3: 6 * g + k * 3 + 3] * cfg.lr_scaling])
            out["s"].append(torch.sqrt(s * s + f32(cfg.filter_kernel_size ** 2)))
            r = row[9 * g + k * 4: 9 * g + k * 4 + 4] * cfg.lr_rotation + f32([1.0, 0, 0, 0])
            out["r"].append(r / max(float(r.norm()), 1e-12))
            out["o"].append(torch.sigmoid(row[13 * g + k] * cfg.lr_opacity + o_off))
    st = lambda k: torch.stack(out[k])
    return Splats(st("xyz"), st("dc"), st("s"), st("r"), st("o"))


def splat_ply_rows(s: Splats) -> torch.Tensor:
    """[n, 17] FP32 rows: x, -z, y, three zero normals, colour, logit(opacity), log scales, rotation turned with the
    axes (left-multiplied by the quaternion (sqrt 1/2, sqrt 1/2, 0, 0), computed in FP64)."""
    n = s.xyz.shape[0]
    op = s.opacity.float().clamp(1e-6, 1.0 - 1e-6)
    q = s.rotation.double()
    c = math.sqrt(0.5)
    w, x, y, z = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    rot = torch.stack([c * w - c * x, c * x + c * w, c * y - c * z, c * z + c * y], dim=1).float()
    xyz = s.xyz.float()
    return torch.cat([xyz[:, 0:1], -xyz[:, 2:3], xyz[:, 1:2], torch.zeros(n, 3, device=xyz.device), s.features_dc.float(),
                      torch.log(op / (1.0 - op))[:, None], torch.log(s.scaling.float().clamp(min=1e-6)), rot], dim=1)


SPLAT_PLY_PROPERTIES = ("x", "y", "z", "nx", "ny", "nz", "f_dc_0", "f_dc_1", "f_dc_2", "opacity", "scale_0", "scale_1", "scale_2",
                        "rot_0", "rot_1", "rot_2", "rot_3")


def write_splat_ply(target, s: Splats) -> None:
    """Binary little-endian PLY with the 17 float properties splat viewers read."""
    rows = splat_ply_rows(s).cpu().contiguous()
    header = f"ply\nformat binary_little_endian 1.0\nelement vertex {rows.shape[0]}\n" + \
        "".join(f"property float {p}\n" for p in SPLAT_PLY_PROPERTIES) + "end_header\n"
    data = header.encode() + rows.numpy().astype("<f4").tobytes()
    if hasattr(target, "write"):
        target.write(data)
    else:
        Path(target).write_bytes(data)
