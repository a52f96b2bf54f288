"""Gaussian-splat parameter head and its PLY rows."""
import io
import math

import numpy as np
import pytest
import torch

from flyingfish_b200.ops import splat_ops as so


def test_parameters_match_the_scalar_restatement():
    cfg = so.SplatConfig(per_anchor=4, lr_xyz=0.5, lr_features_dc=2.0, lr_scaling=0.7, lr_rotation=0.3, lr_opacity=1.5,
                         perturbe_size=0.02, filter_kernel_size=0.001, scaling_bias=0.004, opacity_bias=0.1)
    g = torch.Generator().manual_seed(0)
    points = torch.rand(6, 3, generator=g)
    feats = torch.randn(6, cfg.feature_width, generator=g) * 2.0
    feats[0, 14 * 4] = 30.0                                                   # large-argument branch of softplus
    pert = torch.randn(4, 3, generator=g) * 0.1
    got = so.splat_parameters(points, feats, pert, -1.0, cfg)
    want = so.splat_parameters_reference(points, feats, pert, -1.0, cfg)
    for name in ("xyz", "features_dc", "scaling", "rotation", "opacity"):
        a, b = getattr(got, name), getattr(want, name)
        assert a.shape == b.shape and torch.allclose(a, b, atol=1e-6, rtol=1e-5), name
    assert got.xyz.shape == (24, 3) and torch.allclose(got.rotation.norm(dim=1), torch.ones(24), atol=1e-6)
    assert (got.scaling >= cfg.filter_kernel_size).all() and ((got.opacity > 0) & (got.opacity < 1)).all()
    # zero features: every Gaussian sits at its anchor's offset pattern, identity rotation, bias opacity and bias scale
    zero = so.splat_parameters(points, torch.zeros_like(feats), torch.zeros(4, 3), 0.0, cfg)
    assert torch.allclose(zero.xyz.reshape(6, 4, 3), (points - 0.5)[:, None, :].expand(6, 4, 3), atol=1e-7)
    assert torch.allclose(zero.rotation, torch.tensor([1.0, 0, 0, 0]).expand(24, 4))
    assert torch.allclose(zero.opacity, torch.full((24,), cfg.opacity_bias), atol=1e-6)
    assert torch.allclose(zero.scaling, torch.full((24, 3), math.sqrt(cfg.scaling_bias ** 2 + cfg.filter_kernel_size ** 2)), atol=1e-6)
    with pytest.raises(ValueError):
        so.splat_parameters(points, feats[:, :-1], pert, 0.0, cfg)
    with pytest.raises(ValueError):
        so.splat_parameters(points, feats, pert, 0.0, so.SplatConfig(per_anchor=4, opacity_bias=1.0))


def test_ply_rows_and_file():
    s = so.Splats(xyz=torch.tensor([[1.0, 2.0, 3.0]]), features_dc=torch.tensor([[0.1, 0.2, 0.3]]), scaling=torch.tensor([[0.5, 1.0, 2.0]]),
                  rotation=torch.tensor([[1.0, 0.0, 0.0, 0.0]]), opacity=torch.tensor([0.25]))
    rows = so.splat_ply_rows(s)
    c = math.sqrt(0.5)
    want = [1.0, -3.0, 2.0, 0, 0, 0, 0.1, 0.2, 0.3, math.log(0.25 / 0.75), math.log(0.5), 0.0, math.log(2.0), c, c, 0.0, 0.0]
    assert rows.shape == (1, 17) and torch.allclose(rows[0], torch.tensor(want, dtype=torch.float32), atol=1e-6)
    # the turned rotation is still a unit quaternion, and opacity 0 / 1 stay finite
    g = torch.Generator().manual_seed(1)
    q = torch.randn(5, 4, generator=g)
    many = so.Splats(torch.randn(5, 3, generator=g), torch.randn(5, 3, generator=g), torch.rand(5, 3, generator=g) + 0.1,
                     q / q.norm(dim=1, keepdim=True), torch.tensor([0.0, 1.0, 0.5, 0.2, 0.9]))
    r = so.splat_ply_rows(many)
    assert torch.isfinite(r).all() and torch.allclose(r[:, 13:].norm(dim=1), torch.ones(5), atol=1e-5)
    buf = io.BytesIO()
    so.write_splat_ply(buf, many)
    data = buf.getvalue()
    head = data[: data.index(b"end_header\n") + 11].decode()
    assert head.startswith("ply\nformat binary_little_endian 1.0\nelement vertex 5\nproperty float x\n") and head.count("property float") == 17
    body = np.frombuffer(data[len(head):], dtype="<f4").reshape(5, 17)
    assert np.allclose(body, r.numpy())
