"""Image input processing: the reference's golden grid sizes, PNG data URLs, resampling and packing."""
import base64
import struct
import zlib

import numpy as np
import pytest

from flyingfish_b200.serve import image as im


def _png(w, h, rgba_rows, color=6):
    def chunk(t, b):
        return struct.pack(">I", len(b)) + t + b + struct.pack(">I", zlib.crc32(t + b))
    raw = b"".join(b"\x00" + bytes(r) for r in rgba_rows)
    return b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, color, 0, 0, 0)) + chunk(b"IDAT", zlib.compress(raw)) + chunk(b"IEND", b"")


def test_smart_resize_golden_grid():
    assert im.smart_resize(1024, 1024, 65536, 16777216) == (1024, 1024)
    assert im.smart_resize(1500, 900, 65536, 16777216) == (1504, 896)
    assert im.smart_resize(64, 64, 65536, 16777216) == (256, 256)
    assert im.smart_resize(80, 80, 1024, 16777216) == (64, 64)
    for bad in ((0, 32), (1, 201)):
        with pytest.raises(ValueError):
            im.smart_resize(*bad, 65536, 16777216)


def test_png_data_url_rgb_without_alpha_compositing_and_refusals():
    data = base64.b64encode(_png(2, 1, [[255, 0, 0, 0, 0, 128, 255, 255]])).decode()
    img = im.load_image(f"data:image/png;base64,{data}")
    assert (img.width, img.height) == (2, 1) and img.pixels.reshape(-1).tolist() == [255, 0, 0, 0, 128, 255]
    for bad in (f"data:image/jpeg;base64,{data}", "https://example.com/image.png", "file:///etc/passwd",
                "data:image/gif;base64,R0lGODlh"):
        with pytest.raises(ValueError):
            im.load_image(bad)


def test_resize_pack_and_token_expansion():
    rng = np.random.default_rng(0)
    img = im.Image(90, 70, rng.integers(0, 256, (70, 90, 3), dtype=np.uint8))
    flat = im.resize_bicubic(np.full((10, 10, 3), 77, dtype=np.uint8), 32, 64)
    assert np.allclose(flat, 77.0)                                   # normalised weights keep constants
    patches, grid = im.pack_patches(img, min_pixels=65536)
    assert grid[1] * grid[2] == patches.shape[0] and patches.shape[1] == 3 * 2 * 16 * 16
    n = im.image_token_count(grid)
    assert n == (grid[1] // 2) * (grid[2] // 2)
    assert im.expand_image_tokens([1, 9, 2, 9], 9, [n, 3]) == [1] + [9] * n + [2] + [9] * 3
    with pytest.raises(ValueError):
        im.expand_image_tokens([1, 9], 9, [])


# ---- JPEG, MiniCPM slicing, video frames --------------------------------------------------------------------------
def _jpeg_bytes(arr, mode="RGB", **kw):
    import io
    from PIL import Image as PI
    buf = io.BytesIO()
    PI.fromarray(arr, mode).save(buf, format="JPEG", **kw)
    return buf.getvalue()


def _pil_decode(data):
    import io
    from PIL import Image as PI
    return np.asarray(PI.open(io.BytesIO(data)).convert("RGB"))


def _smooth(h, w, seed=0):
    rng = np.random.default_rng(seed)
    yy, xx = np.mgrid[0:h, 0:w]
    base = np.stack([128 + 100 * np.sin(xx / 9.0 + c) * np.cos(yy / 13.0 - c) for c in range(3)], -1)
    return np.clip(base + rng.normal(0, 6, (h, w, 3)), 0, 255).astype(np.uint8)


@pytest.mark.parametrize("h,w,kw", [(64, 64, dict(quality=90, subsampling=0)), (37, 53, dict(quality=85, subsampling=2)),
                                    (48, 100, dict(quality=75, subsampling=1)), (33, 31, dict(quality=95, subsampling=2, optimize=True))])
def test_jpeg_decoder_matches_pillow(h, w, kw):
    pytest.importorskip("PIL")
    data = _jpeg_bytes(_smooth(h, w, seed=h), **kw)
    got = im.decode_jpeg(data)
    want = _pil_decode(data).astype(np.int32)
    assert (got.height, got.width) == (h, w)
    err = np.abs(got.pixels.astype(np.int32) - want)
    # same coefficients; the inverse DCT, chroma upsampling filter and colour rounding differ between decoders
    assert err.mean() < (1.5 if kw["subsampling"] == 0 else 3.0) and np.percentile(err, 99) <= 16


def test_jpeg_grayscale_restart_intervals_and_refusals():
    pytest.importorskip("PIL")
    gray = _smooth(40, 56)[:, :, 0]
    got = im.decode_jpeg(_jpeg_bytes(gray, "L", quality=90))
    assert np.abs(got.pixels[:, :, 0].astype(int) - _pil_decode(_jpeg_bytes(gray, "L", quality=90))[:, :, 0]).max() <= 2
    assert (got.pixels[:, :, 0] == got.pixels[:, :, 1]).all()
    rst = _jpeg_bytes(_smooth(64, 96), quality=80, subsampling=2, restart_marker_blocks=2)
    assert b"\xff\xdd" in rst
    assert np.abs(im.decode_jpeg(rst).pixels.astype(int) - _pil_decode(rst)).mean() < 3.0
    with pytest.raises(ValueError, match="unsupported"):
        im.decode_jpeg(_jpeg_bytes(_smooth(32, 32), progressive=True))
    with pytest.raises(ValueError, match="truncated|corrupt"):
        im.decode_jpeg(rst[: len(rst) // 3])
    with pytest.raises(ValueError, match="pixel limit"):
        im.decode_jpeg(rst, max_pixels=1000)
    with pytest.raises(ValueError):
        im.decode_image(b"GIF89a....")
    url = "data:image/jpeg;base64," + base64.b64encode(rst).decode()
    assert im.load_image(url).width == 96
    with pytest.raises(ValueError, match="does not match"):
        im.load_image("data:image/png;base64," + base64.b64encode(rst).decode())


def test_minicpm_slicing_grids():
    # a 720p frame with one slice allowed is shown whole: 448-pixel budget, multiples of 4 patches (patch 14)
    plan = im.slice_plan(720, 1280, patch=14, max_slices=1)
    assert (plan.rows, plan.cols) == (0, 0) and plan.source == (336, 616) and plan.grids(14) == [(1, 24, 44)]
    # nine slices allowed: 1280x720 has 4.6 budget areas -> 5 +- 1 slices, the factorisation closest to 16:9 in log space
    plan = im.slice_plan(720, 1280, patch=14, max_slices=9)
    assert (plan.rows, plan.cols) == (2, 3) and plan.tile[0] % 56 == 0 and plan.tile[1] % 56 == 0
    assert plan.refine == (plan.tile[0] * 2, plan.tile[1] * 3) and len(plan.grids(14)) == 7
    assert im.slice_grid(448, 448, 9) is None and im.slice_grid(2000, 500, 9) == (4, 1) or im.slice_grid(2000, 500, 9)[1] == 1
    img = im.Image(1280, 720, _smooth(720, 1280))
    packed, plan2 = im.pack_slices(img)
    assert plan2 == plan and len(packed) == 7
    assert packed[0].shape == ((plan.source[0] // 14) * (plan.source[1] // 14), 3 * 14 * 14)
    assert packed[1].shape == ((plan.tile[0] // 14) * (plan.tile[1] // 14), 588) and abs(float(packed[1].mean())) < 1.0
    assert im.slice_token_count(plan) == 7 * 66 + 1


def test_video_frame_sampling_rule():
    V = im.VideoMeta
    assert im.sample_frame_indices(V(60, 30.0, 2.0), 8) == [0, 30] == im.sample_frame_indices(V(60, 30.0, 2.0), 128)
    assert im.sample_frame_indices(V(600, 30.0, 20.0), 8) == [0, 84, 168, 255, 339, 426, 510, 597]
    assert im.sample_frame_indices(V(30, 30.0, 1.0), 8) == [0] == im.sample_frame_indices(V(12, 30.0, 0.4), 8)
    capped = im.sample_frame_indices(V(3900, 30.0, 130.0), 128)
    assert len(capped) == 128 and capped[:3] == [0, 30, 60] and capped[125:] == [3834, 3864, 3897]
    assert im.sample_frame_indices(V(216, 24.0, 9.0), 8) == [0, 28, 60, 91, 120, 151, 182, 213]
    assert im.sample_frame_indices(V(240, 24.0, 10.0), 8) == [0, 33, 67, 100, 134, 168, 201, 237]
    exact = im.sample_frame_indices(V(3840, 30.0, 128.0), 128)
    assert len(exact) == 128 and exact[:2] == [0, 30] and exact[126:] == [3780, 3810]
    end = im.sample_frame_indices(V(12210, 30.0, 407.0), 128)
    assert end[:4] == [0, 96, 192, 288] and end[124:] == [11916, 12012, 12108, 12207]
    with pytest.raises(ValueError):
        im.sample_frame_indices(V(10, 30.0, 2.0), 8)
    frames = [im.Image(96, 64, _smooth(64, 96, seed=i)) for i in range(3)]
    patches, grid = im.pack_video_frames(frames, min_pixels=1024)
    assert grid[0] == 2 and patches.shape == (2 * grid[1] * grid[2], 3 * 2 * 16 * 16)
